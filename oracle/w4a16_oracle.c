/*
 * TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT.
 *
 * CPU restatement (plain C, bit-level fp16 emulation) of the W4A16 path of
 * sparklesea/sparse-quant's `quant` extension (quantization/nvidia/kernel).  Only the
 * test-suite, the smoke check and the CPU-baseline leg of the benchmark may load this
 * library; the product (the CUDA library and its Python host side) never does.
 *
 * Every function cites the reference file:line it restates.  Paths are relative to the
 * reference project root.
 *
 * Parity pin: checked against (i) vectors produced by importing the reference's own
 * Python quantizer (test/nvidia/utils/quant_dequant_nvidia.py) on CPU and (ii) vectors
 * produced by the reference's own CUDA extension rebuilt for sm_100a and run on a B200
 * (both stored under tests/golden/ together with the generating script).
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include <math.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------ */
/* IEEE binary16 helpers (bit exact; no hardware fp16 needed)                            */
/* ------------------------------------------------------------------------------------ */

static inline double h2d(uint16_t h)
{
    const int s = h >> 15, e = (h >> 10) & 0x1f, m = h & 0x3ff;
    double v;
    if (e == 0)       v = ldexp((double)m, -24);                  /* zero / subnormal */
    else if (e == 31) v = m ? NAN : INFINITY;
    else              v = ldexp((double)(m | 0x400), e - 25);
    return s ? -v : v;
}

static inline float h2f(uint16_t h) { return (float)h2d(h); }

/* round-to-nearest-even conversion of a double to binary16 (subnormals kept) */
static inline uint16_t d2h(double d)
{
    uint64_t bits;
    memcpy(&bits, &d, 8);
    const uint16_t sign = (uint16_t)((bits >> 48) & 0x8000);
    if (isnan(d)) return sign | 0x7e00;
    double a = fabs(d);
    if (a == 0.0) return sign;
    if (isinf(a) || a >= 65520.0) return sign | 0x7c00;          /* overflow -> inf */
    int e;
    (void)frexp(a, &e);                                           /* a = f * 2^e, f in [0.5,1) */
    int ulp_exp = e - 11;                                         /* ulp of a normal binary16 with that exponent */
    if (ulp_exp < -24) ulp_exp = -24;                             /* subnormal range: fixed ulp 2^-24 */
    double q = ldexp(a, -ulp_exp);                                /* exact: power-of-two scaling */
    double r = nearbyint(q);                                      /* default rounding mode = nearest even */
    double v = ldexp(r, ulp_exp);
    /* re-encode v (exactly representable now, possibly bumped to the next binade) */
    if (v >= 65520.0) return sign | 0x7c00;
    if (v < ldexp(1.0, -14)) return sign | (uint16_t)ldexp(v, 24);
    (void)frexp(v, &e);
    const int be = e - 1 + 15;
    const uint16_t m = (uint16_t)(ldexp(v, 11 - e)) & 0x3ff;
    return sign | (uint16_t)(be << 10) | m;
}

static inline int h_is_subnormal(uint16_t h) { return ((h >> 10) & 0x1f) == 0 && (h & 0x3ff) != 0; }
static inline uint16_t h_ftz(uint16_t h) { return h_is_subnormal(h) ? (uint16_t)(h & 0x8000) : h; }

/* PTX add.f16 / __hadd : round-to-nearest-even, subnormals preserved */
static inline uint16_t h_add(uint16_t a, uint16_t b) { return d2h(h2d(a) + h2d(b)); }

/* PTX sub.ftz.f16 : subnormal inputs and results flushed to sign-preserving zero */
static inline uint16_t h_sub_ftz(uint16_t a, uint16_t b)
{
    return h_ftz(d2h(h2d(h_ftz(a)) - h2d(h_ftz(b))));
}

/* PTX mul.ftz.f16 */
static inline uint16_t h_mul_ftz(uint16_t a, uint16_t b)
{
    a = h_ftz(a); b = h_ftz(b);
    double p = h2d(a) * h2d(b);
    uint16_t r = d2h(p);
    if (p == 0.0) r = (uint16_t)((a ^ b) & 0x8000);               /* signed zero of a product */
    return h_ftz(r);
}

/* cvt.rn.f16.f32 */
static inline uint16_t f2h(float f) { return d2h((double)f); }

ORACLE_API uint16_t oracle_f2h(float f) { return f2h(f); }
ORACLE_API float    oracle_h2f(uint16_t h) { return h2f(h); }
ORACLE_API uint16_t oracle_hadd(uint16_t a, uint16_t b) { return h_add(a, b); }
ORACLE_API uint16_t oracle_hsub_ftz(uint16_t a, uint16_t b) { return h_sub_ftz(a, b); }
ORACLE_API uint16_t oracle_hmul_ftz(uint16_t a, uint16_t b) { return h_mul_ftz(a, b); }

/* ------------------------------------------------------------------------------------ */
/* Layout step 1: "ours" uint8 [N, K/2]  ->  AWQ uint32 [K, N/8]                          */
/* Restates convert_ours_to_awq_kernel, kernel/gemm_s4_f16/format.cu:151-189.            */
/* One destination word (k, n/8) gathers eight source bytes (rows 8*(n/8)+j, column k/2),*/
/* takes the high nibble for even k and the low nibble for odd k, and stores the eight   */
/* values in the nibble order 0,2,4,6,1,3,5,7 (bytes (v2<<4)+v0, (v6<<4)+v4, ...).        */
/* ------------------------------------------------------------------------------------ */
ORACLE_API void oracle_convert_ours_to_awq(const uint8_t* src, uint32_t* dst, int K, int N)
{
    const int dst_w = N / 8, src_w = K / 2;
    #pragma omp parallel for schedule(static)
    for (int k = 0; k < K; ++k) {
        for (int c = 0; c < dst_w; ++c) {
            uint32_t v[8];
            for (int j = 0; j < 8; ++j) {
                const uint8_t b = src[(size_t)(c * 8 + j) * src_w + k / 2];
                v[j] = (k & 1) ? (b & 0x0f) : (b >> 4);
            }
            const uint32_t b0 = (v[2] << 4) + v[0], b1 = (v[6] << 4) + v[4];
            const uint32_t b2 = (v[3] << 4) + v[1], b3 = (v[7] << 4) + v[5];
            dst[(size_t)k * dst_w + c] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* Layout step 2: AWQ uint32 [K, N/8] -> TurboMind tile order (nominal int32 [K, N/8])   */
/* Literal restatement of reformat_s4_k_m8 + permute_u4<0,5,9,8,3,1,6,4,2,7>,            */
/* kernel/gemm_s4_f16/format.cu:24-57,66-71: view the source nibbles as a 10-D tensor of  */
/* shape {K/32,2,2,4,2, N/32,2,2,2,4} (row-major, last dim fastest), permute the axes,    */
/* write nibble by nibble.                                                                */
/* ------------------------------------------------------------------------------------ */
ORACLE_API void oracle_convert_awq_to_lmdeploy(const uint32_t* src, uint32_t* dst, int K, int N)
{
    const int dims[10]  = {K / 32, 2, 2, 4, 2, N / 32, 2, 2, 2, 4};
    const int order[10] = {0, 5, 9, 8, 3, 1, 6, 4, 2, 7};
    const size_t count = (size_t)K * N;
    memset(dst, 0, count / 2);
    for (size_t i = 0; i < count; ++i) {
        int idx[10];
        size_t ii = i;
        for (int j = 9; j >= 0; --j) { idx[j] = (int)(ii % dims[j]); ii /= dims[j]; }
        const uint32_t data = (src[i / 8] >> ((i % 8) * 4)) & 0xf;
        size_t index = 0, stride = 1;
        for (int j = 9; j >= 0; --j) { index += (size_t)idx[order[j]] * stride; stride *= dims[order[j]]; }
        dst[index / 8] |= data << ((index % 8) * 4);
    }
}

/* ------------------------------------------------------------------------------------ */
/* Layout step 3: zeros, scales fp16 [N, K/g]  ->  half2 (zero+64, scale) [K/g, N]        */
/* Restates transpose_merge_zeros_scales_kernel, format.cu:206-224 (fp16 __hadd of 64).   */
/* ------------------------------------------------------------------------------------ */
ORACLE_API void oracle_transpose_merge_zeros_scales(const uint16_t* zeros, const uint16_t* scales,
                                                    uint16_t* zs, int K, int N, int g)
{
    const int width = K / g;
    const uint16_t h64 = 0x5400;
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < width; ++c) {
            const size_t i = (size_t)n * width + c, t = (size_t)c * N + n;
            zs[2 * t]     = h_add(zeros[i], h64);
            zs[2 * t + 1] = scales[i];
        }
}

/* ------------------------------------------------------------------------------------ */
/* Element addressing of the final `weight` buffer.  The physical order is                */
/* [K/32][N/32][lane 0..31][word 0..3] (cta_iterator.h:86-88, warp_iterator.h:44-84): a   */
/* lane's uint4 holds the mma.m16n8k16 A-fragments of the four 16x16 sub-blocks of a      */
/* 32(k) x 32(n) tile.  The closed form below is what the permutation of step 2 yields;   */
/* tests check it against the literal restatement above for every (n,k).                  */
/* ------------------------------------------------------------------------------------ */
static inline uint32_t packed_get(const uint32_t* qw, int N, int n, int k)
{
    const size_t tile = (size_t)(k / 32) * (N / 32) + (n / 32);
    const int lane = (n % 8) * 4 + (k % 8) / 2;
    const int word = ((k / 16) % 2) * 2 + ((n / 16) % 2);
    const int nib  = (k % 2) * 4 + ((k / 8) % 2) * 2 + ((n / 8) % 2);
    return (qw[(tile * 32 + lane) * 4 + word] >> (4 * nib)) & 0xf;
}

ORACLE_API void oracle_unpack(const uint32_t* qw, uint8_t* q /*[N,K]*/, int K, int N)
{
    #pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k)
            q[(size_t)n * K + k] = (uint8_t)packed_get(qw, N, n, k);
}

/* ------------------------------------------------------------------------------------ */
/* Dequantisation.  Restates dequantize_s4_to_fp16x2_v2 (common.h:114-153: nibble ->      */
/* fp16 bit pattern 0x5400|q<<4, i.e. exactly 64+q) followed by apply_Q (common.h:210-225 */
/* with TURBOMIND_S4_DEQUANT_USE_FMA=0: u = sub.ftz.f16(t, zero+64); w = mul.ftz.f16(u,   */
/* scale)).  Output fp16 bits, row-major [N, K] (the orientation of nn.Linear.weight).    */
/* ------------------------------------------------------------------------------------ */
ORACLE_API void oracle_dequant(const uint32_t* qw, const uint16_t* zs, uint16_t* w, int K, int N, int g)
{
    #pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k) {
            const uint32_t q = packed_get(qw, N, n, k);
            const uint16_t t = (uint16_t)(0x5400u | (q << 4));
            const size_t qi = (size_t)(k / g) * N + n;
            const uint16_t u = h_sub_ftz(t, zs[2 * qi]);
            w[(size_t)n * K + k] = h_mul_ftz(u, zs[2 * qi + 1]);
        }
}

/* same, to fp32 (for the CPU baseline: dequantise, then fp32 matmul) */
ORACLE_API void oracle_dequant_f32(const uint32_t* qw, const uint16_t* zs, float* w, int K, int N, int g)
{
    #pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k) {
            const uint32_t q = packed_get(qw, N, n, k);
            const uint16_t t = (uint16_t)(0x5400u | (q << 4));
            const size_t qi = (size_t)(k / g) * N + n;
            w[(size_t)n * K + k] = h2f(h_mul_ftz(h_sub_ftz(t, zs[2 * qi]), zs[2 * qi + 1]));
        }
}

/* ------------------------------------------------------------------------------------ */
/* GEMM numerics: fp16 x fp16 products accumulated in fp32 (mma.sync ...f32.f16.f16.f32,  */
/* gemm_template.h:29-47), one final fp32->fp16 round-to-nearest (gemm_template.h:298),   */
/* bias added afterwards in fp16 (test/nvidia/module/qlinear/qlinear.py:69-70).  The      */
/* reference leaves the summation order unspecified; this restatement sums k ascending.   */
/* x fp16 [M,K], w fp16 [N,K] (dequantised), bias fp16 [N] or NULL, out fp16 [M,N].        */
/* ------------------------------------------------------------------------------------ */
ORACLE_API void oracle_gemm_f16(const uint16_t* x, const uint16_t* w, const uint16_t* bias,
                                uint16_t* out, int M, int N, int K)
{
    #pragma omp parallel
    {
        float* wf = (float*)__builtin_alloca(sizeof(float) * (size_t)K);
        #pragma omp for schedule(static)
        for (int n = 0; n < N; ++n) {
            for (int k = 0; k < K; ++k) wf[k] = h2f(w[(size_t)n * K + k]);
            for (int m = 0; m < M; ++m) {
                float acc = 0.f;
                const uint16_t* xr = x + (size_t)m * K;
                for (int k = 0; k < K; ++k) acc = fmaf(h2f(xr[k]), wf[k], acc);
                uint16_t r = f2h(acc);
                if (bias) r = h_add(r, bias[n]);
                out[(size_t)m * N + n] = r;
            }
        }
    }
}

/* end-to-end restatement of gemm_awq_ut (kernel/gemm_quant.cu:98-122) + the bias add */
ORACLE_API void oracle_gemm_awq(const uint16_t* x, const uint32_t* qw, const uint16_t* zs,
                                const uint16_t* bias, uint16_t* out, uint16_t* w_scratch /*[N,K]*/,
                                int M, int N, int K, int g)
{
    oracle_dequant(qw, zs, w_scratch, K, N, g);
    oracle_gemm_f16(x, w_scratch, bias, out, M, N, K);
}

ORACLE_API int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
