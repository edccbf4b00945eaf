// Decode kernel: skinny W4A16 GEMM (tokens <= 32 per pass), HBM-bandwidth bound.
//
//   out[t, n] = fp16( sum_k fp32( dq(W)[n, k] * x[t, k] ) ) (+ bias[n])
//
// Replaces the small-token instantiations of gemm_s4_f16_nn (gemm_template.h:358-464 of the
// reference, CTA shapes (x, 8|16, 256|512) of gemm_s4_f16.cu:66-87), which run at most N/64 CTAs
// and stream K serially.  Here the whole machine streams the weight matrix once:
//
//   * a warp owns one 32-wide out-feature tile and a contiguous K slice; every lane issues one
//     128-bit non-allocating load per 32x32 tile (512 contiguous bytes per warp), four tiles
//     (one 128-k unit) double-buffered, so 8 x 16 B are in flight per lane;
//   * nibbles are expanded in registers to fp16 (64+q), then (t - z) * s with sub.ftz/mul.ftz -
//     bit-exact with the reference - and fed as the A fragment of mma.m16n8k16 (the packed layout
//     IS that fragment); activations are staged once per CTA in shared memory and read with
//     ldmatrix as the B fragment; accumulation is fp32;
//   * split-K: WK warps of a CTA cover different K slices of the same tiles and S CTAs of one
//     thread-block cluster cover different K ranges; partial sums meet in shared memory and are
//     reduced across the cluster through distributed shared memory in a fixed order, so results
//     are deterministic and no global scratch or atomics are needed;
//   * bias add, fp16 rounding and the [tokens, N] store are fused into the reduction.
#include <cooperative_groups.h>

#include "w4a16_common.cuh"

namespace cg = cooperative_groups;

namespace w4a16 {

namespace {

constexpr int kWarps   = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kUnitK   = 128;               // k per pipeline unit (4 tiles)
constexpr int kUnitTiles = kUnitK / kTileK;

struct SkinnyParams {
    const __half*   x;
    const uint4*    qw;
    const uint32_t* zs;
    const __half*   bias;
    __half*         out;
    int tokens, N, K;
    int wn;          // out-feature tiles per CTA (1,2,4,8); WK = 8 / wn K-slices per CTA
    int splits;      // cluster size along K (gridDim.y)
    int xs_stride;   // halfs per staged activation row
};

template <int G>
struct UnitRegs {
    uint4    q[kUnitTiles];
    uint32_t zs[kUnitK / G][2][2];          // [group in unit][n half][row hi]
};

template <int G>
__device__ __forceinline__ void load_unit(UnitRegs<G>& u, const SkinnyParams& p, int unit, int nt, int lane, int k_tiles)
{
    const int n_tiles = p.N / kTileN;
    const int kt0 = unit * kUnitTiles;
#pragma unroll
    for (int t = 0; t < kUnitTiles; ++t) {
        if (kt0 + t < k_tiles)
            u.q[t] = ldg_nc_v4(p.qw + ((size_t)(kt0 + t) * n_tiles + nt) * 32 + lane);
        else
            u.q[t] = make_uint4(0, 0, 0, 0);
    }
    const int r = lane >> 2;
    const int groups = p.K / G;
#pragma unroll
    for (int gi = 0; gi < kUnitK / G; ++gi) {
        const int kg = unit * (kUnitK / G) + gi;
        const int kgc = kg < groups ? kg : groups - 1;          // clamp: value unused when past the end
        const uint32_t* row = p.zs + (size_t)kgc * p.N + nt * kTileN + r;
#pragma unroll
        for (int nh = 0; nh < 2; ++nh)
#pragma unroll
            for (int hi = 0; hi < 2; ++hi) u.zs[gi][nh][hi] = ldg_nc_u32(row + nh * 16 + hi * 8);
    }
}

template <int TG, int G>
__device__ __forceinline__ void compute_unit(const UnitRegs<G>& u, float (&acc)[TG][2][4], uint32_t xs_lane_addr,
                                             int xs_stride_bytes, int unit_local, int kt0, int k_tiles)
{
    constexpr int kTilesPerGroup = G / kTileK;
#pragma unroll
    for (int t = 0; t < kUnitTiles; ++t) {
        if (kt0 + t < k_tiles) {                                // warp-uniform
            // activations of this tile: B fragments for both 16-k halves, per token group
            uint32_t b[TG][4];
#pragma unroll
            for (int tg = 0; tg < TG; ++tg)
                ldmatrix_x4(b[tg], xs_lane_addr + tg * 8 * xs_stride_bytes + (unit_local * kUnitK + t * kTileK) * 2);
            const int gi = t / kTilesPerGroup;
            uint32_t zz[2][2], ss[2][2];
#pragma unroll
            for (int nh = 0; nh < 2; ++nh)
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) split_zs(u.zs[gi][nh][hi], zz[nh][hi], ss[nh][hi]);
            const uint32_t words[4] = {u.q[t].x, u.q[t].y, u.q[t].z, u.q[t].w};
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
                const int kh = wd >> 1, nh = wd & 1;
                uint32_t a[4];
                unpack_s4x8(words[wd], a);
                a[0] = dequant_h2(a[0], zz[nh][0], ss[nh][0]);
                a[1] = dequant_h2(a[1], zz[nh][1], ss[nh][1]);
                a[2] = dequant_h2(a[2], zz[nh][0], ss[nh][0]);
                a[3] = dequant_h2(a[3], zz[nh][1], ss[nh][1]);
#pragma unroll
                for (int tg = 0; tg < TG; ++tg) mma_m16n8k16(acc[tg][nh], a, b[tg][2 * kh], b[tg][2 * kh + 1]);
            }
        }
    }
}

// TG = token groups of 8 handled per pass (1, 2, 4); G = quantisation group size.
template <int TG, int G>
__global__ void __launch_bounds__(kThreads) skinny_kernel(const SkinnyParams p)
{
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int kTok = 8 * TG;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wn = p.wn, wk = kWarps / wn;
    const int wn_idx = warp % wn, wk_idx = warp / wn;
    const int n_tiles = p.N / kTileN;
    const int nt = blockIdx.x * wn + wn_idx;
    const bool nt_valid = nt < n_tiles;
    const int tok0 = blockIdx.z * kTok;

    // K decomposition in 128-k units: cluster rank -> CTA range -> warp slice
    const int k_tiles = p.K / kTileK;
    const int units = (p.K + kUnitK - 1) / kUnitK;
    const int S = p.splits, rank = blockIdx.y;
    const int cu0 = (int)((long long)units * rank / S), cu1 = (int)((long long)units * (rank + 1) / S);
    const int cta_units = cu1 - cu0;
    const int wu0 = cu0 + (int)((long long)cta_units * wk_idx / wk), wu1 = cu0 + (int)((long long)cta_units * (wk_idx + 1) / wk);

    __half* xs  = reinterpret_cast<__half*>(smem);
    float*  red = reinterpret_cast<float*>(smem + (size_t)kTok * p.xs_stride * sizeof(__half));
    // red: [wk][wn*32][kTok] fp32

    UnitRegs<G> cur, nxt;
    if (nt_valid && wu0 < wu1) load_unit<G>(cur, p, wu0, nt, lane, k_tiles);   // weights first: they do not depend on x

    // stage x[tok0 .. tok0+kTok) x [cu0*128, cu1*128) in shared memory (zero beyond tokens / K)
    {
        const int kc0 = cu0 * kUnitK;
        const int vec_per_row = cta_units * (kUnitK / 8);
        for (int i = threadIdx.x; i < kTok * vec_per_row; i += kThreads) {
            const int row = i / vec_per_row, v = i % vec_per_row;
            const int k = kc0 + v * 8;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (tok0 + row < p.tokens && k < p.K)
                val = *reinterpret_cast<const uint4*>(p.x + (size_t)(tok0 + row) * p.K + k);
            *reinterpret_cast<uint4*>(xs + (size_t)row * p.xs_stride + v * 8) = val;
        }
    }
    __syncthreads();

    float acc[TG][2][4];
#pragma unroll
    for (int tg = 0; tg < TG; ++tg)
#pragma unroll
        for (int nh = 0; nh < 2; ++nh)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[tg][nh][j] = 0.f;

    if (nt_valid) {
        // ldmatrix row address of this lane: matrix j = lane/8 covers k offset 8j, row = token lane%8
        const uint32_t xs_lane_addr = smem_u32(xs) + ((lane & 7) * p.xs_stride + (lane >> 3) * 8) * 2;
        const int xs_stride_bytes = p.xs_stride * 2;
        for (int u = wu0; u < wu1; ++u) {
            const bool more = u + 1 < wu1;
            if (more) load_unit<G>(nxt, p, u + 1, nt, lane, k_tiles);
            compute_unit<TG, G>(cur, acc, xs_lane_addr, xs_stride_bytes, u - cu0, u * kUnitTiles, k_tiles);
            if (more) cur = nxt;
        }
    }

    // ---- reduction: warps -> CTA (shared memory), CTAs -> cluster (distributed shared memory) ----
    const int nloc = wn * kTileN;                       // out-features per CTA
    {
        const int r = lane >> 2, c = lane & 3;
        float* dst = red + ((size_t)wk_idx * nloc + wn_idx * kTileN) * kTok;
#pragma unroll
        for (int tg = 0; tg < TG; ++tg)
#pragma unroll
            for (int nh = 0; nh < 2; ++nh) {
                float* d0 = dst + (size_t)(nh * 16 + r) * kTok + tg * 8 + 2 * c;
                *reinterpret_cast<float2*>(d0)            = make_float2(acc[tg][nh][0], acc[tg][nh][1]);
                *reinterpret_cast<float2*>(d0 + 8 * kTok) = make_float2(acc[tg][nh][2], acc[tg][nh][3]);
            }
    }
    __syncthreads();
    const int E = nloc * kTok;
    if (wk > 1) {
        for (int e = threadIdx.x; e < E; e += kThreads) {
            float s = red[e];
            for (int w = 1; w < wk; ++w) s += red[(size_t)w * E + e];
            red[e] = s;
        }
    }

    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) cluster.sync(); else __syncthreads();

    // element e' = tok * nloc + n_local (n fastest -> coalesced stores); rank r finalises a slice
    const int e_lo = (int)((long long)E * rank / S), e_hi = (int)((long long)E * (rank + 1) / S);
    for (int e = e_lo + threadIdx.x; e < e_hi; e += kThreads) {
        const int tok = e / nloc, nl = e % nloc;
        const int src = nl * kTok + tok;
        float s = 0.f;
        if (S > 1) {
            for (int q = 0; q < S; ++q) s += *cluster.map_shared_rank(red + src, q);
        } else {
            s = red[src];
        }
        const int n = blockIdx.x * nloc + nl, t = tok0 + tok;
        if (t < p.tokens && n < p.N) {
            __half h = __float2half_rn(s);
            if (p.bias) h = __hadd(h, p.bias[n]);
            p.out[(size_t)t * p.N + n] = h;
        }
    }
    if (S > 1) cluster.sync();                           // peers may still be reading this CTA's partials
}

struct Config { int tg, wn, splits; };

int g_force_wn = 0, g_force_splits = 0;

Config pick_config(int tokens, int N, int K)
{
    Config c;
    c.tg = tokens <= 8 ? 1 : (tokens <= 16 ? 2 : 4);
    const int n_tiles = N / kTileN, units = (K + kUnitK - 1) / kUnitK;
    const int passes = (tokens + 8 * c.tg - 1) / (8 * c.tg);
    // two out-feature tiles per CTA (four K slices) unless the matrix is so wide that whole-K CTAs
    // already fill the machine
    c.wn = 2;
    if (n_tiles * passes >= 148 * 16) c.wn = 4;
    while (c.wn > 1 && n_tiles % c.wn) c.wn >>= 1;
    const int wk = kWarps / c.wn;
    const int ctas_n = (n_tiles + c.wn - 1) / c.wn * passes;
    // cluster split-K until ~4 CTAs per SM, keeping at least one unit per warp slice
    c.splits = 1;
    while (c.splits < 8 && ctas_n * c.splits < 148 * 4 && units >= 2 * c.splits * wk) c.splits <<= 1;
    if (g_force_wn) c.wn = g_force_wn;
    if (g_force_splits) c.splits = g_force_splits;
    return c;
}

template <int TG, int G>
int launch_instance(const SkinnyParams& p, dim3 grid, size_t smem, cudaStream_t st)
{
    static int configured_dev[64] = {0};   // benign race: the attribute call is idempotent
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    static int max_optin[64] = {0};
    if (dev < 64 && !max_optin[dev]) {
        int v = 0;
        e = cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (e != cudaSuccess) return record_cuda_error(e);
        max_optin[dev] = v;
    }
    if (dev < 64 && (int)smem > max_optin[dev]) return W4A16_ERR_BAD_SHAPE;
    if (dev >= 64 || configured_dev[dev] < (int)smem) {
        e = cudaFuncSetAttribute(skinny_kernel<TG, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev < 64) configured_dev[dev] = (int)smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = grid.y;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, skinny_kernel<TG, G>, p);
    count_launch();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

template <int G>
int launch_g(int tg, const SkinnyParams& p, dim3 grid, size_t smem, cudaStream_t st)
{
    switch (tg) {
        case 1: return launch_instance<1, G>(p, grid, smem, st);
        case 2: return launch_instance<2, G>(p, grid, smem, st);
        default: return launch_instance<4, G>(p, grid, smem, st);
    }
}

}  // namespace

void skinny_force_config(int wn, int splits)
{
    g_force_wn = wn;
    g_force_splits = splits;
}

int launch_skinny(const GemmArgs& a, cudaStream_t st)
{
    if (a.tokens == 0) return W4A16_OK;
    Config c = pick_config(a.tokens, a.N, a.K);
    const int units = (a.K + kUnitK - 1) / kUnitK;
    if (c.splits > units) c.splits = 1;
    if (c.wn != 1 && c.wn != 2 && c.wn != 4 && c.wn != 8) return W4A16_ERR_BAD_ALGO;
    if (c.splits != 1 && c.splits != 2 && c.splits != 4 && c.splits != 8) return W4A16_ERR_BAD_ALGO;

    SkinnyParams p;
    p.x = a.x; p.qw = reinterpret_cast<const uint4*>(a.qw); p.zs = a.zs; p.bias = a.bias; p.out = a.out;
    p.tokens = a.tokens; p.N = a.N; p.K = a.K; p.wn = c.wn; p.splits = c.splits;
    const int max_cta_units = (units + c.splits - 1) / c.splits;
    p.xs_stride = max_cta_units * kUnitK + 8;           // +16 B: ldmatrix rows fall in distinct banks
    const int tok = 8 * c.tg;
    const size_t smem = (size_t)tok * p.xs_stride * sizeof(__half) + (size_t)kWarps * kTileN * tok * sizeof(float);
    const int n_tiles = a.N / kTileN;
    dim3 grid((n_tiles + c.wn - 1) / c.wn, c.splits, (a.tokens + tok - 1) / tok);
    if (grid.z > 65535) return W4A16_ERR_BAD_SHAPE;
    switch (a.g) {
        case 128: return launch_g<128>(c.tg, p, grid, smem, st);
        case 64:  return launch_g<64>(c.tg, p, grid, smem, st);
        case 32:  return launch_g<32>(c.tg, p, grid, smem, st);
        default:  return W4A16_ERR_GROUP_SIZE;
    }
}

}  // namespace w4a16
