// Quantise and pack in one kernel: fp16 weight [N, K] -> tile-ordered int4 `weight` + `zeros_scales`.
//
// Replaces, for the offline quantise-and-pack flow of the reference (quant_lmdeploy,
// test/nvidia/utils/quant_dequant_nvidia.py:5-32), the chain
//     quantize_tensor  (:124-148: seven fp16 torch elementwise / reduce kernels)
//  -> write_4bit_tensor (:79-88)
//  -> transpose_merge_zeros_scales (kernel/gemm_s4_f16/format.cu:206-239)
//  -> convert_ours_to_awq          (format.cu:151-201)
//  -> convert_awq_to_lmdeploy      (format.cu:135-149, 24-71: one nibble per thread iteration through atomicCAS)
// with ONE pass over the weight: a CTA takes a block of 32 out-features x 128 in-features, computes min/max, scale,
// zero point and the 4-bit codes of every quantisation group in it with the reference's fp16 operation order, and
// writes the packed 32x32 tiles directly in their final order (the AWQ intermediate never exists).
//
// Arithmetic, bit for bit what the torch fp16 ops of the reference produce (each step rounds to fp16 once,
// round-to-nearest-even, computed in fp32 like torch's half kernels; division is IEEE fp32 division):
//     d      = fp16(max - min);  d = max(d, fp16(1e-5))              (.clamp(min=1e-5))
//     scale  = fp16(d / 15)
//     zero   = clamp(-rint(fp16(min / scale)), 0, 15)                (torch.round = half to even)
//     q      = clamp(fp16(rint(fp16(w / scale)) + zero), 0, 15)
//     w_fp16 = fp16((q - zero) * scale)                              (no flush-to-zero: this is the quantizer's own
//                                                                    dequantised copy, not the kernel's)
// Outputs: weight int32 [K, N/8] in tile order, zeros_scales fp16 [K/g, 2N] = (zero + 64, scale), and optionally
// w_fp16 [N, K], zeros / scales fp16 [N, K/g] and the reference's intermediate "ours" bytes uint8 [N, K/2].
#include "w4a16_common.cuh"

namespace w4a16 {
namespace {

constexpr int kBlockK = 128;      // in-features per CTA: one to four quantisation groups
constexpr int kRows   = 32;       // out-features per CTA: one packed tile column

struct QuantParams {
    const __half* w;        // [N, K]
    uint32_t* qweight;      // [K/32][N/32][32 lanes][4 words]
    __half2* zs;            // [K/g][N]
    __half* w_fp16;         // [N, K] or null
    __half* zeros;          // [N, K/g] or null
    __half* scales;         // [N, K/g] or null
    uint8_t* ours;          // [N, K/2] or null
    int N, K, g;
};

__device__ __forceinline__ float h2f(__half h) { return __half2float(h); }
__device__ __forceinline__ __half f2h(float f) { return __float2half_rn(f); }

__global__ void __launch_bounds__(256) quantize_pack_kernel(const QuantParams p)
{
    __shared__ uint8_t qs[kRows][kBlockK + 4];          // 4-bit codes of the block, one byte each
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kRows, k0 = blockIdx.y * kBlockK;
    const int kw = min(kBlockK, p.K - k0);              // in-features of this block (a multiple of g and of 32)
    const int lanes_per_group = p.g / 4;                // a lane holds 4 consecutive in-features
    const int groups_total = p.K / p.g;

    // phase 1: a warp takes rows warp, warp + 8, ...; lane l holds in-features k0 + 4l .. 4l + 3
    for (int row = warp; row < kRows; row += 8) {
        const int n = n0 + row;
        const int k = k0 + 4 * lane;
        const bool live = k < k0 + kw;
        __half v[4];
        if (live) {
            const uint2 raw = *reinterpret_cast<const uint2*>(p.w + (size_t)n * p.K + k);
            *reinterpret_cast<uint2*>(v) = raw;
        } else {
            v[0] = v[1] = v[2] = v[3] = __half();
        }
        float mx = fmaxf(fmaxf(h2f(v[0]), h2f(v[1])), fmaxf(h2f(v[2]), h2f(v[3])));
        float mn = fminf(fminf(h2f(v[0]), h2f(v[1])), fminf(h2f(v[2]), h2f(v[3])));
        for (int off = 1; off < lanes_per_group; off <<= 1) {       // reduce inside the lanes of one group
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
        }
        // max, min are exact fp16 values; every step below rounds to fp16 like the reference's torch ops
        float d = h2f(f2h(mx - mn));
        d = fmaxf(d, h2f(f2h(1e-5f)));
        const __half scale_h = f2h(__fdiv_rn(d, 15.f));
        const float scale = h2f(scale_h);
        const float t = h2f(f2h(__fdiv_rn(mn, scale)));
        const float zero = fminf(fmaxf(-rintf(t), 0.f), 15.f);      // -rint(+-inf) clamps as torch does; min == 0 gives 0
        uint32_t code[4];
        __half deq[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float r = rintf(h2f(f2h(__fdiv_rn(h2f(v[j]), scale))));
            const float q = fminf(fmaxf(h2f(f2h(r + zero)), 0.f), 15.f);
            code[j] = (uint32_t)q;
            deq[j] = f2h((q - zero) * scale);
        }
        if (live) {
            *reinterpret_cast<uint32_t*>(&qs[row][4 * lane]) = code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24);
            if (p.w_fp16) *reinterpret_cast<uint2*>(p.w_fp16 + (size_t)n * p.K + k) = *reinterpret_cast<const uint2*>(deq);
            if (p.ours) {
                const uint32_t b0 = (code[0] << 4) | code[1], b1 = (code[2] << 4) | code[3];       // high nibble = even k
                *reinterpret_cast<uint16_t*>(p.ours + (size_t)n * (p.K / 2) + k / 2) = (uint16_t)(b0 | (b1 << 8));
            }
            if ((lane & (lanes_per_group - 1)) == 0) {
                const int kg = k / p.g;
                p.zs[(size_t)kg * p.N + n] = __halves2half2(f2h(zero + 64.f), scale_h);           // zero + 64 is exact in fp16
                if (p.zeros) p.zeros[(size_t)n * groups_total + kg] = f2h(zero);
                if (p.scales) p.scales[(size_t)n * groups_total + kg] = scale_h;
            }
        }
    }
    __syncthreads();

    // phase 2: the block's kw / 32 packed tiles, one 32-bit word (8 codes) per thread and step.  For element (n, k) of
    // a tile: lane = (n % 8) * 4 + (k % 8) / 2, word = ((k / 16) % 2) * 2 + (n / 16) % 2,
    // nibble = (k % 2) * 4 + ((k / 8) % 2) * 2 + (n / 8) % 2.
    const int n_tiles = p.N / kTileN;
    const int words = (kw / kTileK) * 128;
    for (int i = threadIdx.x; i < words; i += blockDim.x) {
        const int t = i >> 7, l = (i >> 2) & 31, wd = i & 3;
        uint32_t out = 0;
#pragma unroll
        for (int nib = 0; nib < 8; ++nib) {
            const int n = (l >> 2) + 8 * (nib & 1) + 16 * (wd & 1);
            const int k = t * kTileK + 2 * (l & 3) + ((nib >> 2) & 1) + 8 * ((nib >> 1) & 1) + 16 * (wd >> 1);
            out |= (uint32_t)qs[n][k] << (4 * nib);
        }
        p.qweight[((size_t)(k0 / kTileK + t) * n_tiles + blockIdx.x) * 128 + (i & 127)] = out;
    }
}

}  // namespace
}  // namespace w4a16

using namespace w4a16;

extern "C" int w4a16_quantize_pack(const void* weight, void* qweight, void* zeros_scales, void* w_fp16, void* zeros,
                                   void* scales, void* qweight_ours, int in_features, int out_features, int group_size,
                                   void* stream)
{
    const int K = in_features, N = out_features, g = group_size;
    if (g != 32 && g != 64 && g != 128) return W4A16_ERR_GROUP_SIZE;
    if (N <= 0 || K <= 0 || (N % 32) || (K % g)) return W4A16_ERR_BAD_SHAPE;
    if ((long long)N * K >= (1ll << 40) || (K + kBlockK - 1) / kBlockK > 65535) return W4A16_ERR_BAD_SHAPE;
    if (!weight || !qweight || !zeros_scales) return W4A16_ERR_NULL_POINTER;
    if (((uintptr_t)weight & 7) || ((uintptr_t)qweight & 3) || ((uintptr_t)zeros_scales & 3) || ((uintptr_t)w_fp16 & 7) ||
        ((uintptr_t)zeros & 1) || ((uintptr_t)scales & 1) || ((uintptr_t)qweight_ours & 1))
        return W4A16_ERR_MISALIGNED;
    QuantParams p;
    p.w = (const __half*)weight; p.qweight = (uint32_t*)qweight; p.zs = (__half2*)zeros_scales;
    p.w_fp16 = (__half*)w_fp16; p.zeros = (__half*)zeros; p.scales = (__half*)scales; p.ours = (uint8_t*)qweight_ours;
    p.N = N; p.K = K; p.g = g;
    dim3 grid(N / kRows, (K + kBlockK - 1) / kBlockK);
    quantize_pack_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}
