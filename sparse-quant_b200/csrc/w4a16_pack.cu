// Layout (packer) kernels and the standalone dequantiser.
//
// These are the offline ops of the path: they run once per linear when a model is quantised
// (quant_lmdeploy, test/nvidia/utils/quant_dequant_nvidia.py:5-32 of the reference).  All of
// them are HBM-bound byte shuffles: one thread produces one 32-bit (or 128-bit) output word
// with plain coalesced stores - no per-nibble atomics.
#include "w4a16_common.cuh"

namespace w4a16 {

namespace {

constexpr int kThreads = 256;

inline unsigned grid_for(size_t work, int threads = kThreads)
{
    size_t b = (work + threads - 1) / threads;
    const size_t cap = 148u * 32u;            // grid-stride beyond this
    return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

// zeros_scales[kg][n] = half2(zeros[n][kg] + 64, scales[n][kg])   (format.cu:206-224)
// Thread index runs over the OUTPUT so the 4-byte stores coalesce; the transposed reads of the
// two small [N, K/g] inputs are served by L2.
__global__ void transpose_merge_zeros_scales_kernel(const __half* __restrict__ zeros,
                                                    const __half* __restrict__ scales,
                                                    __half2* __restrict__ zs, int groups, int N)
{
    const size_t count = (size_t)groups * N;
    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < count; t += (size_t)gridDim.x * blockDim.x) {
        const int kg = (int)(t / N), n = (int)(t % N);
        const size_t i = (size_t)n * groups + kg;
        zs[t] = __halves2half2(__hadd(zeros[i], __float2half(64.0f)), scales[i]);
    }
}

// "ours" uint8 [N, K/2] -> AWQ uint32 [K, N/8]   (format.cu:151-189)
// word (k, c): nibble p holds q[8c + e, k], e = {0,2,4,6,1,3,5,7}[p].
__global__ void convert_ours_to_awq_kernel(const uint8_t* __restrict__ src, uint32_t* __restrict__ dst, int K, int N)
{
    const int dst_w = N / 8, src_w = K / 2;
    const size_t count = (size_t)K * dst_w;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const int k = (int)(i / dst_w), c = (int)(i % dst_w);
        const int shift = (k & 1) ? 0 : 4;
        uint32_t v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (src[(size_t)(c * 8 + j) * src_w + (k >> 1)] >> shift) & 0xf;
        dst[i] = v[0] | (v[2] << 4) | (v[4] << 8) | (v[6] << 12) | (v[1] << 16) | (v[3] << 20) | (v[5] << 24) | (v[7] << 28);
    }
}

// AWQ uint32 [K, N/8] -> tile order [K/32][N/32][32][4]   (format.cu:24-71, closed form).
// One thread builds one destination word = 8 nibbles (k%2, (k/8)%2, (n/8)%2) of a fixed
// (tile, lane, word); each comes from AWQ word (k, n/8), nibble slot of n%8.
__global__ void convert_awq_to_lmdeploy_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int K, int N)
{
    const int n_tiles = N / 32;
    const size_t count = (size_t)K * N / 8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const int word = (int)(i & 3), lane = (int)((i >> 2) & 31);
        const size_t tile = i >> 7;
        const int kt = (int)(tile / n_tiles), nt = (int)(tile % n_tiles);
        const int r = lane >> 2, c = lane & 3;
        const int kh = word >> 1, nh = word & 1;
        // AWQ nibble slot of out-feature e = n % 8:  e even -> e/2, e odd -> 4 + e/2
        const int slot = (r & 1) ? 4 + (r >> 1) : (r >> 1);
        uint32_t out = 0;
#pragma unroll
        for (int nib = 0; nib < 8; ++nib) {
            const int k = kt * 32 + kh * 16 + ((nib >> 1) & 1) * 8 + 2 * c + (nib >> 2);
            const int n = nt * 32 + nh * 16 + (nib & 1) * 8 + r;
            const uint32_t w = src[(size_t)k * (N / 8) + (n >> 3)];
            out |= ((w >> (4 * slot)) & 0xf) << (4 * nib);
        }
        dst[i] = out;
    }
}

// Packed -> fp16 [N, K], bit-exact (common.h:114-153,210-225).  One thread handles one lane of
// one tile (16 bytes in, 32 weights out); the 2-byte-pair stores of a warp land in 8 rows of 64
// contiguous bytes each.
template <int G>
__global__ void dequant_kernel(const uint4* __restrict__ qw, const uint32_t* __restrict__ zs,
                               __half* __restrict__ w, int K, int N)
{
    const int n_tiles = N / 32;
    const size_t count = (size_t)(K / 32) * n_tiles * 32;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const int lane = (int)(i & 31);
        const size_t tile = i >> 5;
        const int kt = (int)(tile / n_tiles), nt = (int)(tile % n_tiles);
        const int r = lane >> 2, c = lane & 3;
        const uint4 q = qw[i];
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
        const int kg = (kt * 32) / G;
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
            const int kh = wd >> 1, nh = wd & 1;
            uint32_t h[4];
            unpack_s4x8(words[wd], h);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = nt * 32 + nh * 16 + (j & 1) * 8 + r;
                const int k = kt * 32 + kh * 16 + (j >> 1) * 8 + 2 * c;
                uint32_t zz, ss;
                split_zs(zs[(size_t)kg * N + n], zz, ss);
                const uint32_t v = dequant_h2(h[j], zz, ss);
                *reinterpret_cast<uint32_t*>(w + (size_t)n * K + k) = v;
            }
        }
    }
}

}  // namespace

}  // namespace w4a16

using namespace w4a16;

extern "C" int w4a16_transpose_merge_zeros_scales(const void* zeros, const void* scales, void* zeros_scales,
                                                  int in_features, int out_features, int group_size, void* stream)
{
    if (!zeros || !scales || !zeros_scales) return W4A16_ERR_NULL_POINTER;
    if (group_size <= 0) return W4A16_ERR_GROUP_SIZE;
    if (in_features <= 0 || out_features <= 0 || in_features % group_size) return W4A16_ERR_BAD_SHAPE;
    if (((uintptr_t)zeros_scales & 3)) return W4A16_ERR_MISALIGNED;
    const int groups = in_features / group_size;
    transpose_merge_zeros_scales_kernel<<<grid_for((size_t)groups * out_features), kThreads, 0, (cudaStream_t)stream>>>(
        (const __half*)zeros, (const __half*)scales, (__half2*)zeros_scales, groups, out_features);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

extern "C" int w4a16_convert_ours_to_awq(const void* qweight_src, void* qweight_dst, int in_features,
                                         int out_features, void* stream)
{
    if (!qweight_src || !qweight_dst) return W4A16_ERR_NULL_POINTER;
    if (in_features <= 0 || out_features <= 0 || (in_features & 1) || (out_features & 7)) return W4A16_ERR_BAD_SHAPE;
    if (((uintptr_t)qweight_dst & 3)) return W4A16_ERR_MISALIGNED;
    convert_ours_to_awq_kernel<<<grid_for((size_t)in_features * out_features / 8), kThreads, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)qweight_src, (uint32_t*)qweight_dst, in_features, out_features);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

extern "C" int w4a16_convert_awq_to_lmdeploy(const void* qweight_src, void* qweight_dst, int in_features,
                                             int out_features, void* stream)
{
    if (!qweight_src || !qweight_dst) return W4A16_ERR_NULL_POINTER;
    if (in_features <= 0 || out_features <= 0 || (in_features % 32) || (out_features % 32)) return W4A16_ERR_BAD_SHAPE;
    if (((uintptr_t)qweight_dst & 3) || ((uintptr_t)qweight_src & 3)) return W4A16_ERR_MISALIGNED;
    if (qweight_src == qweight_dst) return W4A16_ERR_BAD_SHAPE;   // not an in-place transform
    convert_awq_to_lmdeploy_kernel<<<grid_for((size_t)in_features * out_features / 8), kThreads, 0, (cudaStream_t)stream>>>(
        (const uint32_t*)qweight_src, (uint32_t*)qweight_dst, in_features, out_features);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

extern "C" int w4a16_dequant(const void* qweight, const void* zeros_scales, void* w_out, int N, int K,
                             int group_size, void* stream)
{
    if (!qweight || !zeros_scales || !w_out) return W4A16_ERR_NULL_POINTER;
    if (group_size != 32 && group_size != 64 && group_size != 128) return W4A16_ERR_GROUP_SIZE;
    if (N <= 0 || K <= 0 || (N % 32) || (K % group_size)) return W4A16_ERR_BAD_SHAPE;
    if (((uintptr_t)qweight & 15) || ((uintptr_t)zeros_scales & 3) || ((uintptr_t)w_out & 3)) return W4A16_ERR_MISALIGNED;
    const unsigned grid = grid_for((size_t)K * N / 32);
    cudaStream_t st = (cudaStream_t)stream;
    if (group_size == 128)
        dequant_kernel<128><<<grid, kThreads, 0, st>>>((const uint4*)qweight, (const uint32_t*)zeros_scales, (__half*)w_out, K, N);
    else if (group_size == 64)
        dequant_kernel<64><<<grid, kThreads, 0, st>>>((const uint4*)qweight, (const uint32_t*)zeros_scales, (__half*)w_out, K, N);
    else
        dequant_kernel<32><<<grid, kThreads, 0, st>>>((const uint4*)qweight, (const uint32_t*)zeros_scales, (__half*)w_out, K, N);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}
