// Residual add fused with the normalisation that follows it (decode-sized inputs: a handful of rows).
//
// Around every quantised linear the reference's decoder layers run `hidden = residual + hidden` followed by a
// LayerNorm (OPT: modeling_opt_ours.py:590,603-604 and :614 -> next layer's :561-562) or an RMSNorm (LLaMA:
// LlamaRMSNorm, modeling_llama_ours.py:113-118), each as separate torch kernels - for an [8, 4096] input that is
// launch latency only.  One launch here:
//     s     = fp16(x + delta)                      (written to x_out; skipped when delta is NULL)
//     h_out = LayerNorm(s) * weight + bias         mean / variance / affine in fp32, one rounding to fp16
//     h_out = weight * fp16(s * rsqrt(mean(s^2) + eps))    for RMSNorm, with the reference's intermediate rounding
// One CTA per row; the row stays in registers between the statistics passes.  Bound: latency (a few KB per row).
#include "w4a16_common.cuh"

namespace w4a16 {
namespace {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;                 // 16-byte vectors per thread: rows of up to 256 * 4 * 8 = 8192 halfs

struct NormParams {
    const __half* x;
    const __half* delta;
    __half* x_out;
    __half* h_out;
    const __half* weight;
    const __half* bias;
    int cols;
    float eps;
    int rms;
};

__device__ __forceinline__ float block_sum(float v, float* scratch)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                           // scratch may still be read from the previous reduction
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) s += scratch[w];
    return s;
}

__global__ void __launch_bounds__(kNormThreads) add_norm_kernel(const NormParams p)
{
    __shared__ float scratch[kNormThreads / 32];
    // lets a following kernel launched with programmatic stream serialization (the decode GEMV) start its
    // weight prefetch while these few CTAs run; this kernel itself is launched the same way and must not read its
    // inputs before the previous grid has completed
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t row = (size_t)blockIdx.x * p.cols;
    const int nvec = p.cols / 8;
    float v[kNormMaxVec][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
        const int c = threadIdx.x + i * kNormThreads;
        if (c < nvec) {
            uint4 a = *reinterpret_cast<const uint4*>(p.x + row + c * 8);
            __half2* ah = reinterpret_cast<__half2*>(&a);
            if (p.delta) {
                const uint4 d = *reinterpret_cast<const uint4*>(p.delta + row + c * 8);
                const __half2* dh = reinterpret_cast<const __half2*>(&d);
#pragma unroll
                for (int e = 0; e < 4; ++e) ah[e] = __hadd2(ah[e], dh[e]);
                *reinterpret_cast<uint4*>(p.x_out + row + c * 8) = a;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(ah[e]);
                v[i][2 * e] = f.x;
                v[i][2 * e + 1] = f.y;
                sum += p.rms ? f.x * f.x + f.y * f.y : f.x + f.y;
            }
        }
    }
    sum = block_sum(sum, scratch);
    float mean = 0.f, rstd;
    if (p.rms) {
        rstd = rsqrtf(sum / p.cols + p.eps);
    } else {
        mean = sum / p.cols;
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < kNormMaxVec; ++i)
            if (threadIdx.x + i * kNormThreads < nvec)
#pragma unroll
                for (int e = 0; e < 8; ++e) sq += (v[i][e] - mean) * (v[i][e] - mean);
        sq = block_sum(sq, scratch);
        rstd = rsqrtf(sq / p.cols + p.eps);
    }
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
        const int c = threadIdx.x + i * kNormThreads;
        if (c < nvec) {
            const uint4 w = *reinterpret_cast<const uint4*>(p.weight + c * 8);
            const __half* wh = reinterpret_cast<const __half*>(&w);
            uint4 b = make_uint4(0, 0, 0, 0);
            if (p.bias) b = *reinterpret_cast<const uint4*>(p.bias + c * 8);
            const __half* bh = reinterpret_cast<const __half*>(&b);
            uint4 o;
            __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (p.rms) oh[e] = __hmul(wh[e], __float2half_rn(v[i][e] * rstd));
                else oh[e] = __float2half_rn((v[i][e] - mean) * rstd * __half2float(wh[e]) + (p.bias ? __half2float(bh[e]) : 0.f));
            }
            *reinterpret_cast<uint4*>(p.h_out + row + c * 8) = o;
        }
    }
}

// out[r, c] = fp16(silu(gate[r, c])) * up[r, c] with in = [rows][gate (n) | up (n)]: the SwiGLU product between the fused
// gate/up GEMV and down_proj (act_fn(gate_proj(x)) * up_proj(x) in the reference's LlamaMLP, modeling_llama_ours.py:272), same roundings as
// the two torch kernels it replaces.
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* in, __half* out, int n, int total_vec)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int nvec = n / 8;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += gridDim.x * blockDim.x) {
        const int r = i / nvec, c = i - r * nvec;
        const uint4 g = *reinterpret_cast<const uint4*>(in + (size_t)r * 2 * n + c * 8);
        const uint4 u = *reinterpret_cast<const uint4*>(in + (size_t)r * 2 * n + n + c * 8);
        const __half* gh = reinterpret_cast<const __half*>(&g);
        const __half* uh = reinterpret_cast<const __half*>(&u);
        uint4 o;
        __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float x = __half2float(gh[e]);
            oh[e] = __hmul(__float2half_rn(x / (1.f + __expf(-x))), uh[e]);
        }
        *reinterpret_cast<uint4*>(out + (size_t)r * n + c * 8) = o;
    }
}

}  // namespace
}  // namespace w4a16

using namespace w4a16;

extern "C" int w4a16_silu_mul(const void* gate_up, void* out, int rows, int n, void* stream)
{
    if (!gate_up || !out) return W4A16_ERR_NULL_POINTER;
    if (rows <= 0 || n <= 0 || (n % 8) || (long long)rows * n >= (1ll << 31)) return W4A16_ERR_BAD_SHAPE;
    if (((uintptr_t)gate_up & 15) || ((uintptr_t)out & 15)) return W4A16_ERR_MISALIGNED;
    const int total_vec = rows * (n / 8);
    const int blocks = (total_vec + 255) / 256 < 592 ? (total_vec + 255) / 256 : 592;
    cudaError_t e = launch_after_previous(silu_mul_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const __half*)gate_up,
                                          (__half*)out, n, total_vec);
    count_launch();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

extern "C" int w4a16_add_norm(const void* x, const void* delta, void* x_out, void* h_out, const void* weight, const void* bias,
                              int rows, int cols, float eps, int rms, void* stream)
{
    if (!x || !h_out || !weight || (delta && !x_out)) return W4A16_ERR_NULL_POINTER;
    if (rows <= 0 || cols <= 0 || (cols % 8)) return W4A16_ERR_BAD_SHAPE;
    if (cols > kNormThreads * kNormMaxVec * 8) return W4A16_ERR_TOO_LARGE;
    if (((uintptr_t)x & 15) || ((uintptr_t)h_out & 15) || ((uintptr_t)weight & 15) || ((uintptr_t)delta & 15) ||
        ((uintptr_t)x_out & 15) || ((uintptr_t)bias & 15))
        return W4A16_ERR_MISALIGNED;
    NormParams p;
    p.x = (const __half*)x; p.delta = (const __half*)delta; p.x_out = (__half*)x_out; p.h_out = (__half*)h_out;
    p.weight = (const __half*)weight; p.bias = (const __half*)bias; p.cols = cols; p.eps = eps; p.rms = rms ? 1 : 0;
    cudaError_t e = launch_after_previous(add_norm_kernel, dim3(rows), dim3(kNormThreads), 0, (cudaStream_t)stream, p);
    count_launch();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}
