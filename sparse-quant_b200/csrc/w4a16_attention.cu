// Decode attention over a static key/value cache, one new token per sequence.
//
// What the reference does per decoded token with torch ops - append the new key/value with torch.cat
// (modeling_opt_ours.py:249-250), bmm(q, K^T) (:306), mask + softmax, bmm(P, V) (:456), then a transpose/reshape copy
// before out_proj - is one launch here, and it consumes the output of the fused q/k/v GEMV directly:
//
//   qkv  fp16 [batch, qkv_stride]: row b = [ q (heads*D) | k (heads*D) | v (heads*D) ] of the new token
//   cache fp16 [batch, heads, max_len, D] (keys and values): row `pos` is written here, rows 0..pos are read
//   out  fp16 [batch, heads*D], ready to be the row-parallel out_proj's input
//   pos  int64 on the device (so that a captured graph can be replayed for every token)
//   optional rotary tables cos/sin fp16 [positions, D] ("rotate half" convention), applied to q and the new k
//
// One CTA per (head, sequence), 256 threads.  Scores: one lane per cached position, 16-byte loads along the key
// row, fp32 dot product against q held in shared memory.  Softmax in fp32 over the scores kept in shared memory.
// P.V: a thread owns eight adjacent output dims (16-byte loads) and every G-th position, eight loads in flight;
// the G partial sums meet in shared memory.  Bound: HBM (the cache is read once: 2 * (pos+1) * D * 2 bytes per CTA).
#include "w4a16_common.cuh"

namespace w4a16 {
namespace {

constexpr int kAttnThreads = 256;

struct AttnParams {
    const __half* qkv;
    __half* k_cache;
    __half* v_cache;
    __half* out;
    const long long* pos;
    const __half* rope_cos;
    const __half* rope_sin;
    int* error;
    int heads, max_len, qkv_stride;
    float scale;
};

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads) decode_attention_kernel(const AttnParams p)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kCols = D / 8, kGroups = kAttnThreads / kCols;          // P.V thread layout
    float* q_s = reinterpret_cast<float*>(smem_raw);                        // [D]
    float* red = q_s + D;                                                   // [kGroups][D] partial outputs; also warp scratch
    float* sc = red + kGroups * D;                                          // [max_len] scores / probabilities
    const int head = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // a following kernel launched with programmatic stream serialization (the decode GEMV prefetching its static
    // weights) may start its preamble as soon as every CTA of this grid is running
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const long long cur_ll = *p.pos;
    if (cur_ll < 0 || cur_ll >= p.max_len) {                                // position outside the cache: refuse
        if (tid == 0) atomicExch(p.error, 3);
        return;
    }
    const int cur = (int)cur_ll, n = cur + 1;
    const size_t row0 = ((size_t)b * p.heads + head) * p.max_len;          // first cache row of this (sequence, head)
    const __half* qrow = p.qkv + (size_t)b * p.qkv_stride + head * D;
    const __half* krow = qrow + p.heads * D;
    const __half* vrow = krow + p.heads * D;

    // new token: rotary embedding on q and k, k/v appended to the cache, q (scaled) to shared memory
    if (tid < D) {
        const int i = tid, j = i < D / 2 ? i + D / 2 : i - D / 2;
        float q = __half2float(qrow[i]), k = __half2float(krow[i]);
        if (p.rope_cos) {
            const float c = __half2float(p.rope_cos[(size_t)cur * D + i]), s = __half2float(p.rope_sin[(size_t)cur * D + i]);
            const float qo = __half2float(qrow[j]), ko = __half2float(krow[j]);
            const float sign = i < D / 2 ? -1.f : 1.f;                      // rotate_half: (-x[D/2:], x[:D/2])
            q = q * c + sign * qo * s;
            k = k * c + sign * ko * s;
        }
        q_s[i] = q * p.scale;
        p.k_cache[(row0 + cur) * D + i] = __float2half_rn(k);
        p.v_cache[(row0 + cur) * D + i] = vrow[i];
    }
    __syncthreads();                                                        // the appended row is visible to the CTA

    // scores: lane <-> position, 32 positions per warp pass
    float lmax = -INFINITY;
    for (int t0 = warp * 32; t0 < n; t0 += (kAttnThreads / 32) * 32) {
        const int t = t0 + lane;
        if (t < n) {
            const uint4* kr = reinterpret_cast<const uint4*>(p.k_cache + (row0 + t) * D);
            uint4 kv[D / 8];
#pragma unroll
            for (int c = 0; c < D / 8; ++c) kv[c] = kr[c];
            float dot = 0.f;
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                const __half2* h = reinterpret_cast<const __half2*>(&kv[c]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h[e]);
                    dot = fmaf(f.x, q_s[c * 8 + 2 * e], dot);
                    dot = fmaf(f.y, q_s[c * 8 + 2 * e + 1], dot);
                }
            }
            sc[t] = dot;
            lmax = fmaxf(lmax, dot);
        }
    }
    // softmax over sc[0..n)
    lmax = warp_max(lmax);
    if (lane == 0) red[warp] = lmax;
    __syncthreads();
    float gmax = red[0];
#pragma unroll
    for (int w = 1; w < kAttnThreads / 32; ++w) gmax = fmaxf(gmax, red[w]);
    __syncthreads();                                                        // red[] is reused below
    float lsum = 0.f;
    for (int t = tid; t < n; t += kAttnThreads) {
        const float e = __expf(sc[t] - gmax);
        sc[t] = e;
        lsum += e;
    }
    lsum = warp_sum(lsum);
    if (lane == 0) red[warp] = lsum;
    __syncthreads();
    float gsum = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnThreads / 32; ++w) gsum += red[w];
    const float inv = 1.f / gsum;
    __syncthreads();

    // out = P . V: thread (group, col) adds positions group, group + G, ... for dims 8 col .. 8 col + 7
    {
        const int col = tid % kCols, grp = tid / kCols;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const __half* vbase = p.v_cache + row0 * D + col * 8;
        constexpr int kUnroll = 8;
        auto add_row = [&](const uint4& v, float pr) {
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]);
                acc[2 * e] = fmaf(pr, f.x, acc[2 * e]);
                acc[2 * e + 1] = fmaf(pr, f.y, acc[2 * e + 1]);
            }
        };
        // whole chunks of kUnroll positions, the last one predicated: all loads of a chunk are in flight together
        for (int t = grp; t < n; t += kUnroll * kGroups) {
            uint4 v[kUnroll];
            float pr[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int tu = t + u * kGroups;
                const bool in = tu < n;
                v[u] = in ? *reinterpret_cast<const uint4*>(vbase + (size_t)tu * D) : make_uint4(0, 0, 0, 0);
                pr[u] = in ? sc[tu] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) add_row(v[u], pr[u]);
        }
        *reinterpret_cast<float4*>(red + grp * D + col * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(red + grp * D + col * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    __syncthreads();
    if (tid < D) {
        float s = 0.f;
#pragma unroll
        for (int g = 0; g < kGroups; ++g) s += red[g * D + tid];
        p.out[((size_t)b * p.heads + head) * D + tid] = __float2half_rn(s * inv);
    }
}

template <int D>
int launch_attention(const AttnParams& p, int batch, cudaStream_t st)
{
    constexpr int kGroups = kAttnThreads / (D / 8);
    const size_t smem = sizeof(float) * ((size_t)D + (size_t)kGroups * D + p.max_len);
    if (smem > 200 * 1024) return W4A16_ERR_TOO_LARGE;
    static int configured[64] = {0};   // benign race: the attribute call is idempotent
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (smem > 48 * 1024 && (dev >= 64 || configured[dev] < (int)smem)) {
        e = cudaFuncSetAttribute(decode_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev < 64) configured[dev] = (int)smem;
    }
    decode_attention_kernel<D><<<dim3(p.heads, batch), kAttnThreads, smem, st>>>(p);
    count_launch();
    e = cudaGetLastError();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

}  // namespace
}  // namespace w4a16

using namespace w4a16;

extern "C" int w4a16_decode_attention(const void* qkv, void* k_cache, void* v_cache, void* out, const void* pos,
                                      const void* rope_cos, const void* rope_sin, int batch, int heads, int head_dim,
                                      int max_len, int qkv_stride, float scale, void* stream)
{
    if (!qkv || !k_cache || !v_cache || !out || !pos) return W4A16_ERR_NULL_POINTER;
    if ((rope_cos == nullptr) != (rope_sin == nullptr)) return W4A16_ERR_NULL_POINTER;
    if (batch <= 0 || heads <= 0 || max_len <= 0 || batch > 65535 || qkv_stride < 3 * heads * head_dim) return W4A16_ERR_BAD_SHAPE;
    if (head_dim != 64 && head_dim != 128) return W4A16_ERR_BAD_SHAPE;
    if (((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)pos & 7)) return W4A16_ERR_MISALIGNED;
    AttnParams p;
    p.qkv = (const __half*)qkv; p.k_cache = (__half*)k_cache; p.v_cache = (__half*)v_cache; p.out = (__half*)out;
    p.pos = (const long long*)pos; p.rope_cos = (const __half*)rope_cos; p.rope_sin = (const __half*)rope_sin;
    p.error = device_error_word();
    if (!p.error) return W4A16_ERR_CUDA;
    p.heads = heads; p.max_len = max_len; p.qkv_stride = qkv_stride; p.scale = scale;
    return head_dim == 128 ? launch_attention<128>(p, batch, (cudaStream_t)stream)
                           : launch_attention<64>(p, batch, (cudaStream_t)stream);
}
