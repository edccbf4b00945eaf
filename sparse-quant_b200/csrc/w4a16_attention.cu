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
// One CTA - or a cluster of up to 8 splitting the positions - per (head, sequence), 256 threads.  Scores: D/8
// adjacent lanes per cached key row (coalesced 16-byte loads, eight in flight per lane), q in registers, shuffle
// reduction, fp32.  Softmax in fp32 over the scores kept in shared memory.
// P.V: a thread owns eight adjacent output dims (16-byte loads) and every G-th position, eight loads in flight;
// the G partial sums meet in shared memory.  Bound: HBM (the cache is read once: 2 * (pos+1) * D * 2 bytes per CTA).
#include <cooperative_groups.h>

#include "w4a16_common.cuh"

namespace cg = cooperative_groups;

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

// fp32 load from the shared memory of CTA `rank` of this cluster
__device__ __forceinline__ float ld_cluster(const float* local, unsigned rank)
{
    unsigned remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// grid = (heads, batch, S); the S CTAs of a thread-block cluster split the cached positions of one (head, sequence)
// evenly, each produces (max, sum, unnormalised output) of its range, and CTA 0 combines them through distributed
// shared memory.  S is fixed by the host (it cannot know the position), so that few (head, sequence) pairs - the
// head-sharded case under tensor parallelism - still fill the machine and keep the per-CTA chain of dependent
// memory round trips short.
template <int D>
__global__ void __launch_bounds__(kAttnThreads) decode_attention_kernel(const AttnParams p)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kCols = D / 8, kGroups = kAttnThreads / kCols;          // P.V thread layout
    float* q_s = reinterpret_cast<float*>(smem_raw);                        // [D]
    float* part = q_s + D;                                                  // [D] this CTA's unnormalised output, then [2]: max, sum
    float* red = part + D + 8;                                              // [kGroups][D] partial outputs; also warp scratch
    float* sc = red + kGroups * D;                                          // [max_len] scores / probabilities
    const int head = blockIdx.x, b = blockIdx.y;
    const int S = gridDim.z, rank = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // a following kernel launched with programmatic stream serialization (the decode GEMV prefetching its static
    // weights) may start its preamble as soon as every CTA of this grid is running
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");      // launched early itself: q/k/v and the position come from earlier work
    const long long cur_ll = *p.pos;
    if (cur_ll < 0 || cur_ll >= p.max_len) {                                // position outside the cache: refuse
        if (tid == 0) atomicExch(p.error, 3);                               // (uniform over the cluster: nobody waits)
        return;
    }
    const int cur = (int)cur_ll, n = cur + 1;
    const int t_lo = (int)((unsigned)(n * rank) / (unsigned)S), t_hi = (int)((unsigned)(n * (rank + 1)) / (unsigned)S);   // the last rank owns `cur`
    const size_t row0 = ((size_t)b * p.heads + head) * p.max_len;          // first cache row of this (sequence, head)
    const __half* qrow = p.qkv + (size_t)b * p.qkv_stride + head * D;
    const __half* krow = qrow + p.heads * D;
    const __half* vrow = krow + p.heads * D;

    // new token: rotary embedding on q and k, k/v appended to the cache (by the rank that reads it back), q
    // (scaled) to shared memory
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
        if (rank == S - 1) {
            p.k_cache[(row0 + cur) * D + i] = __float2half_rn(k);
            p.v_cache[(row0 + cur) * D + i] = vrow[i];
        }
    }
    __syncthreads();                                                        // the appended row is visible to the CTA

    // scores: D/8 adjacent lanes read one key row with 16-byte loads (a warp load covers 32/(D/8) whole rows: fully
    // coalesced), eight row groups in flight per lane; each lane multiplies its 8 dims by q from registers and the
    // row's lanes add up with shuffles
    constexpr int kLPR = D / 8, kRPI = 32 / kLPR, kU = 8;                   // lanes per row, rows per warp load, loads in flight
    const int sub = lane / kLPR, li = lane % kLPR;
    float qreg[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) qreg[e] = q_s[li * 8 + e];
    float lmax = -INFINITY;
    for (int base = t_lo + warp * (kRPI * kU); base < t_hi; base += (kAttnThreads / 32) * (kRPI * kU)) {
        uint4 kv[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int t = base + u * kRPI + sub;
            kv[u] = t < t_hi ? *reinterpret_cast<const uint4*>(p.k_cache + (row0 + t) * D + li * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const __half2* h = reinterpret_cast<const __half2*>(&kv[u]);
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]);
                dot = fmaf(f.x, qreg[2 * e], dot);
                dot = fmaf(f.y, qreg[2 * e + 1], dot);
            }
#pragma unroll
            for (int o = kLPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            const int t = base + u * kRPI + sub;
            if (li == 0 && t < t_hi) {
                sc[t - t_lo] = dot;
                lmax = fmaxf(lmax, dot);
            }
        }
    }
    // softmax numerators over this CTA's range, relative to its own maximum
    lmax = warp_max(lmax);
    if (lane == 0) red[warp] = lmax;
    __syncthreads();
    float gmax = red[0];
#pragma unroll
    for (int w = 1; w < kAttnThreads / 32; ++w) gmax = fmaxf(gmax, red[w]);
    __syncthreads();                                                        // red[] is reused below
    const int cnt = t_hi - t_lo;
    float lsum = 0.f;
    for (int t = tid; t < cnt; t += kAttnThreads) {
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
    __syncthreads();

    // P . V: thread (group, col) adds positions group, group + G, ... for dims 8 col .. 8 col + 7
    {
        const int col = tid % kCols, grp = tid / kCols;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const __half* vbase = p.v_cache + (row0 + t_lo) * D + col * 8;
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
        for (int t = grp; t < cnt; t += kUnroll * kGroups) {
            uint4 v[kUnroll];
            float pr[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int tu = t + u * kGroups;
                const bool in = tu < cnt;
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
    float mine = 0.f;
    if (tid < D) {
#pragma unroll
        for (int g = 0; g < kGroups; ++g) mine += red[g * D + tid];
    }
    __half* dst = p.out + ((size_t)b * p.heads + head) * D;
    if (S == 1) {
        if (tid < D) dst[tid] = __float2half_rn(mine / gsum);
        return;
    }
    // combine the ranks: out = sum_r acc_r e^(m_r - M) / sum_r l_r e^(m_r - M); a rank without positions has
    // m_r = -inf, l_r = 0 and drops out
    if (tid < D) part[tid] = mine;
    if (tid == 0) { part[D] = gmax; part[D + 1] = gsum; }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (rank == 0 && tid < D) {
        float M = -INFINITY;
        for (int r = 0; r < S; ++r) M = fmaxf(M, ld_cluster(part + D, (unsigned)r));
        float num = 0.f, den = 0.f;
        for (int r = 0; r < S; ++r) {
            const float w = __expf(ld_cluster(part + D, (unsigned)r) - M);
            num = fmaf(ld_cluster(part + tid, (unsigned)r), w, num);
            den = fmaf(ld_cluster(part + D + 1, (unsigned)r), w, den);
        }
        dst[tid] = __float2half_rn(num / den);
    }
    cluster.sync();                                                         // rank 0 may still be reading this CTA's part[]
}

int g_force_attn_split = 0;

template <int D>
int launch_attention(const AttnParams& p, int batch, cudaStream_t st)
{
    constexpr int kGroups = kAttnThreads / (D / 8);
    const size_t smem = sizeof(float) * ((size_t)2 * D + 8 + (size_t)kGroups * D + p.max_len);
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
    // context split: enough CTAs for two per SM, at most 8 per (head, sequence), not more than one per 32 cache rows
    int split = 1;
    while (split < 8 && (long long)p.heads * batch * split < 2 * 148 && split * 2 * 32 <= p.max_len) split <<= 1;
    if (g_force_attn_split) split = g_force_attn_split;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.heads, batch, split);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = split;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = aux_programmatic_launch() ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, decode_attention_kernel<D>, p);
    count_launch();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

}  // namespace
}  // namespace w4a16

using namespace w4a16;

// Tuning hook for tests and benchmarks: CTAs per (head, sequence), 0 = automatic.  Not part of the drop-in surface.
extern "C" void w4a16_tune_attention(int split) { w4a16::g_force_attn_split = (split == 1 || split == 2 || split == 4 || split == 8) ? split : 0; }

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
