// Peer-memory exchange buffers and the C-ABI entry point of the decode GEMV fused with its all-reduce.
//
// A row-parallel linear (out_proj / fc2 / o_proj / down_proj under tensor parallelism) multiplies its K shard and
// then needs the sum over ranks.  For decode-sized inputs the sum is done inside the GEMV kernel: each CTA pushes
// its fp32 partial outputs over NVLink into every rank's exchange buffer as (value, tag) pairs in single 8-byte
// stores, polls (bounded) its own buffer until every rank's pair carries the call's tag, and adds the `world`
// partials in rank order.  No NCCL call, nothing that a
// stream capture cannot record; partials stay fp32 until the single final rounding.
//
// The buffers are ordinary device allocations shared through CUDA IPC: w4a16_exchange_alloc on every rank, the
// 64-byte handles exchanged by the host program (any transport), w4a16_exchange_open on every peer handle.
#include <atomic>
#include <cstddef>
#include <cstring>

#include "w4a16_common.cuh"

namespace w4a16 {
static std::atomic<unsigned long long> g_peer_wait_ns{2000ull * 1000 * 1000};
unsigned long long exchange_wait_budget_ns() { return g_peer_wait_ns.load(std::memory_order_relaxed); }
}  // namespace w4a16

using namespace w4a16;

namespace {

__device__ __forceinline__ unsigned long long timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

struct GatherParams {
    unsigned char* peer[kExchangeMaxWorld];
    unsigned char* self;
    const unsigned* in;      // `words` 32-bit words of this rank
    unsigned* out;           // [world][words]
    int* error;
    int words, world, rank;
    long long capacity;
    unsigned long long wait_budget_ns;
};

// All-gather of a few 32-bit words per rank through the exchange buffers (one CTA): write (word, tag) into slot
// [half][rank][i] of every rank's buffer, poll this rank's `world` slots of word i until all carry this call's tag,
// copy them out in rank order, advance the epoch.  Same protocol as the fused GEMV epilogue, so the two can be
// mixed on one set of buffers.
__global__ void __launch_bounds__(256) exchange_allgather_kernel(const GatherParams p)
{
    ExchangeHeader* hdr = reinterpret_cast<ExchangeHeader*>(p.self);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const unsigned epoch = *reinterpret_cast<volatile unsigned*>(&hdr->epoch);
    const unsigned half_sel = epoch & 1u, tag = epoch + 1u;
    for (int i = threadIdx.x; i < p.words; i += blockDim.x) {
        const unsigned v = p.in[i];
        const size_t idx = (size_t)(half_sel * p.world + p.rank) * p.capacity + i;
#pragma unroll
        for (int d = 0; d < kExchangeMaxWorld; ++d)
            if (d < p.world)
                asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(reinterpret_cast<uint2*>(p.peer[d] + kExchangeDataOffset) + idx), "r"(v), "r"(tag) : "memory");
    }
    const uint2* data = reinterpret_cast<const uint2*>(p.self + kExchangeDataOffset) + (size_t)half_sel * p.world * p.capacity;
    bool dead = *reinterpret_cast<volatile int*>(&hdr->error) != 0;      // an earlier wait gave up: do not wait again
    for (int i = threadIdx.x; i < p.words * p.world; i += blockDim.x) {
        const int src = i / p.words, w = i - src * p.words;
        const uint2* slot = data + (size_t)src * p.capacity + w;
        uint2 v;
        unsigned long long t0 = 0;
        for (unsigned polls = 0;; ++polls) {
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(slot) : "memory");
            if (v.y == tag || dead) break;
            if ((polls & 63u) == 63u) {
                const unsigned long long now = timer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > p.wait_budget_ns) {
                    atomicExch(p.error, 2);
                    atomicExch(&hdr->error, 1 + src);
                    dead = true;
                }
            }
        }
        p.out[i] = v.x;
    }
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned*>(&hdr->epoch) = epoch + 1;
}

}  // namespace

extern "C" size_t w4a16_exchange_bytes(int world, size_t capacity_elems)
{
    if (world < 1 || world > kExchangeMaxWorld) return 0;
    return kExchangeDataOffset + 2 * (size_t)world * capacity_elems * 8;   // (payload, tag) slots
}

extern "C" int w4a16_exchange_alloc(int world, size_t capacity_elems, void** buffer)
{
    if (!buffer) return W4A16_ERR_NULL_POINTER;
    const size_t bytes = w4a16_exchange_bytes(world, capacity_elems);
    if (!bytes || !capacity_elems) return W4A16_ERR_BAD_SHAPE;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return record_cuda_error(e);
    e = cudaMemset(p, 0, bytes);                       // epoch 0, all flags 0: no call has happened yet
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { cudaFree(p); return record_cuda_error(e); }
    *buffer = p;
    return W4A16_OK;
}

extern "C" int w4a16_exchange_free(void* buffer)
{
    if (!buffer) return W4A16_OK;
    cudaError_t e = cudaFree(buffer);
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

extern "C" int w4a16_exchange_export(void* buffer, void* handle64)
{
    if (!buffer || !handle64) return W4A16_ERR_NULL_POINTER;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, buffer);
    if (e != cudaSuccess) return record_cuda_error(e);
    std::memcpy(handle64, &h, 64);
    return W4A16_OK;
}

extern "C" int w4a16_exchange_open(const void* handle64, void** peer_buffer)
{
    if (!handle64 || !peer_buffer) return W4A16_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return record_cuda_error(e);
    *peer_buffer = p;
    return W4A16_OK;
}

extern "C" int w4a16_exchange_close(void* peer_buffer)
{
    if (!peer_buffer) return W4A16_OK;
    cudaError_t e = cudaIpcCloseMemHandle(peer_buffer);
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

extern "C" int w4a16_exchange_status(const void* buffer, unsigned* epoch, int* error)
{
    if (!buffer) return W4A16_ERR_NULL_POINTER;
    ExchangeHeader h;
    cudaError_t e = cudaMemcpy(&h, buffer, sizeof(h), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (epoch) *epoch = h.epoch;
    if (error) *error = h.error;
    return W4A16_OK;
}

extern "C" int w4a16_exchange_reset(void* buffer)
{
    if (!buffer) return W4A16_ERR_NULL_POINTER;
    cudaError_t e = cudaDeviceSynchronize();                 // no call may be using the buffer
    if (e == cudaSuccess) e = cudaMemset((unsigned char*)buffer + offsetof(ExchangeHeader, ticket), 0, sizeof(unsigned) + sizeof(int));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

extern "C" void w4a16_tune_exchange_wait(unsigned milliseconds)
{
    g_peer_wait_ns.store(milliseconds ? (unsigned long long)milliseconds * 1000000ull : 2000ull * 1000 * 1000, std::memory_order_relaxed);
}

extern "C" int w4a16_gemm_allreduce_residual(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                                             const void* residual, void* out, void* row_stats_out, int tokens, int N, int K,
                                             int group_size, int k_config, void* const* buffers, int world, int rank,
                                             size_t capacity_elems, void* stream, unsigned flags)
{
    if ((residual && ((uintptr_t)residual & 1)) || ((uintptr_t)row_stats_out & 15)) return W4A16_ERR_MISALIGNED;
    if (group_size != 32 && group_size != 64 && group_size != 128) return W4A16_ERR_GROUP_SIZE;
    if (tokens <= 0 || N <= 0 || K <= 0 || (N % 32) || (K % group_size) || k_config < K) return W4A16_ERR_BAD_SHAPE;
    if (tokens > 32) return W4A16_ERR_TOO_LARGE;
    if (!x || !qweight || !zeros_scales || !out || !buffers) return W4A16_ERR_NULL_POINTER;
    if (((uintptr_t)x & 15) || ((uintptr_t)qweight & 15) || ((uintptr_t)zeros_scales & 15) || ((uintptr_t)out & 15))
        return W4A16_ERR_MISALIGNED;
    if (world < 1 || world > kExchangeMaxWorld || rank < 0 || rank >= world) return W4A16_ERR_BAD_SHAPE;
    if (flags & ~(unsigned)(W4A16_FLAG_STATIC_WEIGHTS | W4A16_FLAG_RELU)) return W4A16_ERR_BAD_ALGO;
    int dev = 0, major = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (major != 10) return W4A16_ERR_UNSUPPORTED_GPU;

    ExchangeArgs ex;
    for (int d = 0; d < kExchangeMaxWorld; ++d) ex.peer[d] = d < world ? (unsigned char*)buffers[d] : nullptr;
    ex.world = world; ex.rank = rank; ex.capacity = (long long)capacity_elems; ex.k_config = k_config;
    GemmArgs a;
    a.x = (const __half*)x; a.qw = (const uint32_t*)qweight; a.zs = (const uint32_t*)zeros_scales;
    a.bias = (const __half*)bias; a.out = (__half*)out;
    a.tokens = tokens; a.N = N; a.K = K; a.g = group_size;
    a.static_weights = (flags & W4A16_FLAG_STATIC_WEIGHTS) != 0;
    a.relu = (flags & W4A16_FLAG_RELU) != 0;
    a.exchange = &ex;
    a.residual = (const __half*)residual;
    a.row_stats_out = (float*)row_stats_out;
    return launch_skinny(a, (cudaStream_t)stream);
}

// Whether w4a16_gemm_allreduce(_residual) accepts this problem: the fused exchange needs one pass of at most 32 tokens
// whose whole grid is resident at once (the ranks wait for each other inside the kernel).  Deterministic from the
// shapes (and the SM count of the current device), so all ranks of a homogeneous node agree and can choose the
// library all-reduce up front instead.
extern "C" int w4a16_allreduce_supported(int tokens, int N, int K, int k_config, int group_size, int world)
{
    if (group_size != 32 && group_size != 64 && group_size != 128) return 0;
    if (tokens <= 0 || tokens > 32 || N <= 0 || K <= 0 || (N % 32) || (K % group_size) || k_config < K) return 0;
    if (world < 1 || world > kExchangeMaxWorld) return 0;
    static unsigned char dummy;
    ExchangeArgs ex;
    for (int d = 0; d < kExchangeMaxWorld; ++d) ex.peer[d] = d < world ? &dummy : nullptr;
    ex.world = world; ex.rank = 0; ex.capacity = (long long)tokens * N; ex.k_config = k_config;
    GemmArgs a;
    a.x = nullptr; a.qw = nullptr; a.zs = nullptr; a.bias = nullptr; a.out = nullptr;
    a.tokens = tokens; a.N = N; a.K = K; a.g = group_size; a.static_weights = false;
    a.exchange = &ex;
    a.plan_only = true;
    return launch_skinny(a, nullptr) == W4A16_OK ? 1 : 0;
}

extern "C" int w4a16_gemm_allreduce(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                                    void* out, int tokens, int N, int K, int group_size, int k_config,
                                    void* const* buffers, int world, int rank, size_t capacity_elems, void* stream,
                                    unsigned flags)
{
    return w4a16_gemm_allreduce_residual(x, qweight, zeros_scales, bias, nullptr, out, nullptr, tokens, N, K, group_size, k_config,
                                         buffers, world, rank, capacity_elems, stream, flags);
}

extern "C" int w4a16_exchange_allgather(const void* in, void* out, int words, void* const* buffers, int world, int rank,
                                        size_t capacity_elems, void* stream)
{
    if (!in || !out || !buffers) return W4A16_ERR_NULL_POINTER;
    if (words <= 0 || world < 1 || world > kExchangeMaxWorld || rank < 0 || rank >= world) return W4A16_ERR_BAD_SHAPE;
    if ((size_t)words > capacity_elems) return W4A16_ERR_TOO_LARGE;
    GatherParams p;
    for (int d = 0; d < kExchangeMaxWorld; ++d) {
        p.peer[d] = d < world ? (unsigned char*)buffers[d] : nullptr;
        if (d < world && !p.peer[d]) return W4A16_ERR_NULL_POINTER;
    }
    p.self = p.peer[rank];
    p.in = (const unsigned*)in; p.out = (unsigned*)out;
    p.error = device_error_word();
    if (!p.error) return W4A16_ERR_CUDA;
    p.words = words; p.world = world; p.rank = rank; p.capacity = (long long)capacity_elems;
    p.wait_budget_ns = exchange_wait_budget_ns();
    cudaError_t e = launch_after_previous(exchange_allgather_kernel, dim3(1), dim3(256), 0, (cudaStream_t)stream, p);
    count_launch();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}
