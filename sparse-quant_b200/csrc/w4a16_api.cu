// C-ABI entry points: argument validation, kernel selection, error bookkeeping.
#include <atomic>

#include "w4a16_common.cuh"

namespace w4a16 {

namespace {
thread_local int t_last_cuda_error = 0;
std::atomic<unsigned long long> g_launches{0};
}  // namespace

int record_cuda_error(cudaError_t e)
{
    t_last_cuda_error = (int)e;
    (void)cudaGetLastError();   // clear the sticky-free error so later calls start clean
    return W4A16_ERR_CUDA;
}

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void skinny_force_config(int wn, int splits);
void tc_force_config(int tile_tokens, int split_k);

namespace {

int validate(const void* x, const void* qw, const void* zs, const void* out, int tokens, int N, int K, int g)
{
    if (g != 32 && g != 64 && g != 128) return W4A16_ERR_GROUP_SIZE;
    if (tokens < 0 || N <= 0 || K <= 0 || (N % 32) || (K % g)) return W4A16_ERR_BAD_SHAPE;
    if ((long long)tokens * N >= (1ll << 40) || (long long)tokens * K >= (1ll << 40)) return W4A16_ERR_BAD_SHAPE;
    if (tokens == 0) return W4A16_OK;
    if (!x || !qw || !zs || !out) return W4A16_ERR_NULL_POINTER;
    if (((uintptr_t)x & 15) || ((uintptr_t)qw & 15) || ((uintptr_t)zs & 15) || ((uintptr_t)out & 15)) return W4A16_ERR_MISALIGNED;
    return W4A16_OK;
}

int check_device()
{
    static std::atomic<int> ok_mask[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 64 && ok_mask[dev].load(std::memory_order_relaxed) == 1) return W4A16_OK;
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (major != 10) return W4A16_ERR_UNSUPPORTED_GPU;
    if (dev < 64) ok_mask[dev].store(1, std::memory_order_relaxed);
    return W4A16_OK;
}

}  // namespace
}  // namespace w4a16

using namespace w4a16;

extern "C" const char* w4a16_status_str(int status)
{
    switch (status) {
        case W4A16_OK: return "success";
        case W4A16_ERR_NULL_POINTER: return "a required pointer is NULL";
        case W4A16_ERR_BAD_SHAPE: return "bad shape: need N % 32 == 0, K % group_size == 0, sizes >= 0";
        case W4A16_ERR_GROUP_SIZE: return "unsupported group size";
        case W4A16_ERR_MISALIGNED: return "pointer is not sufficiently aligned (16 bytes for x, qweight, zeros_scales, out)";
        case W4A16_ERR_WORKSPACE: return "workspace is NULL or smaller than w4a16_workspace_bytes()";
        case W4A16_ERR_BAD_ALGO: return "unknown algo id or algo cannot run this shape";
        case W4A16_ERR_CUDA: return "a CUDA call failed (see w4a16_last_cuda_error)";
        case W4A16_ERR_UNSUPPORTED_GPU: return "device is not compute capability 10.x (B200)";
        case W4A16_ERR_TOO_LARGE: return "size exceeds a fixed capacity of this entry point";
        default: return "unknown status";
    }
}

extern "C" int w4a16_last_cuda_error(void) { return t_last_cuda_error; }

extern "C" unsigned long long w4a16_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int w4a16_version(void) { return 100; }

extern "C" size_t w4a16_workspace_bytes(int tokens, int N, int K, int group_size)
{
    if (tokens <= 32 || N <= 0 || K <= 0) return 0;
    return tc_workspace_bytes(tokens, N, K, group_size);
}

extern "C" int w4a16_gemm_algo(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                               void* out, int tokens, int N, int K, int group_size, void* workspace,
                               size_t workspace_bytes, void* stream, int algo)
{
    int s = validate(x, qweight, zeros_scales, out, tokens, N, K, group_size);
    if (s != W4A16_OK) return s;
    if (algo != W4A16_ALGO_AUTO && algo != W4A16_ALGO_SKINNY && algo != W4A16_ALGO_TC) return W4A16_ERR_BAD_ALGO;
    if (tokens == 0) return W4A16_OK;
    s = check_device();
    if (s != W4A16_OK) return s;

    GemmArgs a;
    a.x = (const __half*)x; a.qw = (const uint32_t*)qweight; a.zs = (const uint32_t*)zeros_scales;
    a.bias = (const __half*)bias; a.out = (__half*)out;
    a.tokens = tokens; a.N = N; a.K = K; a.g = group_size;

    if (algo == W4A16_ALGO_AUTO) algo = (tokens <= 32 || !tc_supported(tokens, N, K, group_size)) ? W4A16_ALGO_SKINNY : W4A16_ALGO_TC;
    if (algo == W4A16_ALGO_TC) {
        if (!tc_supported(tokens, N, K, group_size)) return W4A16_ERR_BAD_ALGO;
        return launch_tc(a, workspace, workspace_bytes, (cudaStream_t)stream);
    }
    return launch_skinny(a, (cudaStream_t)stream);
}

extern "C" int w4a16_gemm(const void* x, const void* qweight, const void* zeros_scales, const void* bias, void* out,
                          int tokens, int N, int K, int group_size, void* workspace, size_t workspace_bytes, void* stream)
{
    return w4a16_gemm_algo(x, qweight, zeros_scales, bias, out, tokens, N, K, group_size, workspace, workspace_bytes,
                           stream, W4A16_ALGO_AUTO);
}

extern "C" int w4a16_gemm_host(const void* x_host, void* out_host, void* x_dev, void* out_dev, const void* qweight,
                               const void* zeros_scales, const void* bias, int tokens, int N, int K, int group_size,
                               void* workspace, size_t workspace_bytes, void* stream)
{
    if (tokens < 0) return W4A16_ERR_BAD_SHAPE;
    if (tokens == 0) return W4A16_OK;
    if (!x_host || !out_host || !x_dev || !out_dev) return W4A16_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(x_dev, x_host, (size_t)tokens * K * sizeof(__half), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return record_cuda_error(e);
    int s = w4a16_gemm(x_dev, qweight, zeros_scales, bias, out_dev, tokens, N, K, group_size, workspace, workspace_bytes, stream);
    if (s != W4A16_OK) return s;
    e = cudaMemcpyAsync(out_host, out_dev, (size_t)tokens * N * sizeof(__half), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return record_cuda_error(e);
    e = cudaStreamSynchronize(st);
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

// Tuning hooks for benchmarks (0 = automatic).  Not part of the drop-in surface.
extern "C" void w4a16_tune_skinny(int wn, int splits) { skinny_force_config(wn, splits); }
extern "C" void w4a16_tune_tc(int tile_tokens, int split_k) { tc_force_config(tile_tokens, split_k); }
