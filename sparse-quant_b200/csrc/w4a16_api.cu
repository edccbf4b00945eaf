// C-ABI entry points: argument validation, kernel selection, error bookkeeping.
#include <atomic>
#include <mutex>

#include <cuda.h>

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

namespace { std::atomic<int> g_aux_programmatic{0}; }
bool aux_programmatic_launch() { return g_aux_programmatic.load(std::memory_order_relaxed) != 0; }

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int device_sm_count()
{
    static int cache[64] = {};         // benign race: the query is idempotent
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { (void)cudaGetLastError(); return 148; }
    if (!cache[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) { (void)cudaGetLastError(); v = 148; }
        cache[dev] = v;
    }
    return cache[dev];
}

// Allocated once per device (first use; outside stream capture), never freed.  Word 0 is the error word (only ever
// raised by kernels, cleared by w4a16_device_error_clear); word 1 is a generation counter the decode kernel bumps.
int* device_error_word()
{
    static int* words[64] = {nullptr};
    static std::mutex lock;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> guard(lock);
    if (!words[dev]) {
        int* p = nullptr;
        if (cudaMalloc(&p, 64) != cudaSuccess) return nullptr;
        if (cudaMemset(p, 0, 64) != cudaSuccess) return nullptr;
        words[dev] = p;
    }
    return words[dev];
}

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn()
{
    static std::atomic<EncodeTiledFn> fn{nullptr};
    EncodeTiledFn f = fn.load(std::memory_order_acquire);
    if (!f) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            f = (EncodeTiledFn)sym;
            fn.store(f, std::memory_order_release);
        }
    }
    return f;
}
}  // namespace

int encode_tensor_map_2d(void* tmap, const void* base, int elem_bytes, const uint64_t dims[2], uint64_t row_stride_bytes,
                         const uint32_t box[2], bool swizzle128)
{
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return record_cuda_error(cudaErrorNotSupported);
    const cuuint64_t gdims[2] = {dims[0], dims[1]};
    const cuuint64_t gstr[1] = {row_stride_bytes};
    const cuuint32_t gbox[2] = {box[0], box[1]};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    CUresult r = encode((CUtensorMap*)tmap, dt, 2, const_cast<void*>(base), gdims, gstr, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? W4A16_OK : record_cuda_error(cudaErrorInvalidValue);
}

void skinny_force_config(int wn, int splits);
void skinny_set_timeline(unsigned long long* buf);
void gemv_force_config(int tn, int splits, int depth);
void gemv_set_timeline(unsigned long long* buf);
void decode_force_kernel(int which);
int gemv_plan(int tokens, int N, int K, int g, int* plan);
void gemv_force_ahead(int units);
void tc_force_config(int tile_tokens, int split_k);
void tc_set_account(unsigned long long* buf);

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

extern "C" int w4a16_gemm_fused(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                                const void* residual, void* out, int tokens, int N, int K, int group_size, void* workspace,
                                size_t workspace_bytes, void* stream, int algo, unsigned flags)
{
    int s = validate(x, qweight, zeros_scales, out, tokens, N, K, group_size);
    if (s != W4A16_OK) return s;
    if (algo != W4A16_ALGO_AUTO && algo != W4A16_ALGO_SKINNY && algo != W4A16_ALGO_TC) return W4A16_ERR_BAD_ALGO;
    if (flags & ~(unsigned)(W4A16_FLAG_STATIC_WEIGHTS | W4A16_FLAG_RELU | W4A16_FLAG_SILU_MUL)) return W4A16_ERR_BAD_ALGO;
    if (tokens == 0) return W4A16_OK;
    if (residual && ((uintptr_t)residual & 1)) return W4A16_ERR_MISALIGNED;
    s = check_device();
    if (s != W4A16_OK) return s;

    GemmArgs a;
    a.x = (const __half*)x; a.qw = (const uint32_t*)qweight; a.zs = (const uint32_t*)zeros_scales;
    a.bias = (const __half*)bias; a.out = (__half*)out; a.residual = (const __half*)residual;
    a.tokens = tokens; a.N = N; a.K = K; a.g = group_size;
    a.static_weights = (flags & W4A16_FLAG_STATIC_WEIGHTS) != 0;
    a.relu = (flags & W4A16_FLAG_RELU) != 0;
    a.silu_mul = (flags & W4A16_FLAG_SILU_MUL) != 0;

    if (algo == W4A16_ALGO_AUTO) algo = (tokens <= 32 || !tc_supported(tokens, N, K, group_size)) ? W4A16_ALGO_SKINNY : W4A16_ALGO_TC;
    if (a.silu_mul) {
        // the SwiGLU epilogue lives in the decode kernels (one pass of at most 32 tokens); larger inputs use
        // w4a16_silu_mul on the plain output
        if (algo != W4A16_ALGO_SKINNY || tokens > 32 || (N % 64) || residual) return W4A16_ERR_BAD_ALGO;
    }
    if (algo == W4A16_ALGO_TC) {
        if (!tc_supported(tokens, N, K, group_size)) return W4A16_ERR_BAD_ALGO;
        return launch_tc(a, workspace, workspace_bytes, (cudaStream_t)stream);
    }
    return launch_skinny(a, (cudaStream_t)stream);
}

extern "C" size_t w4a16_row_stats_bytes(int N)
{
    // header + one part per CTA of the producing grid (at most one per 32 out-features and K split) x 16 rows x 2 floats
    return N <= 0 ? 0 : (size_t)(4 + (size_t)((N + 31) / 32) * 8 * 16 * 2) * sizeof(float);
}

extern "C" int w4a16_gemm_prenorm(const void* x, const void* row_stats, const void* norm_weight, const void* norm_bias,
                                  float eps, int rms, const void* qweight, const void* zeros_scales, const void* bias,
                                  void* out, int tokens, int N, int K, int group_size, void* stream, unsigned flags)
{
    int s = validate(x, qweight, zeros_scales, out, tokens, N, K, group_size);
    if (s != W4A16_OK) return s;
    if (!norm_weight || !row_stats) return W4A16_ERR_NULL_POINTER;
    if (((uintptr_t)norm_weight & 15) || ((uintptr_t)norm_bias & 15) || ((uintptr_t)row_stats & 15)) return W4A16_ERR_MISALIGNED;
    if (flags & ~(unsigned)(W4A16_FLAG_STATIC_WEIGHTS | W4A16_FLAG_RELU | W4A16_FLAG_SILU_MUL)) return W4A16_ERR_BAD_ALGO;
    if ((flags & W4A16_FLAG_SILU_MUL) && (N % 64)) return W4A16_ERR_BAD_ALGO;
    if (tokens == 0) return W4A16_OK;
    s = check_device();
    if (s != W4A16_OK) return s;
    GemmArgs a;
    a.x = (const __half*)x; a.qw = (const uint32_t*)qweight; a.zs = (const uint32_t*)zeros_scales;
    a.bias = (const __half*)bias; a.out = (__half*)out;
    a.tokens = tokens; a.N = N; a.K = K; a.g = group_size;
    a.static_weights = (flags & W4A16_FLAG_STATIC_WEIGHTS) != 0;
    a.relu = (flags & W4A16_FLAG_RELU) != 0;
    a.silu_mul = (flags & W4A16_FLAG_SILU_MUL) != 0;
    a.norm_weight = (const __half*)norm_weight; a.norm_bias = (const __half*)norm_bias; a.norm_eps = eps; a.norm_rms = rms != 0;
    a.row_stats_in = (const float*)row_stats;
    return launch_skinny(a, (cudaStream_t)stream);       // W4A16_ERR_BAD_ALGO beyond 16 tokens
}

extern "C" int w4a16_gemm_residual_stats(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                                         const void* residual, void* out, void* row_stats_out, int tokens, int N, int K,
                                         int group_size, void* stream, unsigned flags)
{
    int s = validate(x, qweight, zeros_scales, out, tokens, N, K, group_size);
    if (s != W4A16_OK) return s;
    if (!row_stats_out) return W4A16_ERR_NULL_POINTER;
    if (((uintptr_t)row_stats_out & 15) || ((uintptr_t)residual & 1)) return W4A16_ERR_MISALIGNED;
    if (flags & ~(unsigned)(W4A16_FLAG_STATIC_WEIGHTS | W4A16_FLAG_RELU)) return W4A16_ERR_BAD_ALGO;
    if (tokens == 0) return W4A16_OK;
    s = check_device();
    if (s != W4A16_OK) return s;
    GemmArgs a;
    a.x = (const __half*)x; a.qw = (const uint32_t*)qweight; a.zs = (const uint32_t*)zeros_scales;
    a.bias = (const __half*)bias; a.out = (__half*)out; a.residual = (const __half*)residual;
    a.tokens = tokens; a.N = N; a.K = K; a.g = group_size;
    a.static_weights = (flags & W4A16_FLAG_STATIC_WEIGHTS) != 0;
    a.relu = (flags & W4A16_FLAG_RELU) != 0;
    a.row_stats_out = (float*)row_stats_out;
    return launch_skinny(a, (cudaStream_t)stream);       // W4A16_ERR_BAD_ALGO beyond 16 tokens
}

extern "C" int w4a16_gemm_ex(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                             void* out, int tokens, int N, int K, int group_size, void* workspace,
                             size_t workspace_bytes, void* stream, int algo, unsigned flags)
{
    if (flags & W4A16_FLAG_SILU_MUL) return W4A16_ERR_BAD_ALGO;      // changes the output shape: w4a16_gemm_fused only
    return w4a16_gemm_fused(x, qweight, zeros_scales, bias, nullptr, out, tokens, N, K, group_size, workspace, workspace_bytes,
                            stream, algo, flags);
}

extern "C" int w4a16_gemm_algo(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                               void* out, int tokens, int N, int K, int group_size, void* workspace,
                               size_t workspace_bytes, void* stream, int algo)
{
    return w4a16_gemm_ex(x, qweight, zeros_scales, bias, out, tokens, N, K, group_size, workspace, workspace_bytes, stream,
                         algo, 0u);
}

extern "C" int w4a16_gemm(const void* x, const void* qweight, const void* zeros_scales, const void* bias, void* out,
                          int tokens, int N, int K, int group_size, void* workspace, size_t workspace_bytes, void* stream)
{
    return w4a16_gemm_algo(x, qweight, zeros_scales, bias, out, tokens, N, K, group_size, workspace, workspace_bytes,
                           stream, W4A16_ALGO_AUTO);
}

namespace {
int gemm_host_impl(const void* x_host, void* out_host, void* x_dev, void* out_dev, const void* qweight,
                   const void* zeros_scales, const void* bias, int tokens, int N, int K, int group_size,
                   void* workspace, size_t workspace_bytes, void* stream, bool sync)
{
    if (!x_host || !out_host || !x_dev || !out_dev) return tokens == 0 ? W4A16_OK : W4A16_ERR_NULL_POINTER;
    // every argument is checked before the first copy is enqueued
    int v = validate(x_dev, qweight, zeros_scales, out_dev, tokens, N, K, group_size);
    if (v != W4A16_OK) return v;
    if (tokens == 0) return W4A16_OK;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(x_dev, x_host, (size_t)tokens * K * sizeof(__half), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return record_cuda_error(e);
    int s = w4a16_gemm(x_dev, qweight, zeros_scales, bias, out_dev, tokens, N, K, group_size, workspace, workspace_bytes, stream);
    if (s != W4A16_OK) return s;
    e = cudaMemcpyAsync(out_host, out_dev, (size_t)tokens * N * sizeof(__half), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (!sync) return W4A16_OK;
    e = cudaStreamSynchronize(st);
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}
}  // namespace

extern "C" int w4a16_gemm_host(const void* x_host, void* out_host, void* x_dev, void* out_dev, const void* qweight,
                               const void* zeros_scales, const void* bias, int tokens, int N, int K, int group_size,
                               void* workspace, size_t workspace_bytes, void* stream)
{
    return gemm_host_impl(x_host, out_host, x_dev, out_dev, qweight, zeros_scales, bias, tokens, N, K, group_size, workspace,
                          workspace_bytes, stream, true);
}

extern "C" int w4a16_gemm_host_async(const void* x_host, void* out_host, void* x_dev, void* out_dev, const void* qweight,
                                     const void* zeros_scales, const void* bias, int tokens, int N, int K, int group_size,
                                     void* workspace, size_t workspace_bytes, void* stream)
{
    return gemm_host_impl(x_host, out_host, x_dev, out_dev, qweight, zeros_scales, bias, tokens, N, K, group_size, workspace,
                          workspace_bytes, stream, false);
}

extern "C" int w4a16_device_error_flag(int* flag)
{
    if (!flag) return W4A16_ERR_NULL_POINTER;
    int* w = device_error_word();
    if (!w) return W4A16_ERR_CUDA;
    cudaError_t e = cudaMemcpy(flag, w, sizeof(int), cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

extern "C" int w4a16_device_error_clear(void)
{
    int* w = device_error_word();
    if (!w) return W4A16_ERR_CUDA;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemset(w, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

// Tuning hooks for benchmarks (0 = automatic).  Not part of the drop-in surface.
extern "C" void w4a16_tune_skinny(int wn, int splits) { skinny_force_config(wn, splits); }
extern "C" void w4a16_tune_decode(int kernel, int tiles_per_cta, int splits, int depth)
{
    decode_force_kernel(kernel);
    gemv_force_config(tiles_per_cta, splits, depth);
}
extern "C" void w4a16_tune_decode_prefetch(int units_ahead) { gemv_force_ahead(units_ahead); }
extern "C" int w4a16_debug_decode_plan(int tokens, int N, int K, int group_size, int* plan9)
{
    if (!plan9) return W4A16_ERR_NULL_POINTER;
    return gemv_plan(tokens, N, K, group_size, plan9);
}
// Debug aid: device buffer [ctas][16 warps][8] receiving %globaltimer stamps of the decode kernels' phases (NULL = off).
extern "C" void w4a16_debug_skinny_timeline(void* buf)
{
    skinny_set_timeline((unsigned long long*)buf);
    gemv_set_timeline((unsigned long long*)buf);
    tc_set_account((unsigned long long*)buf);
}
extern "C" void w4a16_tune_tc(int tile_tokens, int split_k) { tc_force_config(tile_tokens, split_k); }
// 1: the small decode-step kernels (attention, add+norm, SwiGLU product, exchange all-gather) are launched with
// programmatic stream serialization; 0 (default): plain stream order - measured faster (OPT-6.7B-shaped step 1.8 %,
// LLaMA-2-7B-shaped step 7 %): their early-resident CTAs only compete with the kernel they wait for.
extern "C" void w4a16_tune_aux_launch(int programmatic) { g_aux_programmatic.store(programmatic ? 1 : 0, std::memory_order_relaxed); }
