/*
 * w4a16_b200 — C ABI of the B200 (sm_100a) W4A16 group-quantised linear layer.
 *
 * Drop-in boundary for the `quant` extension of sparklesea/sparse-quant
 * (quantization/nvidia/kernel).  Each entry point names the reference interface it
 * replaces.  All pointers are DEVICE pointers unless stated otherwise, all tensors are
 * dense and row-major, `stream` is a cudaStream_t passed as void* (NULL = legacy default
 * stream).  Every function returns a w4a16_status (0 = success) and never throws; nothing
 * is launched when the status is an argument error.  Launches are asynchronous.
 *
 * Tensor formats (identical to the reference's):
 *   qweight       int32  [K, N/8]      TurboMind "s4_k_m8" tile order, physically
 *                                      [K/32][N/32][32 lanes][4 words] (512 B per 32x32 tile)
 *   zeros_scales  fp16   [K/g, 2N]     per (group, out-feature) the pair (zero + 64, scale)
 *   x             fp16   [tokens, K]
 *   out           fp16   [tokens, N]
 *   bias          fp16   [N] or NULL
 * Constraints: N % 32 == 0, K % g == 0, g in {32, 64, 128}, tokens >= 0; x, qweight,
 * zeros_scales and out 16-byte aligned.  The tcgen05 kernel additionally needs g in {64, 128};
 * W4A16_ALGO_AUTO falls back to the skinny kernel otherwise.
 */
#ifndef W4A16_B200_H_
#define W4A16_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum w4a16_status {
    W4A16_OK                  = 0,
    W4A16_ERR_NULL_POINTER    = 1,  /* a required pointer is NULL */
    W4A16_ERR_BAD_SHAPE       = 2,  /* N % 32 != 0, K % g != 0, negative size, size overflow */
    W4A16_ERR_GROUP_SIZE      = 3,  /* "unsupported group size" (gemm_s4_f16.cu:232-234) */
    W4A16_ERR_MISALIGNED      = 4,  /* pointer not 16-byte aligned where vector access needs it */
    W4A16_ERR_WORKSPACE       = 5,  /* workspace missing or smaller than w4a16_workspace_bytes() */
    W4A16_ERR_BAD_ALGO        = 6,  /* unknown algo id, or algo cannot run this shape */
    W4A16_ERR_CUDA            = 7,  /* a CUDA runtime/driver call failed (see w4a16_last_cuda_error) */
    W4A16_ERR_UNSUPPORTED_GPU = 8,  /* device is not compute capability 10.x */
    W4A16_ERR_TOO_LARGE       = 9   /* size beyond a stated fixed capacity */
} w4a16_status;

/* kernel selection for w4a16_gemm_algo */
typedef enum w4a16_algo {
    W4A16_ALGO_AUTO   = 0,  /* tokens <= 32: decode kernels; otherwise the tcgen05 kernel */
    W4A16_ALGO_SKINNY = 1,  /* mma.sync decode kernels (up to 8 tokens: two CTAs per SM; up to 32: cluster split-K) */
    W4A16_ALGO_TC     = 2   /* TMA + tcgen05/TMEM GEMM (prefill) */
} w4a16_algo;

/* Human readable text for a status code (static storage, never NULL). */
const char* w4a16_status_str(int status);

/* cudaError_t of the most recent failing CUDA call made by this library on the calling
 * thread (0 if none). */
int w4a16_last_cuda_error(void);

/*
 * out[t, n] = fp16( sum_k fp32( dequant(qweight)[n, k] * x[t, k] ) ) (+ bias[n], fp16 add)
 *
 * Replaces gemm_awq_ut / Gemm_awq_pure / gemm_awq_api (kernel/gemm_quant.cu:98-122,42-96,
 * 13-40, declared kernel/gemm_quant.h:15-17) and the fp16 bias add of WALinear.forward
 * (test/nvidia/module/qlinear/qlinear.py:69-70), which is fused here.  Unlike the
 * reference the launch goes to `stream`, g may be 32/64/128 and any N % 32 == 0 is
 * accepted.  `workspace` may be NULL when w4a16_workspace_bytes() returns 0.
 */
int w4a16_gemm(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
               void* out, int tokens, int N, int K, int group_size,
               void* workspace, size_t workspace_bytes, void* stream);

/* Same as w4a16_gemm with an explicit kernel choice (tests and benchmarks). */
int w4a16_gemm_algo(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                    void* out, int tokens, int N, int K, int group_size,
                    void* workspace, size_t workspace_bytes, void* stream, int algo);

/*
 * w4a16_gemm_algo plus flags.  W4A16_FLAG_STATIC_WEIGHTS promises that qweight, zeros_scales and
 * bias were completely written before any work still in flight on `stream` was enqueued (true
 * for the buffers of a loaded module; NOT true right after running the packer on the same
 * stream).  The decode kernel is then launched with programmatic stream serialization: it
 * starts fetching weights while the previous kernel of the stream drains, and waits for that
 * kernel to complete before it reads x or writes out.  No counterpart in the reference.
 * W4A16_FLAG_RELU clamps the outputs at zero after the bias add: the ReLU that follows fc1 in the reference's OPT
 * layer (modeling_opt_ours.py:606, activation_fn) without a launch of its own.
 */
#define W4A16_FLAG_STATIC_WEIGHTS 1u
#define W4A16_FLAG_RELU 2u
int w4a16_gemm_ex(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                  void* out, int tokens, int N, int K, int group_size,
                  void* workspace, size_t workspace_bytes, void* stream, int algo, unsigned flags);

/*
 * w4a16_gemm_ex with the epilogues the reference carries as hooks around its kernel (its test script calls them
 * gemm_awq_residual_ut and gemm_awq_silu_dot_ut, quantization/nvidia/script/gemm_awq_test.py:63-72; the kernel side
 * is ops::SiluActivation, kernel/gemm_s4_f16/gemm_s4_f16.cu:30-40, over weights interleaved by fuse_w1_w3_s4_k_m8,
 * format.cu:114-120):
 *   residual (fp16 [tokens, N] or NULL): out = (fp16(acc) + bias) + residual, both adds in fp16 - the `x + linear(h)`
 *     of a decoder block without a launch of its own; every kernel takes it;
 *   W4A16_FLAG_SILU_MUL: the packed matrix holds the gate and up projections of a SwiGLU block with their 32-wide
 *     out-feature tiles alternating (tile 2j = gate tile j, tile 2j+1 = up tile j; w4a16.tp.fuse_gate_up builds it in
 *     the packed domain); out is fp16 [tokens, N/2], out[t, j] = fp16(silu(gate[t, j])) * up[t, j] with gate and up
 *     rounded to fp16 (+ bias) first, i.e. the roundings of act_fn(gate_proj(x)) * up_proj(x).  Decode kernels only
 *     (tokens <= 32, N % 64 == 0, no residual); W4A16_ERR_BAD_ALGO otherwise - use w4a16_silu_mul on the plain output.
 */
#define W4A16_FLAG_SILU_MUL 4u
int w4a16_gemm_fused(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                     const void* residual, void* out, int tokens, int N, int K, int group_size,
                     void* workspace, size_t workspace_bytes, void* stream, int algo, unsigned flags);

/* Scratch bytes w4a16_gemm needs for this problem (0 = none).  The reference has no
 * workspace (the WorkSpace argument of Gemm_awq_pure, gemm_quant.cu:45, is unused). */
size_t w4a16_workspace_bytes(int tokens, int N, int K, int group_size);

/*
 * w[n, k] = mul.ftz.f16( sub.ftz.f16( 64 + q[n,k], zero[n,k/g] + 64 ), scale[n,k/g] )
 * written as fp16 [N, K] (the orientation of nn.Linear.weight), bit-exact with the
 * in-kernel dequantisation of the reference (dequantize_s4_to_fp16x2_v2 + apply_Q,
 * kernel/gemm_s4_f16/common.h:114-153,210-225).  The NVIDIA reference binds no such op;
 * the name and argument order follow the `dequant` op of its sibling backend
 * (quantization/tianshu/backend/pybind.cpp:12).
 */
int w4a16_dequant(const void* qweight, const void* zeros_scales, void* w_out,
                  int N, int K, int group_size, void* stream);

/*
 * zeros_scales[k/g][n] = half2(zeros[n][k/g] + 64, scales[n][k/g]).
 * Replaces transpose_merge_zeros_scales (kernel/gemm_s4_f16/format.cu:206-239,
 * declared kernel/gemm_quant.h:19-24).  zeros, scales: fp16 [N, K/g].
 */
int w4a16_transpose_merge_zeros_scales(const void* zeros, const void* scales, void* zeros_scales,
                                       int in_features, int out_features, int group_size, void* stream);

/*
 * uint8 [N, K/2] (byte = q[n,2i] << 4 | q[n,2i+1]) -> uint32 [K, N/8] AWQ nibble order.
 * Replaces convert_ours_to_awq (format.cu:151-201, declared gemm_quant.h:26-29).
 */
int w4a16_convert_ours_to_awq(const void* qweight_src, void* qweight_dst,
                              int in_features, int out_features, void* stream);

/*
 * AWQ uint32 [K, N/8] -> TurboMind tile order int32 [K, N/8].  Replaces
 * convert_awq_to_lmdeploy -> convert_s4_k_m8 -> reformat_s4_k_m8 -> permute_u4
 * (format.cu:135-149,90-105,66-71,24-57, declared gemm_quant.h:31-33).  Needs K % 32 == 0
 * and N % 32 == 0.
 */
int w4a16_convert_awq_to_lmdeploy(const void* qweight_src, void* qweight_dst,
                                  int in_features, int out_features, void* stream);

/*
 * Quantise and pack in one pass: fp16 weight [N, K] -> qweight int32 [K, N/8] (tile order) and zeros_scales fp16
 * [K/g, 2N], bit-identical to the reference's flow quant_lmdeploy (test/nvidia/utils/quant_dequant_nvidia.py:5-32):
 * quantize_tensor (:124-148, per-group asymmetric min-max in fp16, torch.round = half to even) + write_4bit_tensor
 * (:79-88) + transpose_merge_zeros_scales + convert_ours_to_awq + convert_awq_to_lmdeploy (format.cu:206-239,
 * 151-201, 135-149).  Optional outputs (NULL to skip): w_fp16 [N, K] = (q - zero) * scale as the quantizer returns
 * it, zeros / scales fp16 [N, K/g] and the "ours" bytes uint8 [N, K/2] (byte = q[n,2i] << 4 | q[n,2i+1]) that
 * generate_quant (:103-122) returns.  g in {32, 64, 128}, N % 32 == 0, K % g == 0; weight and w_fp16 8-byte aligned.
 */
int w4a16_quantize_pack(const void* weight, void* qweight, void* zeros_scales, void* w_fp16, void* zeros,
                        void* scales, void* qweight_ours, int in_features, int out_features, int group_size,
                        void* stream);

/*
 * The same GEMM through HOST buffers: copies x (and nothing else) host->device, runs
 * w4a16_gemm on `stream`, copies out device->host and synchronises the stream.  The
 * packed weights stay resident on the device, as they do in the reference's WALinear
 * module (qlinear.py:26-34).  `x_dev`/`out_dev` are caller-provided device staging
 * buffers of tokens*K and tokens*N fp16.  For pinned host memory the copies are
 * asynchronous on `stream`.
 */
int w4a16_gemm_host(const void* x_host, void* out_host, void* x_dev, void* out_dev,
                    const void* qweight, const void* zeros_scales, const void* bias,
                    int tokens, int N, int K, int group_size,
                    void* workspace, size_t workspace_bytes, void* stream);

/* The same without the final synchronisation: enqueues copy-in, GEMM and copy-out on `stream` and returns; the
 * caller synchronises the stream (once for a whole batch of calls) before reading `out_host`.  Host buffers must be
 * pinned for the copies to be asynchronous. */
int w4a16_gemm_host_async(const void* x_host, void* out_host, void* x_dev, void* out_dev,
                    const void* qweight, const void* zeros_scales, const void* bias,
                    int tokens, int N, int K, int group_size,
                    void* workspace, size_t workspace_bytes, void* stream);

/*
 * Decode GEMV fused with the all-reduce of a row-parallel linear (tensor parallelism; no counterpart in the
 * reference, which is single-GPU: it stands where a sharded WALinear.forward, qlinear.py:58-72, would be followed
 * by an all-reduce).  Rank `rank` of `world` (<= 8, one process per GPU, all GPUs peer-accessible) holds the K
 * shard [K of this call] of the packed weight; every rank calls this with its own shard and the same tokens (<= 32),
 * N, group_size, k_config (the largest K shard over the ranks: all ranks must launch the same shape) and bias
 * (added once, after the sum).  out = fp16(sum over ranks of x_r W_r^T) + bias on EVERY rank, bit-identical across
 * ranks; partial sums cross NVLink in fp32.
 *
 * Exchange buffers: each rank allocates one (w4a16_exchange_alloc; capacity_elems >= tokens * N of any call that
 * uses it), exports a 64-byte handle (w4a16_exchange_export), the host program moves the handles between the
 * processes, and each rank opens its peers' handles (w4a16_exchange_open).  `buffers[r]` is rank r's buffer as
 * mapped in the calling process (own allocation at index `rank`).  Calls that use the same buffers must be issued
 * in the same order on every rank and must not overlap on one GPU (use one stream).  A rank whose peers do not
 * show up within 2 s gives up: the library's device error word (w4a16_device_error_flag) and the buffer's error
 * field (w4a16_exchange_status) are set and the output of that call is undefined; the kernel still returns.
 * Allocates nothing per call and contains no library collective, so a stream capture can record it.
 */
size_t w4a16_exchange_bytes(int world, size_t capacity_elems);
int w4a16_exchange_alloc(int world, size_t capacity_elems, void** buffer);
int w4a16_exchange_free(void* buffer);
int w4a16_exchange_export(void* buffer, void* handle64);
int w4a16_exchange_open(const void* handle64, void** peer_buffer);
int w4a16_exchange_close(void* peer_buffer);
int w4a16_exchange_status(const void* buffer, unsigned* epoch, int* error);
/* All-gather of `words` 32-bit words per rank through the same buffers and protocol (one small kernel):
 * out[r * words + i] = rank r's in[i].  For what a decode step exchanges besides the row-parallel sums, e.g. each
 * rank's best logit of its vocabulary shard. */
int w4a16_exchange_allgather(const void* in, void* out, int words, void* const* buffers, int world, int rank,
                             size_t capacity_elems, void* stream);
/* 1 if w4a16_gemm_allreduce(_residual) takes this problem on the current device (at most 32 tokens in one pass whose
 * grid fits the GPU in one wave), else 0: decide between the fused exchange and a library all-reduce from the shapes,
 * identically on every rank. */
int w4a16_allreduce_supported(int tokens, int N, int K, int k_config, int group_size, int world);
int w4a16_gemm_allreduce(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                         void* out, int tokens, int N, int K, int group_size, int k_config,
                         void* const* buffers, int world, int rank, size_t capacity_elems, void* stream,
                         unsigned flags);
/* The same with `residual` (fp16 [tokens, N], the same values on every rank, or NULL) added once to the summed
 * output after bias / ReLU: the residual add that follows a row-parallel out_proj / fc2.  row_stats_out != NULL
 * (tokens <= 16): the row statistics of the output for w4a16_gemm_prenorm, see there. */
int w4a16_gemm_allreduce_residual(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                                  const void* residual, void* out, void* row_stats_out, int tokens, int N, int K,
                                  int group_size, int k_config, void* const* buffers, int world, int rank,
                                  size_t capacity_elems, void* stream, unsigned flags);

/*
 * Decode attention over a static key/value cache: one new token per sequence, one launch.  Replaces, for the
 * decode step, the reference's torch ops around its quantised projections: torch.cat of the new key/value onto the
 * cache (modeling_opt_ours.py:249-250), bmm(q, K^T) (:306), mask + softmax, bmm(P, V) (:456) and the
 * transpose/reshape before out_proj.
 *   qkv      fp16 [batch, qkv_stride], row b = [q (heads*head_dim) | k (heads*head_dim) | v (heads*head_dim)]: the output
 *            of the q/k/v projections fused into one GEMV (unscaled q)
 *   k_cache, v_cache  fp16 [batch, heads, max_len, head_dim]; row *pos is written, rows 0..*pos are read
 *   out      fp16 [batch, heads*head_dim]
 *   pos      device pointer to one int64: index of the new token (0 <= *pos < max_len, else the device error word is
 *            set to 3 and nothing is written)
 *   rope_cos, rope_sin  fp16 [>= *pos+1, head_dim] rotary tables ("rotate half" convention) or both NULL
 *   scale    multiplies q.k (head_dim^-0.5 in both OPT and LLaMA)
 * head_dim 64 or 128.  Scores, softmax and the weighted sum are fp32; outputs are rounded to fp16 once.
 */
int w4a16_decode_attention(const void* qkv, void* k_cache, void* v_cache, void* out, const void* pos,
                           const void* rope_cos, const void* rope_sin, int batch, int heads, int head_dim,
                           int max_len, int qkv_stride, float scale, void* stream);
/* Tuning hook (tests, benchmarks): CTAs per (head, sequence) splitting the cached positions, 0 = automatic. */
void w4a16_tune_attention(int split);
/* Tuning hook: 1 launches the small decode-step kernels with programmatic stream serialization, 0 (default) in plain
 * stream order. */
void w4a16_tune_aux_launch(int programmatic);

/*
 * Residual add fused with the normalisation that follows it, for decode-sized inputs.  Replaces the reference's
 * `hidden = residual + hidden` + nn.LayerNorm (modeling_opt_ours.py:590,603-604,614,561-562) or + LlamaRMSNorm
 * (modeling_llama_ours.py:113-118), which run as separate torch kernels.
 *   s = fp16(x + delta) -> x_out (delta NULL: s = x, x_out unused);  h_out = norm(s)
 *   rms == 0: LayerNorm with fp16 `weight` and `bias` (bias may be NULL), statistics and affine in fp32
 *   rms != 0: weight * fp16(s * rsqrt(mean(s^2) + eps)), `bias` ignored
 * x, delta, x_out, h_out fp16 [rows, cols] contiguous, cols % 8 == 0, cols <= 8192 (W4A16_ERR_TOO_LARGE beyond).
 * x_out may alias x or delta.
 */
int w4a16_add_norm(const void* x, const void* delta, void* x_out, void* h_out, const void* weight, const void* bias,
                   int rows, int cols, float eps, int rms, void* stream);

/* out[r, c] = fp16(silu(gate_up[r, c])) * gate_up[r, n + c]: the SwiGLU product of the reference's LlamaMLP
 * (act_fn(gate_proj(x)) * up_proj(x), modeling_llama_ours.py:272) on the output [rows, 2n] of the gate/up projections
 * fused into one GEMV; fp16, n % 8 == 0. */
int w4a16_silu_mul(const void* gate_up, void* out, int rows, int n, void* stream);

/*
 * Normalisation folded into the decode GEMV that consumes it, residual add into the GEMV that produces the block
 * output: two launches fewer per decoder layer.  The reference runs `hidden = residual + hidden` and LayerNorm /
 * LlamaRMSNorm as torch kernels around q/k/v and fc1 / gate-up (modeling_opt_ours.py:561-562,590,603-604,614;
 * modeling_llama_ours.py:113-118).  Here
 *   w4a16_gemm_residual_stats  (and w4a16_gemm_allreduce_residual with row_stats_out != NULL):
 *       out = linear(x) + residual, and per CTA of the grid the sum and the sum of squares of its slice of every
 *       output row are left in `row_stats_out` (w4a16_row_stats_bytes(N) bytes, 16-byte aligned);
 *   w4a16_gemm_prenorm:
 *       out = linear(norm(x)) where x is that output and `row_stats` that buffer: the consumer adds the parts of a
 *       row in index order (deterministic), mean = sum / K, variance = sum of squares / K - mean^2 in fp32, and
 *       normalises its staged activations in place before the main loop.
 *       rms == 0: LayerNorm(x) * norm_weight + norm_bias (norm_bias may be NULL), affine in fp32, one rounding to
 *       fp16; rms != 0: norm_weight * fp16(x * rsqrt(mean(x^2) + eps)) - the arithmetic of w4a16_add_norm except for
 *       the one-pass variance.  norm_weight / norm_bias fp16 [K], 16-byte aligned.
 * Both need tokens <= 16 (one pass of the one-CTA-per-SM decode kernel), w4a16_gemm_prenorm also K <= 8192;
 * W4A16_ERR_BAD_ALGO beyond that: call
 * w4a16_add_norm and w4a16_gemm_fused instead.  flags as for w4a16_gemm_fused (no W4A16_FLAG_SILU_MUL for the
 * producers).
 */
size_t w4a16_row_stats_bytes(int N);
int w4a16_gemm_residual_stats(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                              const void* residual, void* out, void* row_stats_out, int tokens, int N, int K,
                              int group_size, void* stream, unsigned flags);
int w4a16_gemm_prenorm(const void* x, const void* row_stats, const void* norm_weight, const void* norm_bias, float eps,
                       int rms, const void* qweight, const void* zeros_scales, const void* bias, void* out, int tokens,
                       int N, int K, int group_size, void* stream, unsigned flags);

/*
 * No counterpart in the reference.  The tcgen05 GEMM with K split in two, for callers that cannot
 * allocate device memory (inside stream capture, inside a host runtime that owns the allocator, or
 * with a memory budget pinned at start-up): the fp32 partial tiles, the arrival counters and the
 * error word live in a file-scope device array of the library (about 16 MiB per GPU that loads the
 * library, held until the process exits).  Nothing is allocated or freed, no workspace argument.
 * Limits: 2 * tokens * N * 4 bytes <= 16 MiB and at most 4096 output tiles, K >= 1024, g in {64, 128};
 * beyond that W4A16_ERR_TOO_LARGE / W4A16_ERR_BAD_SHAPE.  All calls on a device share the array:
 * calls whose kernels could overlap on the GPU (different streams) must be serialised by the caller.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and clears
 * the error word on `stream`: make that first call outside stream capture.
 */
int w4a16_gemm_static_scratch(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                              void* out, int tokens, int N, int K, int group_size, void* stream);

/* Error word of w4a16_gemm_static_scratch on the current device (see w4a16_device_error_flag). */
int w4a16_static_scratch_error_flag(int* flag);

/*
 * Both GEMM kernels bound every barrier wait; if one ever times out the kernel sets a
 * per-device error word, releases what it holds (tensor memory) and returns.  This reads that
 * word (*flag = 0: no kernel on the current device ever gave up; 1: a barrier wait inside a GEMM kernel timed out;
 * 2: a wait for a peer in the exchange gave up; 3: w4a16_decode_attention was given a position outside the
 * cache).  Synchronises the device; the first call on a device allocates the word, so make it outside stream capture.  The
 * reference has no counterpart (it checks no CUDA error at all, gemm_s4_f16_kernel.h:136-145).
 */
int w4a16_device_error_flag(int* flag);

/* Clears the per-device error word (synchronises the device).  After a kernel gave up on a wait the word stays set
 * until this call; the reference has no counterpart. */
int w4a16_device_error_clear(void);

/* Clears the `gave up` mark and the arrival counter of an exchange buffer (w4a16_exchange_alloc) after a wait for a
 * peer ran out, so that later calls wait for their peers again.  Synchronises the device; call it on every rank
 * before the ranks resume calling.  No counterpart in the reference. */
int w4a16_exchange_reset(void* buffer);

/* How long a kernel waits for a peer's partial sums in the exchange buffers before it gives up, in milliseconds
 * (0 restores the default of 2000).  Process-wide; applies to launches made after the call. */
void w4a16_tune_exchange_wait(unsigned milliseconds);

/* Debug aid: runs a one-CTA probe that writes tagged words to tensor memory with the 16-lane
 * fragment store the tcgen05 kernel uses and reads them back lane by lane; out = uint32
 * [128 lanes][32 columns] on the device.  tests/test_gpu_tmem.py decodes it. */
int w4a16_debug_tmem_layout(void* out, void* stream);

/* Debug aid (library built with -DW4A16_SKINNY_DEBUG): device buffer of uint64 [CTAs][16 warps][8] that receives
 * %globaltimer stamps of the decode kernels' phases; NULL switches it off.  8-token kernel: start, previous grid
 * complete, first unit landed, main loop done, partial sums visible, end.  The tcgen05 kernel writes to the same
 * buffer the cycle accounting of CTA 0's MMA warp: int64 [7] = total cycles, cycles waiting for the dequantised A
 * slot, for the activation stage, for the accumulator, stages whose A / activation probe missed, stages. */
void w4a16_debug_skinny_timeline(void* buf);

/* Benchmark/tuning hooks, not part of the drop-in surface (0 = automatic choice):
 * 16-warp decode kernel: out-feature tiles per CTA (1,2,4,8,16) and cluster split-K (1..8);
 * tcgen05 kernel: token tile (64,128,256) and K parts per output tile;
 * decode path: kernel (1 = the kernel for up to 32 tokens per pass, 2 = the kernel for up to 8 tokens per pass,
 * 0 = by token count), and for the 8-token kernel out-feature tiles per CTA (1,2,4,8,16), cluster split-K (1..8)
 * and ring depth (2..4). */
void w4a16_tune_skinny(int wn, int splits);
void w4a16_tune_tc(int tile_tokens, int split_k);
void w4a16_tune_decode(int kernel, int tiles_per_cta, int splits, int depth);
/* 8-token decode kernel: how many 128-k units beyond its shared-memory ring each warp prefetches into L2
 * (negative = automatic). */
void w4a16_tune_decode_prefetch(int units_ahead);

/* Debug aid: the launch shape the 8-token decode kernel would use for a problem, without launching:
 * plan9 = {tokens per pass, out-feature tiles per CTA, cluster size, ring depth, rows per activation box,
 * shared memory bytes, CTAs with work along x, grid y, grid z} (host array). */
int w4a16_debug_decode_plan(int tokens, int N, int K, int group_size, int* plan9);

/* Number of kernels this library has launched on the calling process so far. */
unsigned long long w4a16_launch_count(void);

/* Library version: major*10000 + minor*100 + patch. */
int w4a16_version(void);

#ifdef __cplusplus
}
#endif
#endif /* W4A16_B200_H_ */
