// Shared device helpers of the W4A16 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "w4a16_b200.h"

namespace w4a16 {

// ---------------------------------------------------------------------------------------------
// Packed weight format ("s4_k_m8" tile order of the reference, cta_iterator.h:86-88):
//   physical [K/32][N/32][lane 0..31][word 0..3]; a 32(k) x 32(n) tile is 512 contiguous bytes,
//   16 bytes per lane.  For element (n, k) inside a tile
//       lane   = (n % 8) * 4 + (k % 8) / 2
//       word   = ((k / 16) % 2) * 2 + ((n / 16) % 2)
//       nibble = (k % 2) * 4 + ((k / 8) % 2) * 2 + ((n / 8) % 2)
//   so word (kh, nh) of a lane is the mma.m16n8k16 A fragment (rows = out-features) of the
//   16(n) x 16(k) sub-block (nh, kh): after unpack_s4x8() h[0] = row r, k 2c..2c+1; h[1] = row
//   r+8, same k; h[2] = row r, k+8; h[3] = row r+8, k+8   (r = lane/4, c = lane%4).
// ---------------------------------------------------------------------------------------------

constexpr int kTileK = 32;
constexpr int kTileN = 32;

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}

// Eight nibbles -> four half2 bit patterns, each half = fp16(64 + q) (0x5400 | q << 4), exact.
// Same values as dequantize_s4_to_fp16x2_v2 (common.h:114-153): pairs are nibbles (0,4), (1,5),
// (2,6), (3,7).
__device__ __forceinline__ void unpack_s4x8(uint32_t w, uint32_t (&h)[4])
{
    constexpr uint32_t kMask = 0x00f000f0u, kMagic = 0x54005400u;
    h[0] = lop3_and_or(w << 4, kMask, kMagic);
    h[1] = lop3_and_or(w, kMask, kMagic);
    h[2] = lop3_and_or(w >> 4, kMask, kMagic);
    h[3] = lop3_and_or(w >> 8, kMask, kMagic);
}

// Same result with fewer integer-pipe instructions: the low nibble of each byte is read in place as
// fp16 (1024 + q) and brought to (64 + q) by an exact fp16 subtraction of 960 (FMA pipe).
__device__ __forceinline__ void unpack_s4x8_fast(uint32_t w, uint32_t (&h)[4])
{
    constexpr uint32_t kLo = 0x000f000fu, kHi = 0x00f000f0u, k1024 = 0x64006400u, k64 = 0x54005400u, k960 = 0x63806380u;
    const uint32_t top = w >> 8;
    uint32_t a = lop3_and_or(w, kLo, k1024), c = lop3_and_or(top, kLo, k1024);
    h[1] = lop3_and_or(w, kHi, k64);
    h[3] = lop3_and_or(top, kHi, k64);
    asm("sub.f16x2 %0, %1, %2;" : "=r"(h[0]) : "r"(a), "r"(k960));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(h[2]) : "r"(c), "r"(k960));
}

// Cheapest form, for kernels that rescale in fp32 afterwards: each nibble is only masked in place, which leaves a
// subnormal fp16 bit pattern.  h[0], h[2] (rows r) hold q * 2^-24, h[1], h[3] (rows r+8) hold q * 2^-20; the tensor
// core multiplies subnormal fp16 inputs exactly, so the fp32 accumulators carry exact multiples of q * x.
constexpr float kDenormScaleLo = 16777216.f;     // 2^24, rows r
constexpr float kDenormScaleHi = 1048576.f;      // 2^20, rows r + 8
__device__ __forceinline__ void unpack_s4x8_denorm(uint32_t w, uint32_t (&h)[4])
{
    constexpr uint32_t kLo = 0x000f000fu, kHi = 0x00f000f0u;
    const uint32_t top = w >> 8;
    h[0] = w & kLo;
    h[1] = w & kHi;
    h[2] = top & kLo;
    h[3] = top & kHi;
}

// (t - z) * s in fp16 with flush-to-zero, two lanes at a time: bit-exact with apply_Q
// (common.h:210-225, the non-FMA branch).
__device__ __forceinline__ uint32_t dequant_h2(uint32_t t, uint32_t zz, uint32_t ss)
{
    uint32_t u, v;
    asm("sub.ftz.f16x2 %0, %1, %2;" : "=r"(u) : "r"(t), "r"(zz));
    asm("mul.ftz.f16x2 %0, %1, %2;" : "=r"(v) : "r"(u), "r"(ss));
    return v;
}

// half2 (zero+64, scale) -> (zz, ss) broadcasts
__device__ __forceinline__ void split_zs(uint32_t zs, uint32_t& zz, uint32_t& ss)
{
    zz = __byte_perm(zs, zs, 0x1010);
    ss = __byte_perm(zs, zs, 0x3232);
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p)
{
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

__device__ __forceinline__ uint32_t ldg_nc_u32(const void* p)
{
    uint32_t r;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// D = A * B (accumulator starts at zero)
__device__ __forceinline__ void mma_m16n8k16_zc(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr) : "memory");
}

// ---------------------------------------------------------------------------------------------
// host-side plumbing shared by the translation units
// ---------------------------------------------------------------------------------------------
// Exchange buffer of one rank for the GEMV fused with its all-reduce (row-parallel linears): every rank owns one
// such buffer and maps all its peers' buffers.  Layout:
//   [ExchangeHeader, 256 B][data: 2 halves x world x capacity slots of 8 bytes]
// A slot is (32-bit payload, 32-bit tag) written with ONE 8-byte store, which arrives atomically: the receiver
// polls the slot itself until the tag is the current call's - no separate flag, no fence, one NVLink crossing.
// Tags are epoch + 1, unique per call, so stale slots of earlier calls never match; the two halves alternate so
// that a rank already in the next call cannot overwrite slots a slower rank is still reading.
constexpr int    kExchangeMaxWorld   = 8;
constexpr size_t kExchangeDataOffset = 256;
struct ExchangeHeader {
    unsigned epoch;     // calls completed on this rank; selects the buffer half (epoch & 1) and the flag value (epoch + 1)
    unsigned ticket;    // CTAs of the running call that are done; the last one advances `epoch`
    int      error;     // set when a wait for a peer gave up
};
struct ExchangeArgs {
    unsigned char* peer[kExchangeMaxWorld];   // device pointers to every rank's buffer (own included), by rank
    int world, rank;
    long long capacity;                        // fp32 elements per (half, source rank) slot
    int k_config;                              // K all ranks agree on for choosing the launch shape (largest K shard)
};

struct GemmArgs {
    const __half*   x;
    const uint32_t* qw;
    const uint32_t* zs;    // half2 (zero+64, scale) as 32-bit words, [K/g][N]
    const __half*   bias;  // may be null
    __half*         out;
    int tokens, N, K, g;
    bool static_weights;   // W4A16_FLAG_STATIC_WEIGHTS
    bool relu = false;     // W4A16_FLAG_RELU: out = max(out, 0) after the bias add
    bool silu_mul = false; // W4A16_FLAG_SILU_MUL: gate / up tiles alternate, out = silu(gate) * up, [tokens, N / 2] (decode kernels)
    const __half* residual = nullptr;   // [tokens, N] added after bias / ReLU, or null
    const ExchangeArgs* exchange = nullptr;   // non-null: out = sum over ranks of this rank's partial product (decode kernel only)
    bool plan_only = false;                   // check the arguments and the launch plan, launch nothing
    // non-null: x is normalised row by row (LayerNorm, or RMSNorm when norm_rms) after it is staged - the launch of
    // the normalisation kernel in front of the GEMV is saved (<= 16 tokens, one-CTA-per-SM decode kernel only).  The
    // row statistics come from the GEMV that produced x (row_stats_in = its row_stats_out).
    const float* row_stats_in = nullptr;
    float* row_stats_out = nullptr;       // non-null: row statistics of this call's output for the next GEMV
    const __half* norm_weight = nullptr;
    const __half* norm_bias = nullptr;    // LayerNorm only, may be null
    float norm_eps = 0.f;
    bool norm_rms = false;
};

// Launch, optionally with programmatic stream serialization (the grid may then be scheduled while the previous
// kernel of the stream drains).  Only for kernels that execute griddepcontrol.wait before they touch anything the
// stream's earlier work produces.
int device_sm_count();                           // SMs of the current device (cached); 148 when the query fails
bool aux_programmatic_launch();                  // tuning switch (w4a16_tune_aux_launch), default off
template <typename... KArgs, typename... Args>
cudaError_t launch_after_previous(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = aux_programmatic_launch() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

int  record_cuda_error(cudaError_t e);          // returns W4A16_ERR_CUDA, remembers e
void count_launch(unsigned n = 1);
int* device_error_word();
// cuTensorMapEncodeTiled for a row-major 2-D tensor (dims = {inner, outer} in elements); `tmap` is a CUtensorMap*
int encode_tensor_map_2d(void* tmap, const void* base, int elem_bytes, const uint64_t dims[2], uint64_t row_stride_bytes,
                         const uint32_t box[2], bool swizzle128);                       // per-device word a kernel sets to 1 when a bounded wait gives up

// decode path: tokens <= 16 per pass -> launch_gemv (8-warp CTAs, two per SM), otherwise the 16-warp kernel
int launch_skinny(const GemmArgs& a, cudaStream_t st);
int launch_gemv(const GemmArgs& a, cudaStream_t st);
// how long a kernel waits for a peer's partial sums in the exchange buffers before it gives up (w4a16_tune_exchange_wait)
unsigned long long exchange_wait_budget_ns();
// err_word: device word raised on a barrier timeout (nullptr = the library's per-device word)
// force_split: 0 = planned, otherwise the number of K parts per output tile
int launch_tc(const GemmArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t st, int* err_word = nullptr,
              int force_split = 0);
size_t tc_workspace_bytes(int tokens, int N, int K, int g);
bool tc_supported(int tokens, int N, int K, int g);

}  // namespace w4a16
