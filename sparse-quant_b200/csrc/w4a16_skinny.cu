// Decode kernel: skinny W4A16 GEMM (tokens <= 32 per pass), HBM-bandwidth bound.
//
//   out[t, n] = fp16( sum_k fp32( dq(W)[n, k] * x[t, k] ) ) (+ bias[n])
//
// Replaces the small-token instantiations of gemm_s4_f16_nn (gemm_template.h:358-464 of the
// reference, CTA shapes (x, 8|16, 256|512) of gemm_s4_f16.cu:66-87), which run at most N/64 CTAs,
// stream K serially and re-do the fp16 dequantisation arithmetic in the MMA issue slots.  Here the
// whole machine streams the weight matrix once, in one wave of one 512-thread CTA per SM:
//
//   * a warp owns one 32-wide out-feature tile and a contiguous K slice.  Its lane 0 keeps a
//     private ring of TMA copies in flight into shared memory, two 256-k units deep: per unit one
//     tensor copy (an 8-row box of the packed matrix seen as [K/32][N/32 x 512 B]: eight strided
//     512-byte tiles in one operation) plus one 128-byte bulk copy per quantisation group of its
//     (zero, scale) pairs, all completing on the unit's own mbarrier - about 130 KB in flight per
//     SM with no registers spent on it;
//   * the nibbles are only masked in place (one shift + four ANDs per eight weights), which leaves subnormal
//     fp16 patterns q * 2^-24 / q * 2^-20 that the tensor core multiplies exactly, and are fed straight to
//     mma.m16n8k16 as the A fragment (the packed layout IS that fragment); activations are staged
//     once per CTA in shared memory and read with ldmatrix as the B fragment; sum_k x[t, k] of every
//     group is computed once per CTA by an MMA with an all-ones A fragment.  At the end of each
//     quantisation group the zero point and the scale are applied in fp32 (the power of two folded into
//     both):  acc += s * (sum q x - z sum x).
//     That is (q - z) * s without the intermediate fp16 rounding of the weight; with the identity
//     matrix as input the output reproduces the reference's dequantised weight bit for bit
//     (denormal scales are flushed to zero as mul.ftz does), and for general inputs it agrees with
//     dequantise-then-matmul to ~1e-4 relative, far inside the stated tolerance;
//   * split-K: WK warps of a CTA cover different K slices of the same tiles and S CTAs of one
//     thread-block cluster cover different K ranges (only when the staged activations would not
//     fit); partial sums meet in shared memory and are reduced across the cluster through
//     distributed shared memory in a fixed order: deterministic, no global scratch, no atomics;
//   * bias add, fp16 rounding and the [tokens, N] store are fused into the reduction.
// Every mbarrier wait is bounded; a timeout raises the library's device error word.
#include <cooperative_groups.h>
#include <cuda.h>

#include "w4a16_common.cuh"
#include "w4a16_sm100.cuh"

namespace cg = cooperative_groups;

namespace w4a16 {

using namespace sm100;

namespace {

#ifdef W4A16_SKINNY_DEBUG
constexpr bool kDebug = true;     // phase time stamps and experiment switches compiled in
#else
constexpr bool kDebug = false;
#endif

constexpr int kMaxWarps  = 32;
constexpr int kHeaderBytes = 2048;           // zero chunk, abort flag, mbarriers
constexpr int kMaxDepth  = 4;                 // most units in flight per warp
// k per pipeline unit: 256 (8 tiles) when at most 8 tokens are staged, 128 otherwise (the staged activations
// then need the shared memory); the ring holds 2 x 256-k or up to 4 x 128-k units per warp
__host__ __device__ constexpr int unit_k_for(int tg) { return tg == 1 ? 256 : 128; }
__host__ __device__ constexpr int max_depth_for(int tg) { return tg == 1 ? 2 : 4; }
constexpr uint64_t kWaitBudgetNs = 200ull * 1000 * 1000;

template <int G, int UK>
struct Slot {                                 // one pipeline unit in shared memory
    uint4    tiles[UK / kTileK][32];          // 512 B per 32x32 tile
    uint32_t zs[UK / G][32];                  // per group: (zero+64, scale) of the tile's 32 out-features
};

struct SkinnyParams {
    const __half*   x;
    const uint4*    qw;
    const uint32_t* zs;
    const __half*   bias;
    __half*         out;
    int*            error;
    int tokens, N, K;
    int wn;          // out-feature tiles per CTA (1,2,4,8,16); WK = 16 / wn K-slices per CTA
    int wn_shift;    // log2(wn)
    unsigned inv_splits;   // ceil(2^32 / splits): x / splits == umulhi(x, inv_splits) for the small x used here
    int splits;      // cluster size along K (gridDim.y)
    int xs_stride;   // halfs per staged activation row
    int xsum_offset; // byte offset of the per-group activation sums [groups of the CTA][tokens] fp32
    int ring_offset; // byte offset of the per-warp rings in shared memory
    int depth;       // units in flight per warp (>= 2)
    int warps;       // warps per CTA
    const __half* residual;   // [tokens, N] added to the output after bias / ReLU (fp16 add), or null
    const __half* norm_w;     // non-null: x rows are normalised after they are staged (weight [K]); needs stats_in
    const float* stats_in;    // row statistics of x written by the GEMV that produced it
    float* stats_out;         // non-null: row statistics of this call's output (after bias / ReLU / residual) are written here
    const __half* norm_b;     // LayerNorm bias [K] or null
    float norm_eps;
    int norm_rms;             // 1: RMSNorm (weight * fp16(x * rstd)), 0: LayerNorm
    int silu_mul;    // out-feature tiles alternate gate / up; out[t, j] = silu(gate_j) * up_j, [tokens, N / 2]
    int relu;        // clamp the outputs at zero after the bias add
    int pdl;         // 1: launched with programmatic stream serialization; weights may be fetched before the previous grid ends
    // fused all-reduce over peer memory (world == 0: plain store of this GPU's result)
    unsigned char* peer[kExchangeMaxWorld];
    unsigned char* self;          // = peer[rank]
    int world, rank;
    long long capacity;
    unsigned long long wait_budget_ns;   // how long the exchange waits for a peer
    unsigned long long* timeline;   // debug: [cta][warp][8] globaltimer stamps, or null
    int debug_mode;  // experiments: bit 0 = skip the MMA work, bit 1 = skip staging the activations
};

// lane 0 of a warp: arm the slot's barrier and start the copies of one unit.  `zsrc` points at the unit's first
// (zero, scale) row for this warp's out-feature tile.
template <int G, int kUnitK>
__device__ __forceinline__ void issue_unit(uint32_t slot_addr, uint32_t bar, const CUtensorMap* wmap, const uint32_t* zsrc,
                                           int N, int unit, int nt, int groups)
{
    constexpr int kGroupsPerUnit = kUnitK / G;
    constexpr int kUnitTiles = kUnitK / kTileK;
    const int n_groups = min(kGroupsPerUnit, groups - unit * kGroupsPerUnit);     // < full only at the K edge
    // the tensor copy always delivers the full box of kUnitTiles x 512 B (rows past K/32 arrive as zeros)
    mbar_arrive_expect_tx(bar, kUnitTiles * 512u + n_groups * 128u);
    tma_load_2d(slot_addr, wmap, nt * 128, unit * kUnitTiles, bar);
#pragma unroll
    for (int gi = 0; gi < kGroupsPerUnit; ++gi)
        if (gi < n_groups) bulk_load(slot_addr + kUnitTiles * 512u + gi * 128u, zsrc + (size_t)gi * N, 128u, bar);
}

template <int TG, int G, int kUnitK>
__device__ __forceinline__ void compute_unit(const Slot<G, kUnitK>* slot, float (&acc)[TG][2][4], const uint32_t (&xaddr)[TG],
                                             const int (&kmul)[TG], int k_local, int kt0, int k_tiles, int lane, int dbg,
                                             const float* xsum_s)
{
    constexpr int kTilesPerGroup = G / kTileK;
    constexpr uint32_t kOnes = 0x3c003c00u;
    const int r = lane >> 2, c = lane & 3;
#pragma unroll
    for (int gi = 0; gi < kUnitK / G; ++gi) {
        if (kt0 + gi * kTilesPerGroup < k_tiles) {                  // warp-uniform: the group exists
            // two accumulator chains (out-features 0-15, 16-31) per token group, interleaved per 16-k half
            float accg[TG][2][4];
#pragma unroll
            for (int tt = 0; tt < kTilesPerGroup; ++tt) {
                const int t = gi * kTilesPerGroup + tt;
                uint32_t b[TG][4];
#pragma unroll
                for (int tg = 0; tg < TG; ++tg)
                    ldmatrix_x4(b[tg], xaddr[tg] + (uint32_t)((k_local + t * kTileK) * kmul[tg]));
                const uint4 q = slot->tiles[t][lane];
                const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int kh = 0; kh < 2; ++kh) {
                    uint32_t a0[4], a1[4];
                    if (dbg & 4) {
                        a0[0] = a0[1] = a0[2] = a0[3] = words[kh * 2 + 0];
                        a1[0] = a1[1] = a1[2] = a1[3] = words[kh * 2 + 1];
                    } else {
                        unpack_s4x8_denorm(words[kh * 2 + 0], a0);
                        unpack_s4x8_denorm(words[kh * 2 + 1], a1);
                    }
#pragma unroll
                    for (int tg = 0; tg < TG; ++tg) {
                        if (tt == 0 && kh == 0) {
                            mma_m16n8k16_zc(accg[tg][0], a0, b[tg][0], b[tg][1]);
                            mma_m16n8k16_zc(accg[tg][1], a1, b[tg][0], b[tg][1]);
                        } else {
                            mma_m16n8k16(accg[tg][0], a0, b[tg][2 * kh], b[tg][2 * kh + 1]);
                            mma_m16n8k16(accg[tg][1], a1, b[tg][2 * kh], b[tg][2 * kh + 1]);
                        }
                    }
                }
            }
            // zero point and scale of the group, applied in fp32; sum_k x of the group was precomputed per CTA
            float xsum[TG][2];
#pragma unroll
            for (int tg = 0; tg < TG; ++tg) {
                const float2 v = *reinterpret_cast<const float2*>(xsum_s + (k_local / G + gi) * (8 * TG) + tg * 8 + 2 * c);
                xsum[tg][0] = v.x;
                xsum[tg][1] = v.y;
            }
            if (dbg & 8) {
#pragma unroll
                for (int tg = 0; tg < TG; ++tg)
#pragma unroll
                    for (int j = 0; j < 4; ++j) { acc[tg][0][j] += accg[tg][0][j]; acc[tg][1][j] += accg[tg][1][j]; }
                continue;
            }
#pragma unroll
            for (int nh = 0; nh < 2; ++nh) {
                float zf[2], sf[2];
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {
                    // (zero + 64, scale) * (1, 1) with flush-to-zero: a denormal scale becomes 0, as under mul.ftz
                    uint32_t v = slot->zs[gi][nh * 16 + hi * 8 + r];
                    asm("mul.ftz.f16x2 %0, %1, %2;" : "=r"(v) : "r"(v), "r"(kOnes));
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
                    // the accumulators hold sum(q x) * 2^-24 (rows r) or * 2^-20 (rows r+8): fold the power of two
                    // into the zero point (zero = f.x - 64) and the scale; both products are exact in fp32
                    const float up = hi ? kDenormScaleHi : kDenormScaleLo;
                    zf[hi] = (f.x - 64.f) * (1.f / up);
                    sf[hi] = f.y * up;
                }
#pragma unroll
                for (int tg = 0; tg < TG; ++tg) {
                    acc[tg][nh][0] = fmaf(sf[0], fmaf(-zf[0], xsum[tg][0], accg[tg][nh][0]), acc[tg][nh][0]);
                    acc[tg][nh][1] = fmaf(sf[0], fmaf(-zf[0], xsum[tg][1], accg[tg][nh][1]), acc[tg][nh][1]);
                    acc[tg][nh][2] = fmaf(sf[1], fmaf(-zf[1], xsum[tg][0], accg[tg][nh][2]), acc[tg][nh][2]);
                    acc[tg][nh][3] = fmaf(sf[1], fmaf(-zf[1], xsum[tg][1], accg[tg][nh][3]), acc[tg][nh][3]);
                }
            }
        }
    }
}

__device__ __forceinline__ void st_slot(uint2* p, uint2 v)          // one 8-byte store: payload and tag land together
{
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ uint2 ld_slot(const uint2* p)
{
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// fp32 load from the shared memory of CTA `rank` of this cluster (own rank included)
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank)
{
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// Row statistics handed from a GEMV to the next one (device buffer of floats): [0] = number of parts (int bits),
// [1..3] unused, then per part 16 rows x (sum, sum of squares) of the part's slice of the output row.  A part is one
// CTA of the producing grid; the consumer adds the parts of a row in index order.
constexpr int kStatsHeaderFloats = 4;
constexpr int kStatsRows = 16;
constexpr int kStatsOffset = 1088;             // byte offset in the shared-memory header of 32 floats of scratch

// TG = token groups of 8 handled per pass (1, 2, 4); G = quantisation group size.
template <int TG, int G, int kWarps, bool kPreNorm = false>
__global__ void __launch_bounds__(kWarps * 32, 1) skinny_kernel(const __grid_constant__ CUtensorMap wmap, const SkinnyParams p)
{
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int kTok = 8 * TG;
    constexpr int kThreads = kWarps * 32;
    constexpr int kUnitK = unit_k_for(TG), kUnitTiles = kUnitK / kTileK, kDepth = kMaxDepth;
    using SlotT = Slot<G, kUnitK>;
    static_assert(2 * sizeof(SlotT) >= kTok * 33 * 4, "a warp's partial sums reuse its own ring (depth >= 2)");
    static_assert(sizeof(SlotT) % 16 == 0, "bulk copies need 16-byte aligned destinations");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // all index arithmetic below is shifts, masks and one multiply-high: a 64-bit division costs about a hundred
    // instructions per thread, and with ~30 tiles per warp the fixed part of the kernel is what the small shapes pay for
    static_assert((kWarps & (kWarps - 1)) == 0, "power-of-two warp count");
    const int wn = p.wn, wk = kWarps >> p.wn_shift;
    const int wn_idx = warp & (wn - 1), wk_idx = warp >> p.wn_shift;
    const int wk_sh = 31 - __clz(wk);
    const int n_tiles = p.N / kTileN;
    const int nt = blockIdx.x * wn + wn_idx;
    const bool nt_valid = nt < n_tiles;
    const int tok0 = blockIdx.z * kTok;
    const int rows = min(kTok, p.tokens - tok0);        // real token rows of this pass

    // K decomposition in 128-k units: cluster rank -> CTA range -> warp slice
    const int k_tiles = p.K / kTileK;
    const int units = (p.K + kUnitK - 1) / kUnitK;
    const int S = p.splits, rank = blockIdx.y;
    auto div_splits = [&](int x) { return S == 1 ? x : (int)__umulhi((unsigned)x, p.inv_splits); };
    const int cu0 = div_splits(units * rank), cu1 = div_splits(units * (rank + 1));
    const int cta_units = cu1 - cu0;
    const int wu0 = cu0 + ((cta_units * wk_idx) >> wk_sh), wu1 = cu0 + ((cta_units * (wk_idx + 1)) >> wk_sh);
    const int n_units = nt_valid ? wu1 - wu0 : 0;

    // shared memory: header (kHeaderBytes): [16 B zeros][abort flag][barriers kMaxWarps x kDepth] | activations | per-warp rings
    static_assert(32 + kMaxWarps * kMaxDepth * 8 <= kHeaderBytes, "header overflow");
    const uint32_t bars = smem_u32(smem) + 32 + warp * kDepth * 8;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 16);
    __half* xs = reinterpret_cast<__half*>(smem + kHeaderBytes);
    const int depth = p.depth;
    const int ring_bytes = depth * (int)sizeof(SlotT);   // per warp
    SlotT* ring = reinterpret_cast<SlotT*>(smem + p.ring_offset + (size_t)warp * ring_bytes);

    unsigned long long* tl = nullptr;
    if (kDebug && p.timeline && lane == 0)
        tl = p.timeline + ((size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * kWarps + warp) * 8;
    if (tl) tl[0] = globaltimer_ns();
    if (threadIdx.x == 0) *abort_flag = 0;
    if (threadIdx.x < 4) reinterpret_cast<uint32_t*>(smem)[threadIdx.x] = 0u;
    if (lane == 0) {
        for (int i = 0; i < kDepth; ++i) mbar_init(bars + 8 * i, 1);
        if (warp == 0) mbar_init(smem_u32(smem) + 24, 1);       // the activations' barrier
        mbar_fence_init();
    }

    // Activations x[tok0 .. tok0+rows) x [this CTA's K range] are staged in shared memory by bulk copies, one per
    // token row, all completing on one mbarrier; the part of the range beyond K (last units only) is zero-filled
    // by hand.  Token rows past `rows` all read the 16 zero bytes at the start of shared memory.
    const int kc0 = cu0 * kUnitK;
    const int row_halfs = cta_units * kUnitK;                                  // staged k per row
    const int copy_halfs = max(0, min(row_halfs, p.K - kc0));                 // of which exist in x
    const uint32_t xbar = smem_u32(smem) + 24;
    const bool stage_x = !(kDebug && (p.debug_mode & 2)) && copy_halfs > 0;
    auto issue_x = [&]() {
        if (threadIdx.x == 0 && stage_x) {
            mbar_arrive_expect_tx(xbar, (uint32_t)rows * (uint32_t)copy_halfs * 2u);
            for (int row = 0; row < rows; ++row)
                bulk_load(smem_u32(xs) + (uint32_t)(row * p.xs_stride) * 2u, p.x + (size_t)(tok0 + row) * p.K + kc0, (uint32_t)copy_halfs * 2u, xbar);
        }
    };
    const uint32_t ring_addr = smem_u32(ring);
    const int groups = p.K / G;
    const size_t zs_step = (size_t)(kUnitK / G) * p.N;                        // words between consecutive units
    const uint32_t* zs_next = p.zs + (size_t)wu0 * zs_step + nt * kTileN;     // first unit of this warp
    auto issue_first_units = [&]() {
        if (lane == 0) {
            if (warp == 0) prefetch_tmap(&wmap);
            for (int i = 0; i < depth && i < n_units; ++i)
                issue_unit<G, kUnitK>(ring_addr + i * (uint32_t)sizeof(SlotT), bars + 8 * i, &wmap, zs_next + (size_t)i * zs_step, p.N, wu0 + i, nt, groups);
        }
    };

    constexpr bool prenorm = kPreNorm;                          // its own instantiation: the plain kernel keeps its registers
    // Fused normalisation: thread t owns the 16-byte column vectors c = t % nv (+ nv_step) of the staged K range and the
    // token rows t / nv, t / nv + kThreads / nv, ...  The affine parameters of its columns are static like the packed
    // weights: they are fetched before the wait for the previous kernel, so that no global load sits between the
    // arrival of the activations and the main loop.
    const int pn_nv = copy_halfs >> 3;                          // vectors of the staged range per row
    const int pn_cols = pn_nv < kThreads ? pn_nv : kThreads;    // distinct first columns among the threads
    const int pn_c0 = pn_cols > 0 ? (int)threadIdx.x % pn_cols : 0, pn_r0 = pn_cols > 0 ? (int)threadIdx.x / pn_cols : 0;
    const int pn_rstep = pn_cols > 0 ? kThreads / pn_cols : 1;  // rows advance by this much (0 rows left over when nv > kThreads)
    uint4 pn_w[2], pn_b[2];
    if constexpr (prenorm) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c = pn_c0 + j * kThreads;
            pn_w[j] = make_uint4(0, 0, 0, 0);
            pn_b[j] = make_uint4(0, 0, 0, 0);
            if (c < pn_nv) {
                pn_w[j] = *reinterpret_cast<const uint4*>(p.norm_w + kc0 + c * 8);
                if (p.norm_b) pn_b[j] = *reinterpret_cast<const uint4*>(p.norm_b + kc0 + c * 8);
            }
        }
    }
    if (p.pdl) {
        // Programmatic dependent launch: this grid may start while the previous kernel of the stream is
        // still draining.  The packed weights are static by contract, so their copies start at once; the
        // activations (and everything this kernel writes) wait for the previous grid to complete.
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        issue_first_units();
        asm volatile("griddepcontrol.wait;" ::: "memory");
        issue_x();
    } else {
        // The activation copies are issued BEFORE the weight copies: they are on the critical path and must
        // not queue behind megabytes of weight traffic.
        issue_x();
        issue_first_units();
    }
    if (copy_halfs < row_halfs) {                               // K edge: zeros behind the copied part of every row
        const int tail_vec = (row_halfs - copy_halfs) / 8;
        for (int i = threadIdx.x; i < rows * tail_vec; i += kThreads) {
            const int row = i / tail_vec, v = i - row * tail_vec;
            *reinterpret_cast<uint4*>(xs + row * p.xs_stride + copy_halfs + v * 8) = make_uint4(0, 0, 0, 0);
        }
    }
    __syncthreads();                                            // barrier initialised, zero tail written
    if constexpr (prenorm) {
        // Normalisation folded into this GEMV (the launch of the normalisation kernel in front of it is saved): the
        // row statistics come from the GEMV that produced x (its CTAs each left the sum and the sum of squares of
        // their slice of every row); warp r adds the parts of row r in index order while the activation copies are
        // in flight, then the staged K range is normalised in place.
        static_assert(32 + kMaxWarps * kMaxDepth * 8 <= kStatsOffset && kStatsOffset + 2 * kStatsRows * 4 <= kHeaderBytes, "scratch in the header");
        float* mean_s = reinterpret_cast<float*>(smem + kStatsOffset);
        float* rstd_s = mean_s + kStatsRows;
        if (warp < rows) {
            const int parts = *reinterpret_cast<const int*>(p.stats_in);
            const float2* data = reinterpret_cast<const float2*>(p.stats_in + kStatsHeaderFloats) + tok0 + warp;
            float a = 0.f, b = 0.f;
            for (int i = lane; i < parts; i += 32) {
                const float2 v = data[(size_t)i * kStatsRows];
                a += v.x;
                b += v.y;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, o);
                b += __shfl_xor_sync(0xffffffffu, b, o);
            }
            if (lane == 0) {
                const float mean = p.norm_rms ? 0.f : a / p.K;
                const float var = fmaxf(b / p.K - mean * mean, 0.f);
                mean_s[warp] = mean;
                rstd_s[warp] = rsqrtf(var + p.norm_eps);
            }
        }
        if (stage_x) mbar_wait(xbar, 0, abort_flag, kWaitBudgetNs);
        __syncthreads();                                        // statistics visible to every thread
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c = pn_c0 + j * kThreads;
            if (c < pn_nv) {
                const __half* wh = reinterpret_cast<const __half*>(&pn_w[j]);
                const __half* bh = reinterpret_cast<const __half*>(&pn_b[j]);
                for (int row = pn_r0 < pn_rstep ? pn_r0 : rows; row < rows; row += pn_rstep) {   // threads beyond the last full group idle
                    __half* px = xs + row * p.xs_stride + c * 8;
                    const uint4 xv = *reinterpret_cast<const uint4*>(px);
                    const __half* xh = reinterpret_cast<const __half*>(&xv);
                    const float m = mean_s[row], rs = rstd_s[row];
                    uint4 o;
                    __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float f = __half2float(xh[e]);
                        if (p.norm_rms) oh[e] = __hmul(wh[e], __float2half_rn(f * rs));
                        else oh[e] = __float2half_rn((f - m) * rs * __half2float(wh[e]) + __half2float(bh[e]));
                    }
                    *reinterpret_cast<uint4*>(px) = o;
                }
            }
        }
        __syncthreads();                                        // normalised activations visible to every warp
    } else {
        if (stage_x) mbar_wait(xbar, 0, abort_flag, kWaitBudgetNs);
    }
    if (tl) tl[1] = globaltimer_ns();

    // sum_k x[t, k] per quantisation group, by an MMA with an all-ones A fragment over the staged activations (every
    // row of the result holds the sums); the main loop reads them back when it applies the zero points.  With one
    // out-feature tile per CTA every warp owns a different K slice and computes just its own groups - nobody else
    // needs them, so a warp-level barrier is enough.  With several tiles per CTA the warps of a K slice would repeat
    // each other's work: the groups of the whole CTA are dealt round-robin and a CTA-wide barrier follows.
    {
        float* xsum_w = reinterpret_cast<float*>(smem + p.xsum_offset);
        const int k_end = min(cu1 * kUnitK, p.K);
        const int cta_groups = (k_end - cu0 * kUnitK) / G;
        const bool own_slice = wn == 1;
        const int g_lo = own_slice ? (wu0 - cu0) * (kUnitK / G) : warp;
        const int g_hi = own_slice ? (min(wu1 * kUnitK, p.K) - cu0 * kUnitK) / G : cta_groups;
        const int g_step = own_slice ? 1 : kWarps;
        constexpr uint32_t kOnes = 0x3c003c00u;
        const uint32_t ones[4] = {kOnes, kOnes, kOnes, kOnes};
        for (int gidx = g_lo; gidx < g_hi; gidx += g_step) {
#pragma unroll
            for (int tg = 0; tg < TG; ++tg) {
                const int row = tg * 8 + (lane & 7);
                const bool real = row < rows;
                const uint32_t base = real ? smem_u32(xs) + (uint32_t)((row * p.xs_stride + (lane >> 3) * 8 + gidx * G) * 2) : smem_u32(smem);
                float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int t = 0; t < G / kTileK; ++t) {
                    uint32_t b[4];
                    ldmatrix_x4(b, base + (real ? t * kTileK * 2 : 0));
                    mma_m16n8k16(sum, ones, b[0], b[1]);
                    mma_m16n8k16(sum, ones, b[2], b[3]);
                }
                if (lane < 4) *reinterpret_cast<float2*>(xsum_w + gidx * kTok + tg * 8 + 2 * lane) = make_float2(sum[0], sum[1]);
            }
        }
        if (own_slice) __syncwarp();
        else __syncthreads();
    }
    if (tl) tl[2] = globaltimer_ns();

    float acc[TG][2][4];
#pragma unroll
    for (int tg = 0; tg < TG; ++tg)
#pragma unroll
        for (int nh = 0; nh < 2; ++nh)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[tg][nh][j] = 0.f;

    if (n_units > 0) {
        // ldmatrix row address per token group: matrix j = lane/8 covers k offset 8j, row = token lane%8.
        // Rows beyond the real tokens point at the zero chunk and do not advance with k.
        uint32_t xaddr[TG];
        int kmul[TG];
#pragma unroll
        for (int tg = 0; tg < TG; ++tg) {
            const int row = tg * 8 + (lane & 7);
            const bool real = row < rows;
            xaddr[tg] = real ? smem_u32(xs) + (uint32_t)((row * p.xs_stride + (lane >> 3) * 8) * 2) : smem_u32(smem);
            kmul[tg] = real ? 2 : 0;
        }
        int slot = 0;
        uint32_t phase = 0;
        for (int i = 0; i < n_units; ++i) {
            const bool ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * slot, phase, abort_flag, kWaitBudgetNs));
            if (!ok) break;
            if (tl && i == 0) tl[3] = globaltimer_ns();
            const int u = wu0 + i;
            if (!kDebug || (p.debug_mode & 1) == 0)
                compute_unit<TG, G, kUnitK>(ring + slot, acc, xaddr, kmul, (u - cu0) * kUnitK, u * kUnitTiles, k_tiles, lane, kDebug ? p.debug_mode : 0,
                                            reinterpret_cast<const float*>(smem + p.xsum_offset));
            else
                acc[0][0][0] += __uint_as_float(ring[slot].tiles[0][lane].x & 0x3fu);
            __syncwarp();                                   // every lane is done reading the slot
            if (i + depth < n_units && sm100::elect_one())
                issue_unit<G, kUnitK>(ring_addr + slot * (uint32_t)sizeof(SlotT), bars + 8 * slot, &wmap, zs_next + (size_t)(i + depth) * zs_step, p.N,
                              u + depth, nt, groups);
            if (++slot == depth) { slot = 0; phase ^= 1u; }
        }
    }

    if (tl) tl[4] = globaltimer_ns();
    // ---- reduction: warps -> CTA (shared memory), CTAs -> cluster (distributed shared memory) ----
    // a warp's partial sums [32 out-features][kTok] go to the start of its own (drained) ring
    {
        __syncwarp();
        const int r = lane >> 2, c = lane & 3;
        float* dst = reinterpret_cast<float*>(ring);        // [kTok][33]: out-feature fastest, padded row
#pragma unroll
        for (int tg = 0; tg < TG; ++tg)
#pragma unroll
            for (int nh = 0; nh < 2; ++nh) {
                float* d0 = dst + (tg * 8 + 2 * c) * 33 + nh * 16 + r;
                d0[0]      = acc[tg][nh][0];
                d0[33]     = acc[tg][nh][1];
                d0[8]      = acc[tg][nh][2];
                d0[33 + 8] = acc[tg][nh][3];
            }
    }
    __syncthreads();
    if (tl) tl[5] = globaltimer_ns();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            atomicExch(p.error, 1);
            const uint64_t t0 = globaltimer_ns();           // let copies still in flight land before the CTA retires
            while (globaltimer_ns() - t0 < 200000) { }
        }
        __syncthreads();
    }
    const int nloc = wn * kTileN;                           // out-features per CTA (a power of two)
    const int nloc_shift = 31 - __clz(nloc), wk_shift = 31 - __clz(wk);
    const int kRingFloats = ring_bytes / 4;
    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) cluster.sync();                              // every rank's partial sums are in place
    if (tl) tl[6] = globaltimer_ns();

    // fused all-reduce: the epoch is read after the main loop, i.e. after griddepcontrol.wait under programmatic
    // launch - the previous call on this stream has advanced it by then
    const bool fused = p.world > 0;
    ExchangeHeader* hdr = reinterpret_cast<ExchangeHeader*>(p.self);
    const unsigned epoch = fused ? *reinterpret_cast<volatile unsigned*>(&hdr->epoch) : 0u;
    const unsigned half_sel = epoch & 1u, tag = epoch + 1u;

    const uint32_t ring0 = smem_u32(smem + p.ring_offset);   // same offset in every rank's shared memory
    // Rank r finalises a slice of the (tok, n_local) space (n fastest -> coalesced stores).  An output is
    // the sum of S * wk partials - K slice w of rank q lives in the ring of warp (w * wn + n_local / 32) -
    // added in a fixed order (rank-major) from batches of eight loads in flight: deterministic.
    const int terms = S << wk_shift;
    // sum of the S * wk partials of output (token, local out-feature)
    auto total = [&](int tok, int nl) {
        const int off = (nl >> 5) * kRingFloats + tok * 33 + (nl & 31);
        float s = 0.f;
        for (int t0 = 0; t0 < terms; t0 += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = t0 + j, q = t >> wk_shift, w = t & (wk - 1);
                v[j] = t < terms ? ld_cluster_f32(ring0 + (uint32_t)(off + w * wn * kRingFloats) * 4u, (uint32_t)q) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) s += v[j];
        }
        return s;
    };
    // fp32 sum -> fp16, + bias, ReLU: the value a plain call stores
    auto finish = [&](float s, int n) {
        __half h = __float2half_rn(s);
        if (p.bias) h = __hadd(h, p.bias[n]);
        if (p.relu) h = __hmax(h, __half());
        return h;
    };
    const int Er = p.silu_mul ? rows << (nloc_shift - 1) : rows << nloc_shift;
    const int e_lo = div_splits(Er * rank), e_hi = div_splits(Er * (rank + 1));
    // Which outputs a thread finalises.  Default: the rank's flat slice of the (token, out-feature) space dealt over the
    // threads.  With row statistics requested a warp stays inside ONE token row (token = warp % Rp, the row's columns
    // of this rank dealt over the kWarps / Rp warps of the row), so that the sums of a row are per-thread accumulators
    // added in a fixed order.  Both passes of the fused exchange walk the same elements.
    const bool by_row = p.stats_out != nullptr;
    const int rp_shift = rows <= 1 ? 0 : 32 - __clz(rows - 1);                   // Rp = 2^rp_shift >= rows (rows <= kWarps)
    const int row_tok = warp & ((1 << rp_shift) - 1), row_sub = warp >> rp_shift, row_nsub = max(kWarps >> rp_shift, 1);
    const int col_lo = div_splits(nloc * rank), col_hi = div_splits(nloc * (rank + 1));
    const int row_nl0 = col_lo + ((col_hi - col_lo) * row_sub) / row_nsub, row_nl1 = col_lo + ((col_hi - col_lo) * (row_sub + 1)) / row_nsub;
    float st1 = 0.f, st2 = 0.f;                                                  // sum and sum of squares of this thread's outputs
    auto for_each = [&](auto&& body) {
        if (by_row) {
            if (row_tok < rows)
                for (int nl = row_nl0 + lane; nl < row_nl1; nl += 32) body(row_tok, nl);
        } else {
            for (int e = e_lo + threadIdx.x; e < e_hi; e += kThreads) body(e >> nloc_shift, e & (nloc - 1));
        }
    };
    if (p.silu_mul) {
        // SwiGLU epilogue: the out-feature tiles alternate gate, up, gate, up ... (fused that way at load time), so
        // local out-features nl and nl + 32 are a (gate, up) pair of the same hidden unit and one thread owns both:
        // out[t, j] = fp16(silu(gate)) * up, rounded like the separate activation and product kernels it replaces
        // (the reference carries the same epilogue as ops::SiluActivation, gemm_s4_f16.cu:30-40).
        const int half_shift = nloc_shift - 1;
        for (int e = e_lo + threadIdx.x; e < e_hi; e += kThreads) {
            const int tok = e >> half_shift, pl = e & ((nloc >> 1) - 1);
            const int nl = ((pl >> 5) << 6) + (pl & 31);
            const int n = blockIdx.x * nloc + nl;
            if (n + 32 < p.N) {
                const float gate = __half2float(finish(total(tok, nl), n));
                const __half up = finish(total(tok, nl + 32), n + 32);
                const __half act = __float2half_rn(gate / (1.f + __expf(-gate)));
                p.out[(size_t)(tok0 + tok) * (p.N >> 1) + (blockIdx.x << half_shift) + pl] = __hmul(act, up);
            }
        }
    } else {
        for_each([&](int tok, int nl) {
            const float s = total(tok, nl);
            const int n = blockIdx.x * nloc + nl;
            if (n < p.N) {
                if (fused) {
                    // this rank's fp32 partial goes into slot [half][rank] of EVERY rank's exchange buffer (own included)
                    const size_t idx = (size_t)(half_sel * p.world + p.rank) * p.capacity + (size_t)(tok0 + tok) * p.N + n;
#pragma unroll
                    for (int d = 0; d < kExchangeMaxWorld; ++d)
                        if (d < p.world) st_slot(reinterpret_cast<uint2*>(p.peer[d] + kExchangeDataOffset) + idx, make_uint2(__float_as_uint(s), tag));
                } else {
                    __half h = finish(s, n);
                    const size_t idx = (size_t)(tok0 + tok) * p.N + n;
                    if (p.residual) h = __hadd(h, p.residual[idx]);
                    p.out[idx] = h;
                    const float hv = __half2float(h);
                    st1 += hv;
                    st2 += hv * hv;
                }
            }
        });
    }
    if (S > 1) cluster.sync();                              // peers may still be reading this CTA's partials
    if (fused) {
        // Exchange step.  CTA i of every rank covers the same outputs (all ranks launch the same shape) and thread j
        // the same elements, so each thread polls the slots of exactly the elements it pushed: all `world` slots of
        // an element are re-read until every tag is this call's, then the partials are added in rank order - the
        // same order on every rank, so all ranks end up with bit-identical outputs.
        const uint2* data = reinterpret_cast<const uint2*>(p.self + kExchangeDataOffset) + (size_t)half_sel * p.world * p.capacity;
        // once a wait has given up the buffer stays marked and later calls do not wait at all: the job is lost
        // either way and must not take seconds per call to find out
        bool dead = *reinterpret_cast<volatile int*>(&hdr->error) != 0;
        for_each([&](int tok, int nl) {
            const int n = blockIdx.x * nloc + nl;
            if (n >= p.N) return;
            const size_t idx = (size_t)(tok0 + tok) * p.N + n;
            uint2 v[kExchangeMaxWorld];
            uint64_t t0 = 0;
            for (uint32_t polls = 0;; ++polls) {
                bool all = true;
#pragma unroll
                for (int src = 0; src < kExchangeMaxWorld; ++src)
                    if (src < p.world) {
                        v[src] = ld_slot(data + (size_t)src * p.capacity + idx);
                        all = all && v[src].y == tag;
                    }
                if (all || dead) break;
                if ((polls & 255u) == 255u) {
                    const uint64_t now = globaltimer_ns();
                    if (t0 == 0) t0 = now;
                    if (now - t0 > p.wait_budget_ns) {
                        int late = 0;
#pragma unroll
                        for (int src = 0; src < kExchangeMaxWorld; ++src)
                            if (src < p.world && v[src].y != tag) late = src;
                        atomicExch(p.error, 2);
                        atomicExch(&hdr->error, 1 + late);
                        dead = true;
                    }
                }
            }
            float s = __uint_as_float(v[0].x);
#pragma unroll
            for (int src = 1; src < kExchangeMaxWorld; ++src)
                if (src < p.world) s += __uint_as_float(v[src].x);
            __half h = finish(s, n);
            if (p.residual) h = __hadd(h, p.residual[idx]);
            p.out[idx] = h;
            const float hv = __half2float(h);
            st1 += hv;
            st2 += hv * hv;
        });
        __syncthreads();
        // the last CTA to get here advances the epoch; the next call then uses the other half of the buffers
        if (threadIdx.x == 0) {
            const unsigned done = atomicAdd(&hdr->ticket, 1u);
            if (done == gridDim.x * gridDim.y - 1) {
                hdr->ticket = 0;
                __threadfence();
                *reinterpret_cast<volatile unsigned*>(&hdr->epoch) = epoch + 1;
            }
        }
    }
    if (by_row) {
        // row statistics of this CTA's outputs: lanes, then the warps of a row in index order, then one store per row
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            st1 += __shfl_xor_sync(0xffffffffu, st1, o);
            st2 += __shfl_xor_sync(0xffffffffu, st2, o);
        }
        float2* red = reinterpret_cast<float2*>(smem + kStatsOffset);            // [kWarps]
        if (lane == 0) red[warp] = make_float2(st1, st2);
        __syncthreads();
        if ((int)threadIdx.x < rows) {
            float a = 0.f, b = 0.f;
            for (int sub = 0; sub < row_nsub; ++sub) {
                const float2 v = red[(sub << rp_shift) + threadIdx.x];
                a += v.x;
                b += v.y;
            }
            const int part = blockIdx.x * S + rank;
            reinterpret_cast<float2*>(p.stats_out + kStatsHeaderFloats)[(size_t)part * kStatsRows + tok0 + threadIdx.x] = make_float2(a, b);
        }
        if (threadIdx.x == 0 && blockIdx.x == 0 && rank == 0) *reinterpret_cast<int*>(p.stats_out) = (int)gridDim.x * S;
    }
    if (tl) tl[7] = globaltimer_ns();
}

struct Config { int tg, wn, splits, depth, warps; };

int g_force_wn = 0, g_force_splits = 0, g_force_depth = 0, g_debug_mode = 0;
unsigned long long* g_timeline = nullptr;

constexpr int kSmemBudget = 227 * 1024;                  // opt-in shared memory of one CTA on sm_100

int slot_bytes(int g, int uk) { return (uk / kTileK) * 512 + (uk / g) * 128; }

// shared memory the activations of one CTA need: [header 1 KB][rows x (K/S + 8) halfs], 128-byte aligned
int xs_bytes(int rows, int K, int splits, int kUnitK)
{
    const int units = (K + kUnitK - 1) / kUnitK;
    const int cta_units = (units + splits - 1) / splits;
    const int bytes = (int)(((size_t)rows * (cta_units * kUnitK + 8) * sizeof(__half) + 127) / 128 * 128);
    return bytes < 1152 ? 1152 : bytes;                 // the fused normalisation uses the area as reduction scratch first
}

int xsum_bytes(int tg, int K, int splits, int kUnitK, int g)
{
    const int units = (K + kUnitK - 1) / kUnitK;
    const int cta_units = (units + splits - 1) / splits;
    return ((cta_units * kUnitK / g) * 8 * tg * (int)sizeof(float) + 127) / 128 * 128;
}

int stage_bytes(int rows, int K, int splits, int kUnitK, int tg, int g)
{
    return kHeaderBytes + xs_bytes(rows, K, splits, kUnitK) + xsum_bytes(tg, K, splits, kUnitK, g);
}

// How many clusters of `sp` CTAs of this kernel the current device runs at once (the kernel takes a whole SM per CTA,
// so this is a property of how the SMs are grouped into GPCs, not of the problem).  Cached per device and size.
template <int TG, int G>
int max_clusters_instance(int sp)
{
    static int cache[64][9] = {};      // benign race: the query is idempotent
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return device_sm_count() / sp;
    if (cache[dev][sp]) return cache[dev][sp];
    int n = 0;
    const int smem = 200 * 1024;
    if (cudaFuncSetAttribute(skinny_kernel<TG, G, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, sp, 1);
        cfg.blockDim = dim3(512);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = sp;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, skinny_kernel<TG, G, 16>, &cfg) != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
    } else {
        (void)cudaGetLastError();
    }
    if (n <= 0) n = device_sm_count() / sp;          // query unavailable: assume perfect packing
    cache[dev][sp] = n;
    return n;
}

int max_clusters(int tg, int g, int sp)
{
    if (sp <= 1) return device_sm_count();
    if (tg != 4) return device_sm_count() / sp;
    switch (g) {
        case 128: return max_clusters_instance<4, 128>(sp);
        case 64:  return max_clusters_instance<4, 64>(sp);
        default:  return max_clusters_instance<4, 32>(sp);
    }
}

Config pick_config(int tokens, int N, int K, int g, int max_tg = 4, int min_wn = 1)
{
    Config c;
    c.tg = tokens <= 8 ? 1 : (tokens <= 16 ? 2 : 4);
    if (c.tg > max_tg) c.tg = max_tg;
    const int kUnitK = unit_k_for(c.tg);
    const int n_tiles = N / kTileN, units = (K + kUnitK - 1) / kUnitK;
    const int rows = tokens < 8 * c.tg ? tokens : 8 * c.tg;
    c.warps = 16;
    const int kWarps = c.warps;
    const int ring1 = kWarps * slot_bytes(g, kUnitK);    // one unit per warp
    // cluster split-K only as far as needed for the staged activations to fit next to a ring of depth >= 2
    c.splits = g_force_splits ? g_force_splits : 1;
    while (!g_force_splits && c.splits < 8 && units >= 2 * c.splits &&
           stage_bytes(rows, K, c.splits, kUnitK, c.tg, g) + 2 * ring1 > kSmemBudget) c.splits <<= 1;
    c.depth = (kSmemBudget - stage_bytes(rows, K, c.splits, kUnitK, c.tg, g)) / ring1;
    if (c.depth > max_depth_for(c.tg)) c.depth = max_depth_for(c.tg);
    if (g_force_depth && g_force_depth < c.depth) c.depth = g_force_depth;
    // out-feature tiles per CTA: about one CTA per SM in a single wave
    c.wn = min_wn;
    const int sms = device_sm_count();
    while (c.wn < kWarps && (long long)((n_tiles + c.wn - 1) / c.wn) * c.splits > sms) c.wn <<= 1;
    // every K slice of a CTA should own at least one 128-k unit
    while (c.wn < kWarps && (kWarps / c.wn) * c.splits > units) c.wn <<= 1;
    if (g_force_wn) c.wn = g_force_wn;
    if (c.tg == 4 && !g_force_wn && !g_force_splits) {
        // 17..32 tokens: the staged activations crowd out the rings, and power-of-two clusters often leave a third
        // of the SMs idle (e.g. 384 out-feature tiles: 48 x 2 CTAs).  Search all (tiles per CTA, cluster size <= 8)
        // for the most CTAs within one wave, weighted by how deep a ring still fits; ties go to the smaller cluster.
        double best = -1.0;
        for (int wn = min_wn; wn <= kWarps; wn <<= 1) {
            for (int sp = 1; sp <= 8; ++sp) {
                if (sp > units) break;
                const long long ctas = (long long)((n_tiles + wn - 1) / wn) * sp;
                if (ctas > sms || ctas / sp > max_clusters(c.tg, g, sp)) continue;      // one wave, as the device packs clusters
                const int room = kSmemBudget - stage_bytes(rows, K, sp, kUnitK, c.tg, g);
                int depth = room / ring1;
                if (depth < 2) continue;
                if (depth > max_depth_for(c.tg)) depth = max_depth_for(c.tg);
                if (g_force_depth && g_force_depth < depth) depth = g_force_depth;
                const double score = (double)ctas * (depth >= 4 ? 1.0 : depth == 3 ? 0.9 : 0.7) - 0.01 * sp;
                if (score > best) { best = score; c.wn = wn; c.splits = sp; c.depth = depth; }
            }
        }
        if (best < 0) { c.splits = 8; c.depth = 0; }      // nothing fits in one wave: two passes of 16 tokens (no exchange) or refused
    }
    return c;
}

template <int TG, int G, int kWarps, bool kPreNorm = false>
int launch_instance(const CUtensorMap& wmap, const SkinnyParams& p, dim3 grid, size_t smem, cudaStream_t st)
{
    static int configured_dev[64] = {0};   // benign race: the attribute call is idempotent
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    static int max_optin[64] = {0};
    if (dev < 64 && !max_optin[dev]) {
        int v = 0;
        e = cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (e != cudaSuccess) return record_cuda_error(e);
        max_optin[dev] = v;
    }
    if (dev < 64 && (int)smem > max_optin[dev]) return W4A16_ERR_BAD_SHAPE;
    if (dev >= 64 || configured_dev[dev] < (int)smem) {
        e = cudaFuncSetAttribute(skinny_kernel<TG, G, kWarps, kPreNorm>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev < 64) configured_dev[dev] = (int)smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = grid.y;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, skinny_kernel<TG, G, kWarps, kPreNorm>, wmap, p);
    count_launch();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

template <int G>
int launch_g(int tg, const CUtensorMap& wmap, const SkinnyParams& p, dim3 grid, size_t ring_bytes, cudaStream_t st)
{
    const size_t smem = (size_t)p.ring_offset + ring_bytes;
    if (p.norm_w) {                         // at most 16 tokens (checked by launch_skinny)
        return tg == 1 ? launch_instance<1, G, 16, true>(wmap, p, grid, smem, st) : launch_instance<2, G, 16, true>(wmap, p, grid, smem, st);
    }
    switch (tg) {
        case 1: return launch_instance<1, G, 16>(wmap, p, grid, smem, st);
        case 2: return launch_instance<2, G, 16>(wmap, p, grid, smem, st);
        default: return launch_instance<4, G, 16>(wmap, p, grid, smem, st);
    }
}

}  // namespace

void skinny_set_timeline(unsigned long long* buf) { g_timeline = buf; }

void skinny_force_config(int wn, int splits)
{
    g_force_wn = wn < 0 ? 0 : wn;
    g_force_splits = splits < 0 ? 0 : splits;
}
// debug builds: experiment switches of the kernel (bit 0 no MMAs, bit 1 no activation staging) and a ring-depth cap
void skinny_debug_mode(int mode, int depth) { g_debug_mode = mode; g_force_depth = depth; }

int g_decode_kernel = 0;      // 0: by measured crossover, 1: always the 16-warp kernel, 2: always the two-CTAs-per-SM kernel
void decode_force_kernel(int which) { g_decode_kernel = which; }

int launch_skinny(const GemmArgs& a, cudaStream_t st)
{
    if (a.tokens == 0) return W4A16_OK;
    // Which decode kernel: measured on B200 in CUDA graphs of dependent launches, the two-CTAs-per-SM kernel wins at
    // 5..8 tokens on matrices of up to ~9 MB (4096 x 4096 and every tensor-parallel shard of the OPT / LLaMA
    // shapes: 3.2-5.1 us against 4.5-5.4 us), where the launch ramp it hides is most of the call; the 16-warp
    // single-CTA kernel below, whose main loop issues fewer instructions per tile, wins on larger matrices and at 1..4
    // tokens.
    const bool small = (long long)a.K * a.N <= 20ll * 1000 * 1000;
    if (a.norm_weight || a.row_stats_out) {
        // normalisation folded into the GEMV / row statistics for the next one: one pass of at most 16 tokens in
        // the one-CTA-per-SM kernel
        if (a.tokens > 16 || (a.K % 8) || a.silu_mul && a.row_stats_out) return W4A16_ERR_BAD_ALGO;
        if (a.norm_weight && !a.row_stats_in) return W4A16_ERR_NULL_POINTER;
        if (a.norm_weight && a.K > 2 * 512 * 8) return W4A16_ERR_BAD_ALGO;   // two column vectors per thread
    } else
    if (g_decode_kernel == 2 || (g_decode_kernel == 0 && a.tokens >= 5 && a.tokens <= 8 && small)) return launch_gemv(a, st);
    // with the fused exchange every rank must launch the same shape: choose it from the K all ranks agreed on
    const int k_config = a.exchange ? a.exchange->k_config : a.K;
    if (k_config < a.K) return W4A16_ERR_BAD_SHAPE;
    const int min_wn = a.silu_mul ? 2 : 1;                 // a (gate, up) pair of tiles stays inside one CTA
    if (a.silu_mul && ((a.N % 64) || a.exchange || a.residual)) return W4A16_ERR_BAD_SHAPE;
    Config c = pick_config(a.tokens, a.N, k_config, a.g, 4, min_wn);
    // 17..32 tokens with a K so long that the staged activations need clusters of 8 CTAs: such clusters do not
    // always fit the machine in one wave; two passes of 16 tokens (gridDim.z, the second one reading the weights
    // from L2) are faster.  Not with the fused exchange, which needs all tokens in one pass.
    if (c.tg == 4 && c.splits >= 8 && !a.exchange && !g_force_splits) c = pick_config(a.tokens, a.N, k_config, a.g, 2, min_wn);
    if (c.depth < 2) return W4A16_ERR_BAD_SHAPE;         // forced configuration does not fit in shared memory
    const int kUnitK = unit_k_for(c.tg), kUnitTiles = kUnitK / kTileK;
    const int units = (a.K + kUnitK - 1) / kUnitK;
    if (c.splits > (k_config + kUnitK - 1) / kUnitK) c.splits = 1;
    const int kWarps = c.warps;
    if (c.wn != 1 && c.wn != 2 && c.wn != 4 && c.wn != 8 && c.wn != 16 && c.wn != 32) return W4A16_ERR_BAD_ALGO;
    if (c.wn > kWarps || c.wn < min_wn) return W4A16_ERR_BAD_ALGO;
    if (c.splits < 1 || c.splits > 8) return W4A16_ERR_BAD_ALGO;

    SkinnyParams p;
    p.x = a.x; p.qw = reinterpret_cast<const uint4*>(a.qw); p.zs = a.zs; p.bias = a.bias; p.out = a.out;
    p.error = a.plan_only ? nullptr : device_error_word();
    if (!p.error && !a.plan_only) return W4A16_ERR_CUDA;
    p.world = 0; p.rank = 0; p.capacity = 0; p.self = nullptr; p.wait_budget_ns = exchange_wait_budget_ns();
    for (int d = 0; d < kExchangeMaxWorld; ++d) p.peer[d] = nullptr;
    if (a.exchange) {
        const ExchangeArgs& x = *a.exchange;
        if (x.world < 1 || x.world > kExchangeMaxWorld || x.rank < 0 || x.rank >= x.world) return W4A16_ERR_BAD_SHAPE;
        if (a.tokens > 8 * c.tg) return W4A16_ERR_TOO_LARGE;                          // one pass of at most 32 tokens
        if ((long long)a.tokens * a.N > x.capacity) return W4A16_ERR_TOO_LARGE;
        for (int d = 0; d < x.world; ++d) {
            if (!x.peer[d]) return W4A16_ERR_NULL_POINTER;
            p.peer[d] = x.peer[d];
        }
        p.world = x.world; p.rank = x.rank; p.capacity = x.capacity; p.self = x.peer[x.rank];
    }
    p.wn_shift = 0;
    while ((1 << p.wn_shift) < c.wn) ++p.wn_shift;
    p.inv_splits = c.splits > 1 ? (unsigned)(((1ull << 32) + c.splits - 1) / c.splits) : 0u;
    p.tokens = a.tokens; p.N = a.N; p.K = a.K; p.wn = c.wn; p.splits = c.splits; p.debug_mode = g_debug_mode; p.timeline = g_timeline; p.depth = c.depth; p.warps = c.warps; p.pdl = a.static_weights ? 1 : 0; p.relu = a.relu ? 1 : 0;
    p.residual = a.residual; p.silu_mul = a.silu_mul ? 1 : 0;
    p.norm_w = a.norm_weight; p.norm_b = a.norm_bias; p.norm_eps = a.norm_eps; p.norm_rms = a.norm_rms ? 1 : 0;
    p.stats_in = a.row_stats_in; p.stats_out = a.row_stats_out;
    const int max_cta_units = (units + c.splits - 1) / c.splits;
    p.xs_stride = max_cta_units * kUnitK + 8;           // +16 B: ldmatrix rows fall in distinct banks
    const int tok = 8 * c.tg;
    const int rows = a.tokens < tok ? a.tokens : tok;
    p.xsum_offset = kHeaderBytes + xs_bytes(rows, a.K, c.splits, kUnitK);
    p.ring_offset = p.xsum_offset + xsum_bytes(c.tg, a.K, c.splits, kUnitK, a.g);
    const int n_tiles = a.N / kTileN;
    dim3 grid((n_tiles + c.wn - 1) / c.wn, c.splits, (a.tokens + tok - 1) / tok);
    if (grid.z > 65535) return W4A16_ERR_BAD_SHAPE;
    if (a.exchange && grid.z != 1) return W4A16_ERR_TOO_LARGE;
    // the ranks spin on each other inside the kernel: every CTA of the grid must be resident at once
    if (a.exchange && (long long)grid.x * grid.y > device_sm_count()) return W4A16_ERR_TOO_LARGE;
    if ((a.norm_weight || a.row_stats_out) && grid.z != 1) return W4A16_ERR_BAD_ALGO;
    if (a.plan_only) return (a.g == 128 || a.g == 64 || a.g == 32) ? W4A16_OK : W4A16_ERR_GROUP_SIZE;
    // the packed matrix as a 2-D tensor of 32-bit words: [K/32 rows][N/32 * 128 words], box = 4 rows x 128 words
    CUtensorMap wmap;
    {
        const uint64_t dims[2] = {(uint64_t)n_tiles * 128, (uint64_t)(a.K / kTileK)};
        const uint64_t stride_bytes = (uint64_t)n_tiles * 512;
        const uint32_t box[2] = {128, (uint32_t)kUnitTiles};
        int s = encode_tensor_map_2d(&wmap, a.qw, /*u32*/ 4, dims, stride_bytes, box, /*swizzle128*/ false);
        if (s != W4A16_OK) return s;
    }
    switch (a.g) {
        case 128: return launch_g<128>(c.tg, wmap, p, grid, (size_t)kWarps * c.depth * slot_bytes(128, kUnitK), st);
        case 64:  return launch_g<64>(c.tg, wmap, p, grid, (size_t)kWarps * c.depth * slot_bytes(64, kUnitK), st);
        case 32:  return launch_g<32>(c.tg, wmap, p, grid, (size_t)kWarps * c.depth * slot_bytes(32, kUnitK), st);
        default:  return W4A16_ERR_GROUP_SIZE;
    }
}

}  // namespace w4a16
