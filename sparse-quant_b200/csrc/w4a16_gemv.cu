// Decode kernel for at most 16 tokens per pass: W4A16 GEMV / skinny GEMM, HBM-bandwidth bound.
//
//   out[t, n] = fp16( sum_k fp32( dq(W)[n, k] * x[t, k] ) ) (+ bias[n])
//
// Replaces the small-token instantiations of gemm_s4_f16_nn (gemm_template.h:358-464 of the reference, CTA shapes
// (x, 8|16, 256|512) of gemm_s4_f16.cu:66-87).  Design points, all aimed at keeping HBM busy across launches of a
// decode step, where one call moves only 9-36 MB:
//
//   * a CTA is 8 warps and at most 112 KB of shared memory, so that TWO CTAs fit on an SM: launched with
//     programmatic stream serialization, the CTAs of the next GEMV become resident while this one still computes,
//     fill their rings with packed weights (static by contract) and only then wait for this grid to finish before
//     they touch activations or outputs.  The launch ramp, the barrier set-up and the first DRAM round trip of a
//     call overlap the previous call's arithmetic and tail;
//   * a warp owns one 32-wide out-feature tile and a contiguous K slice, and keeps a private ring of TMA copies in
//     flight: per 128-k unit one tensor copy (four strided 512-byte tiles of the packed matrix seen as
//     [K/32][N/32 x 512 B]) plus one 128-byte bulk copy per quantisation group of its (zero, scale) pairs, all
//     completing on the unit's mbarrier;
//   * activations are NOT staged up front: they flow through a ring as well, one [rows x 128 k] chunk per unit and K
//     slice, fetched by TMA (128-byte swizzle, so the ldmatrix reads are conflict free; rows past the batch are
//     zero-filled by the copy engine) and shared by the warps of the CTA that cover the same K slice with different
//     out-feature tiles.  The warp that fetches a chunk also computes sum_k x per quantisation group (two extra MMAs
//     per tile with a constant A fragment) and publishes it to its siblings through shared memory;
//   * the nibbles are only masked in place (one shift + four ANDs per eight weights), which leaves subnormal fp16
//     patterns q * 2^-24 / q * 2^-20 that the tensor core multiplies exactly, fed straight to mma.m16n8k16 as the A
//     fragment (the packed layout IS that fragment).  At the end of each quantisation group zero point and scale
//     are applied in fp32:  acc += s * (sum q x - z sum x), i.e. (q - z) * s without the intermediate fp16 rounding
//     of the weight; with the identity matrix as input the output reproduces the reference's dequantised weight
//     (denormal scales are flushed to zero as mul.ftz does);
//   * split-K: the K slices of a CTA meet in shared memory, the CTAs of a thread-block cluster (only used when the
//     out-feature tiles alone do not fill the machine) through distributed shared memory, both in a fixed order:
//     deterministic, no global scratch, no atomics;
//   * bias add, optional ReLU, fp16 rounding and the [tokens, N] store - or the all-reduce over peer memory of a
//     row-parallel linear - are fused into the reduction.
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
constexpr bool kDebug = true;     // phase time stamps compiled in
#else
constexpr bool kDebug = false;
#endif

constexpr int kWarps = 16, kThreads = kWarps * 32;            // 64 registers per thread: two CTAs per SM
constexpr int kUnitK = 128, kUnitTiles = kUnitK / kTileK;     // k per pipeline unit
constexpr int kMaxDepth = 4;                                  // most units in flight per warp
constexpr int kHeaderBytes = 1024;                            // zero chunk, abort flag, mbarriers
constexpr int kBarBase = 64;                                  // byte offset of the barrier table in the header
constexpr int kSmemBudget = 113 * 1024 - 512;                 // two CTAs of this kernel (plus 1 KB each for the system) fit on one SM
constexpr int kSmemMax = 227 * 1024;                          // opt-in limit of one CTA
constexpr uint64_t kWaitBudgetNs = 200ull * 1000 * 1000;
static_assert(kBarBase + kWarps * kMaxDepth * 8 <= kHeaderBytes, "header overflow");

struct GemvParams {
    const uint32_t* zs;
    const __half*   bias;
    __half*         out;
    int*            error;         // [0] device error word, [1] generation counter (bumped when a grid's work is done)
    int tokens, N, K;
    int tn_shift;          // log2(out-feature tiles per CTA); 16 >> tn_shift K slices per CTA
    int real_x;            // CTAs along x that have work; the rest only hold their SM's second slot (see kernel)
    int splits;            // cluster size along K (gridDim.y)
    unsigned inv_splits;   // ceil(2^32 / splits)
    int depth;             // units in flight per warp
    int ahead;             // units further ahead that are prefetched into L2
    int rp;                // activation rows per TMA box: 1, 2, 4 or 8
    int swizzled;          // the activation boxes use the 128-byte swizzle
    int x_offset, w_offset;   // byte offsets in dynamic shared memory (x_offset before rounding up to 1024)
    int relu, pdl;
    const __half* residual;   // [tokens, N] added to the output after bias / ReLU (fp16 add), or null
    int silu_mul;          // out-feature tiles alternate gate / up; out[t, j] = silu(gate_j) * up_j, [tokens, N / 2]
    // fused all-reduce over peer memory (world == 0: plain store of this GPU's result)
    unsigned char* peer[kExchangeMaxWorld];
    unsigned char* self;
    int world, rank;
    long long capacity;
    unsigned long long wait_budget_ns;   // how long the exchange waits for a peer
    unsigned long long* timeline;        // debug: [cta][warp][8] globaltimer stamps, or null
};

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
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank)
{
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr)
{
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void l2_prefetch_2d(const void* tmap, int c0, int c1)
{
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// G = quantisation group size.  At most 8 tokens per pass.
template <int G>
__global__ void __launch_bounds__(kThreads, 2)
gemv_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap, const GemvParams p)
{
    extern __shared__ __align__(1024) unsigned char smem[];
    constexpr int kTok = 8;
    constexpr int kGroupsPerUnit = kUnitK / G;
    constexpr int kTilesPerGroup = G / kTileK;
    constexpr int kSlotBytes = kUnitTiles * 512 + kGroupsPerUnit * 128;      // packed tiles + (zero, scale) rows
    static_assert(2 * kSlotBytes >= kTok * 33 * 4, "a warp's partial sums reuse its own ring (depth >= 2)");

    if ((int)blockIdx.x >= p.real_x) {
        // A CTA without work.  Under programmatic launch two grids share every SM: the one that computes and the
        // next one, which prefetches and waits.  That only balances when every SM holds exactly ONE CTA of each
        // grid; a grid with fewer CTAs than SMs would let the next grid put two of its CTAs on the SMs it left
        // free, and those two would later compute at half speed each.  So the grid is padded to one CTA per SM and
        // the padding CTAs keep their slot until the grid's work is done: they wait for the previous grid like
        // everyone else and then for CTA 0 of this grid to bump the generation word (bounded; the word is a
        // performance hint only, a missed or early bump costs balance, never correctness).
        if (threadIdx.x == 0) {
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            asm volatile("griddepcontrol.wait;" ::: "memory");
            const volatile int* gen = p.error + 1;
            const int g0 = *gen;
            const uint64_t t0 = globaltimer_ns();
            while (*gen == g0 && globaltimer_ns() - t0 < 200000ull) __nanosleep(256);
        }
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tn = 1 << p.tn_shift, wk = kWarps >> p.tn_shift;
    const int tn_idx = warp & (tn - 1), slice = warp >> p.tn_shift;
    const int wk_sh = 31 - __clz(wk);
    const int n_tiles = p.N / kTileN;
    const int nt = blockIdx.x * tn + tn_idx;
    const bool nt_valid = nt < n_tiles;
    const int tok0 = blockIdx.z * kTok;
    const int rows = min(kTok, p.tokens - tok0);

    // K decomposition in 128-k units: cluster rank -> CTA range -> K slice of the warp
    const int k_tiles = p.K / kTileK;
    const int groups = p.K / G;
    const int units = (p.K + kUnitK - 1) / kUnitK;
    const int S = p.splits, crank = blockIdx.y;
    auto div_splits = [&](int x) { return S == 1 ? x : (int)__umulhi((unsigned)x, p.inv_splits); };
    const int cu0 = div_splits(units * crank), cu1 = div_splits(units * (crank + 1));
    const int cta_units = cu1 - cu0;
    const int wu0 = cu0 + ((cta_units * slice) >> wk_sh), wu1 = cu0 + ((cta_units * (slice + 1)) >> wk_sh);
    const int n_units = nt_valid ? wu1 - wu0 : 0;

    // shared memory: [16 B zeros][abort flag] [barriers: warp x stage] | activation chunks (1024-aligned) | packed tiles
    const uint32_t smem0 = smem_u32(smem);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 16);
    const int depth = p.depth;
    const int xchunk = p.rp * 256;                                             // [rp rows][128 k] fp16
    const uint32_t xring = ((smem0 + p.x_offset + 1023u) & ~1023u) + (uint32_t)(warp * depth * xchunk);
    const uint32_t wring = smem0 + p.w_offset + (uint32_t)(warp * depth * kSlotBytes);
    const uint32_t bars = smem0 + kBarBase + warp * kMaxDepth * 8;

    unsigned long long* tl = nullptr;
    if (kDebug && p.timeline && lane == 0)
        tl = p.timeline + ((size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + warp) * 8;
    if (tl) tl[0] = globaltimer_ns();

    if (threadIdx.x == 0) *abort_flag = 0;
    if (threadIdx.x < 4) reinterpret_cast<uint32_t*>(smem)[threadIdx.x] = 0u;
    if (lane < depth) mbar_init(bars + lane * 8, 1);
    mbar_fence_init();
    __syncwarp();

    // lane 0 keeps the issue state of the warp: next unit to fetch into the ring and next unit to prefetch into L2
    const size_t zs_step = (size_t)kGroupsPerUnit * p.N;                       // words between consecutive units
    const uint32_t* zs_base = p.zs + (size_t)wu0 * zs_step + nt * kTileN;      // (zero, scale) rows of this warp's first unit
    // packed tiles and (zero, scale) rows of unit wu0 + i; the unit's barrier also expects its activation chunk
    auto issue_w = [&](int i, int slot) {
        const int u = wu0 + i;
        const uint32_t bar = bars + slot * 8;
        const uint32_t dst = wring + (uint32_t)(slot * kSlotBytes);
        const int n_groups = min(kGroupsPerUnit, groups - u * kGroupsPerUnit);  // < full only at the K edge
        // the tensor copies always deliver their full boxes (rows / columns past the tensor arrive as zeros)
        mbar_arrive_expect_tx(bar, kUnitTiles * 512u + (uint32_t)n_groups * 128u + (uint32_t)xchunk);
        tma_load_2d(dst, &wmap, nt * 128, u * kUnitTiles, bar);
        const uint32_t* zsrc = zs_base + (size_t)i * zs_step;
#pragma unroll
        for (int gi = 0; gi < kGroupsPerUnit; ++gi)
            if (gi < n_groups) bulk_load(dst + kUnitTiles * 512u + gi * 128u, zsrc + (size_t)gi * p.N, 128u, bar);
    };
    auto issue_x = [&](int i, int slot) {
        const int u = wu0 + i;
        const uint32_t dst = xring + (uint32_t)(slot * xchunk);
        if (p.swizzled) {                                                       // two boxes of [rp][64 halfs], 128-byte swizzle
            tma_load_2d(dst, &xmap, u * kUnitK, tok0, bars + slot * 8);
            tma_load_2d(dst + (uint32_t)p.rp * 128u, &xmap, u * kUnitK + 64, tok0, bars + slot * 8);
        } else {                                                                // one box of [rp][128 halfs]
            tma_load_2d(dst, &xmap, u * kUnitK, tok0, bars + slot * 8);
        }
    };
    auto prefetch_w = [&](int i) {                                              // unit wu0 + i -> L2
        const int u = wu0 + i;
        l2_prefetch_2d(&wmap, nt * 128, u * kUnitTiles);
        if (u * kGroupsPerUnit < groups) l2_prefetch(zs_base + (size_t)i * zs_step, 128u);
    };

    // The packed weights are static by contract: under programmatic launch their copies start while the previous
    // kernel of the stream is still running; activations and everything this kernel writes wait for it to complete.
    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (lane == 0) {
        if (warp == 0) { prefetch_tmap(&wmap); prefetch_tmap(&xmap); }
        for (int i = 0; i < depth && i < n_units; ++i) issue_w(i, i);
        for (int i = depth; i < depth + p.ahead && i < n_units; ++i) prefetch_w(i);
    }
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tl) tl[1] = globaltimer_ns();
    if (lane == 0)
        for (int i = 0; i < depth && i < n_units; ++i) issue_x(i, i);

    float acc[2][4];
#pragma unroll
    for (int nh = 0; nh < 2; ++nh)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[nh][j] = 0.f;

    if (n_units > 0) {
        const int r = lane >> 2;
        // ldmatrix row addresses inside an activation chunk: matrix j = lane / 8 covers k offset 8j of a 32-k tile,
        // row = token lane % 8.  Offsets are relative to the chunk start (a multiple of 1024 bytes whenever the
        // swizzle is on, so the swizzle term does not depend on the stage).  Rows the copy does not deliver
        // (token >= rp) read the 16 zero bytes at the start of shared memory.
        const bool xreal = (lane & 7) < p.rp;
        uint32_t xoff[kUnitTiles];
#pragma unroll
        for (int t = 0; t < kUnitTiles; ++t) {
            uint32_t logical;
            if (p.swizzled) {
                logical = (uint32_t)((t >> 1) * p.rp * 128 + (lane & 7) * 128 + (t & 1) * 64 + (lane >> 3) * 16);
                logical ^= ((logical >> 7) & 7u) << 4;
            } else {
                logical = (uint32_t)((lane & 7) * 256 + t * 64 + (lane >> 3) * 16);
            }
            xoff[t] = xreal ? logical : 0u;
        }
        const uint32_t wlane = wring + (uint32_t)lane * 16u;
        const uint32_t zlane = wring + kUnitTiles * 512u + (uint32_t)r * 4u;
        constexpr uint32_t kOnesLo = 0x00010001u, kOnesHi = 0x00100010u;       // 2^-24 (rows r) and 2^-20 (rows r + 8)
        const uint32_t ones[4] = {kOnesLo, kOnesHi, kOnesLo, kOnesHi};

        int slot = 0;
        uint32_t phase = 0;
        for (int i = 0; i < n_units; ++i) {
            const bool ok = mbar_wait(bars + slot * 8, phase, abort_flag, kWaitBudgetNs);
            if (!__all_sync(0xffffffffu, ok)) break;
            if (tl && i == 0) tl[2] = globaltimer_ns();

            const int u = wu0 + i;
            const uint32_t wb = wlane + (uint32_t)(slot * kSlotBytes);
            const uint32_t zb = zlane + (uint32_t)(slot * kSlotBytes);
            const uint32_t xb = xreal ? xring + (uint32_t)(slot * xchunk) : smem0;
#pragma unroll
            for (int gi = 0; gi < kGroupsPerUnit; ++gi) {
                if ((u * kUnitTiles + gi * kTilesPerGroup) < k_tiles) {          // warp-uniform: the group exists
                    // xs: sum_k x of the group, scaled by 2^-24 (entries 0, 1: tokens 2c, 2c+1 for rows r) and 2^-20
                    // (entries 2, 3: the same tokens for rows r + 8), from an MMA with a constant A fragment
                    float accg[2][4], xs[4];
#pragma unroll
                    for (int tt = 0; tt < kTilesPerGroup; ++tt) {
                        const int t = gi * kTilesPerGroup + tt;
                        uint32_t b[4];
                        ldmatrix_x4(b, xb + xoff[t]);
                        const uint4 q = ld_shared_v4(wb + t * 512);
                        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int kh = 0; kh < 2; ++kh) {
                            uint32_t a0[4], a1[4];
                            unpack_s4x8_denorm(words[kh * 2 + 0], a0);
                            unpack_s4x8_denorm(words[kh * 2 + 1], a1);
                            if (tt == 0 && kh == 0) {
                                mma_m16n8k16_zc(accg[0], a0, b[0], b[1]);
                                mma_m16n8k16_zc(accg[1], a1, b[0], b[1]);
                                mma_m16n8k16_zc(xs, ones, b[0], b[1]);
                            } else {
                                mma_m16n8k16(accg[0], a0, b[2 * kh], b[2 * kh + 1]);
                                mma_m16n8k16(accg[1], a1, b[2 * kh], b[2 * kh + 1]);
                                mma_m16n8k16(xs, ones, b[2 * kh], b[2 * kh + 1]);
                            }
                        }
                    }
                    // zero point and scale of the group in fp32; the accumulators stay scaled by 2^-24 / 2^-20 until the end
                    constexpr uint32_t kOnes = 0x3c003c00u;
#pragma unroll
                    for (int nh = 0; nh < 2; ++nh) {
#pragma unroll
                        for (int hi = 0; hi < 2; ++hi) {
                            // (zero + 64, scale) * (1, 1) with flush-to-zero: a denormal scale becomes 0, as under mul.ftz
                            uint32_t v = ld_shared_u32(zb + (uint32_t)(gi * 128 + (nh * 16 + hi * 8) * 4));
                            asm("mul.ftz.f16x2 %0, %1, %2;" : "=r"(v) : "r"(v), "r"(kOnes));
                            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
                            const float nz = 64.f - f.x;
                            acc[nh][2 * hi + 0] = fmaf(f.y, fmaf(nz, xs[2 * hi + 0], accg[nh][2 * hi + 0]), acc[nh][2 * hi + 0]);
                            acc[nh][2 * hi + 1] = fmaf(f.y, fmaf(nz, xs[2 * hi + 1], accg[nh][2 * hi + 1]), acc[nh][2 * hi + 1]);
                        }
                    }
                }
            }
            __syncwarp();                                   // every lane is done reading the unit's slot
            if (sm100::elect_one()) {
                if (i + depth < n_units) { issue_w(i + depth, slot); issue_x(i + depth, slot); }
                if (i + depth + p.ahead < n_units) prefetch_w(i + depth + p.ahead);
            }
            if (++slot == depth) { slot = 0; phase ^= 1u; }
        }
    }
#pragma unroll
    for (int nh = 0; nh < 2; ++nh) {
        acc[nh][0] *= kDenormScaleLo; acc[nh][1] *= kDenormScaleLo;
        acc[nh][2] *= kDenormScaleHi; acc[nh][3] *= kDenormScaleHi;
    }

    if (tl) tl[3] = globaltimer_ns();
    // ---- reduction: warps -> CTA (shared memory), CTAs -> cluster (distributed shared memory) ----
    // a warp's partial sums [32 out-features][kTok] go to the start of its own (drained) ring
    const int ring_bytes = depth * kSlotBytes;
    {
        __syncwarp();
        const int r = lane >> 2, c = lane & 3;
        float* dst = reinterpret_cast<float*>(smem + p.w_offset + (size_t)warp * ring_bytes);   // [kTok][33]
#pragma unroll
        for (int nh = 0; nh < 2; ++nh) {
            float* d0 = dst + (2 * c) * 33 + nh * 16 + r;
            d0[0]      = acc[nh][0];
            d0[33]     = acc[nh][1];
            d0[8]      = acc[nh][2];
            d0[33 + 8] = acc[nh][3];
        }
    }
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            atomicExch(p.error, 1);
            const uint64_t t0 = globaltimer_ns();           // let copies still in flight land before the CTA retires
            while (globaltimer_ns() - t0 < 200000) { }
        }
        __syncthreads();
    }
    const int nloc = tn * kTileN, nloc_shift = 5 + p.tn_shift;
    const int kRingFloats = ring_bytes / 4;
    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) cluster.sync();                              // every rank's partial sums are in place
    if (tl) tl[4] = globaltimer_ns();

    const bool fused = p.world > 0;
    ExchangeHeader* hdr = reinterpret_cast<ExchangeHeader*>(p.self);
    const unsigned epoch = fused ? *reinterpret_cast<volatile unsigned*>(&hdr->epoch) : 0u;
    const unsigned half_sel = epoch & 1u, tag = epoch + 1u;

    const uint32_t ring0 = smem0 + p.w_offset;               // same offset in every rank's shared memory
    // Rank q of the cluster finalises a slice of the (token, local out-feature) space (out-feature fastest ->
    // coalesced stores).  An output is the sum of S * wk partials - K slice w of rank q lives in the ring of warp
    // (w * tn + n_local / 32) - added in a fixed order (rank-major): deterministic.
    const int terms = S << wk_sh;
    // sum of the S * wk partials of output (token, local out-feature)
    auto total = [&](int tok, int nl) {
        const int off = (nl >> 5) * kRingFloats + tok * 33 + (nl & 31);
        float s = 0.f;
        if (S == 1) {
#pragma unroll
            for (int w = 0; w < kWarps; ++w)
                if (w < wk) s += ld_shared_f32(ring0 + (uint32_t)(off + w * tn * kRingFloats) * 4u);
        } else {
            for (int t0 = 0; t0 < terms; t0 += 8) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int t = t0 + j, q = t >> wk_sh, w = t & (wk - 1);
                    v[j] = t < terms ? ld_cluster_f32(ring0 + (uint32_t)(off + w * tn * kRingFloats) * 4u, (uint32_t)q) : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) s += v[j];
            }
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
    const int e_lo = div_splits(Er * crank), e_hi = div_splits(Er * (crank + 1));
    if (p.silu_mul) {
        // SwiGLU epilogue: the out-feature tiles alternate gate, up, gate, up ..., so local out-features nl and nl + 32
        // are a (gate, up) pair and one thread owns both: out[t, j] = fp16(silu(gate)) * up, rounded like the separate
        // activation and product kernels it replaces (ops::SiluActivation of the reference, gemm_s4_f16.cu:30-40)
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
        for (int e = e_lo + threadIdx.x; e < e_hi; e += kThreads) {
            const int tok = e >> nloc_shift, nl = e & (nloc - 1);
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
                }
            }
        }
    }
    if (S > 1) cluster.sync();                              // peers may still be reading this CTA's partials
    if (fused) {
        // Exchange step.  CTA i of every rank covers the same outputs (all ranks launch the same shape) and thread j
        // the same elements, so each thread polls the slots of exactly the elements it pushed: all `world` slots of
        // an element are re-read until every tag is this call's, then the partials are added in rank order - the
        // same order on every rank, so all ranks end up with bit-identical outputs.
        const uint2* data = reinterpret_cast<const uint2*>(p.self + kExchangeDataOffset) + (size_t)half_sel * p.world * p.capacity;
        // once a wait has given up the buffer stays marked and later calls do not wait at all
        bool dead = *reinterpret_cast<volatile int*>(&hdr->error) != 0;
        for (int e = e_lo + threadIdx.x; e < e_hi; e += kThreads) {
            const int tok = e >> nloc_shift, nl = e & (nloc - 1);
            const int n = blockIdx.x * nloc + nl;
            if (n >= p.N) continue;
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
                if ((polls & 63u) == 63u) {
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
        }
        __syncthreads();
        // the last CTA to get here advances the epoch; the next call then uses the other half of the buffers
        if (threadIdx.x == 0) {
            const unsigned done = atomicAdd(&hdr->ticket, 1u);
            if (done == (unsigned)p.real_x * gridDim.y * gridDim.z - 1) {
                hdr->ticket = 0;
                __threadfence();
                *reinterpret_cast<volatile unsigned*>(&hdr->epoch) = epoch + 1;
            }
        }
    }
    // CTA 0 tells the padding CTAs of this grid that the work is (as good as) done
    if (p.pdl && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0 && p.real_x < (int)gridDim.x) atomicAdd(p.error + 1, 1);
    if (tl) tl[5] = globaltimer_ns();
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
struct Config { int tn, splits, depth, ahead, rp, swizzled, x_offset, w_offset, smem; };

int g_force_tn = 0, g_force_splits = 0, g_force_depth = 0, g_force_ahead = -1;
unsigned long long* g_timeline = nullptr;

int sm_count() { return device_sm_count(); }

int slot_bytes(int g) { return kUnitTiles * 512 + (kUnitK / g) * 128; }

// Shared memory of one CTA.  Preferred: at most kSmemBudget, so that two CTAs share an SM; when not even two stages
// fit in that (8 tokens: 2 KB of activations per unit and warp) the CTA takes what it needs and runs alone on its SM.
bool layout(Config& c, int g, int max_units_per_warp)
{
    int depth = kMaxDepth;
    if (depth > max_units_per_warp) depth = max_units_per_warp < 2 ? 2 : max_units_per_warp;
    if (g_force_depth && g_force_depth < depth) depth = g_force_depth < 2 ? 2 : g_force_depth;
    for (int budget : {kSmemBudget, kSmemMax}) {
        for (int d = depth; d >= 2; --d) {
            c.depth = d;
            c.x_offset = kHeaderBytes;
            // the kernel rounds the start of the activation chunks up to a multiple of 1024 bytes
            c.w_offset = (c.x_offset + 1023 + kWarps * d * c.rp * 256 + 127) / 128 * 128;
            c.smem = c.w_offset + kWarps * d * slot_bytes(g);
            if (c.smem <= budget) return true;
        }
    }
    return false;
}

template <int G>
int max_clusters_instance(int sp, int smem)
{
    static int cache[64][9] = {};      // benign race: the query is idempotent
    int dev = 0;
    const int sms = sm_count();
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return sms / sp;
    if (cache[dev][sp]) return cache[dev][sp];
    int n = 0;
    if (cudaFuncSetAttribute(gemv_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, sp, 1);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = sp;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, gemv_kernel<G>, &cfg) != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
        if (smem <= kSmemBudget) n /= 2;      // the query counts two CTAs per SM; the grid is one wave of one CTA per SM
    } else {
        (void)cudaGetLastError();
    }
    if (n <= 0) n = sms / sp;          // query unavailable: assume perfect packing
    cache[dev][sp] = n;
    return n;
}

int max_clusters(int g, int sp, int smem)
{
    if (sp <= 1) return 1 << 30;
    if (g == 128) return max_clusters_instance<128>(sp, smem);
    if (g == 64) return max_clusters_instance<64>(sp, smem);
    return max_clusters_instance<32>(sp, smem);
}

// Decomposition: tn out-feature tiles per CTA (16 / tn K slices), S CTAs per cluster along K.  Among the shapes that
// run as one wave of at most one CTA per SM, pick the one with the least work on the busiest warp; clusters pay a
// little for their two barriers and the remote loads of the reduction.
bool pick_config(Config& best, int tokens, int N, int K, int g, int min_tn = 1)
{
    const int sms = sm_count();
    const int n_tiles = N / kTileN, units = (K + kUnitK - 1) / kUnitK;
    Config c0;
    const int rows = tokens < 8 ? tokens : 8;
    c0.rp = rows <= 1 ? 1 : rows <= 2 ? 2 : rows <= 4 ? 4 : 8;
    c0.swizzled = c0.rp >= 4;
    double best_cost = -1.0;
    for (int tn = min_tn; tn <= kWarps; tn <<= 1) {
        if (g_force_tn && tn != g_force_tn) continue;
        const int wk = kWarps / tn;
        for (int sp = 1; sp <= 8; ++sp) {
            if (g_force_splits && sp != g_force_splits) continue;
            if (sp * wk > units) continue;                                        // every K slice owns at least one unit
            const long long ctas = (long long)((n_tiles + tn - 1) / tn) * sp;
            if (ctas > sms) continue;
            const int cta_units = (units + sp - 1) / sp;
            const int uw = (cta_units + wk - 1) / wk;                             // units of the busiest warp
            Config c = c0;
            c.tn = tn; c.splits = sp;
            if (!layout(c, g, uw)) continue;
            if (sp > 1 && ctas / sp > max_clusters(g, sp, c.smem)) continue;
            double cost = uw + 1.0 + (sp > 1 ? 1.0 + 0.15 * sp : 0.0) + 0.02 * tn;
            if (c.smem > kSmemBudget) cost += 2.0;                               // runs alone on its SM: no overlap with its neighbours in the stream
            if (best_cost < 0 || cost < best_cost - 1e-9) { best_cost = cost; best = c; }
        }
    }
    if (best_cost < 0) return false;
    best.ahead = g_force_ahead >= 0 ? g_force_ahead : 4;
    return true;
}

template <int G>
int launch_instance(const CUtensorMap& wmap, const CUtensorMap& xmap, const GemvParams& p, dim3 grid, int smem, cudaStream_t st)
{
    static int configured_dev[64] = {0};   // benign race: the attribute call is idempotent
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev >= 64 || !configured_dev[dev]) {
        e = cudaFuncSetAttribute(gemv_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev < 64) configured_dev[dev] = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = (size_t)smem;
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
    e = cudaLaunchKernelEx(&cfg, gemv_kernel<G>, wmap, xmap, p);
    count_launch();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

}  // namespace

void gemv_set_timeline(unsigned long long* buf) { g_timeline = buf; }
void gemv_force_config(int tn, int splits, int depth) { g_force_tn = tn; g_force_splits = splits; g_force_depth = depth; }
void gemv_force_ahead(int units) { g_force_ahead = units; }

// The decomposition launch_gemv would use: plan[0..8] = tokens per pass, tiles per CTA, cluster size, ring depth, rows per
// activation box, shared memory bytes, grid x (CTAs with work), y, z.  Host only (no launch).
int gemv_plan(int tokens, int N, int K, int g, int* plan)
{
    Config c;
    if (tokens <= 0 || N <= 0 || K <= 0 || (N % 32) || (g != 32 && g != 64 && g != 128) || (K % g)) return W4A16_ERR_BAD_SHAPE;
    if (!pick_config(c, tokens, N, K, g)) return W4A16_ERR_BAD_SHAPE;
    const int n_tiles = N / kTileN;
    const int v[9] = {8, c.tn, c.splits, c.depth, c.rp, c.smem, (n_tiles + c.tn - 1) / c.tn, c.splits, (tokens + 7) / 8};
    for (int i = 0; i < 9; ++i) plan[i] = v[i];
    return W4A16_OK;
}

int launch_gemv(const GemmArgs& a, cudaStream_t st)
{
    if (a.tokens == 0) return W4A16_OK;
    // with the fused exchange every rank must launch the same shape: choose it from the K all ranks agreed on
    const int k_config = a.exchange ? a.exchange->k_config : a.K;
    if (k_config < a.K) return W4A16_ERR_BAD_SHAPE;
    Config c;
    if (a.silu_mul && ((a.N % 64) || a.exchange || a.residual)) return W4A16_ERR_BAD_SHAPE;
    if (!pick_config(c, a.tokens, a.N, k_config, a.g, a.silu_mul ? 2 : 1)) return g_force_tn || g_force_splits ? W4A16_ERR_BAD_ALGO : W4A16_ERR_BAD_SHAPE;

    GemvParams p;
    p.zs = a.zs; p.bias = a.bias; p.out = a.out;
    p.error = a.plan_only ? nullptr : device_error_word();
    if (!p.error && !a.plan_only) return W4A16_ERR_CUDA;
    p.world = 0; p.rank = 0; p.capacity = 0; p.self = nullptr; p.wait_budget_ns = exchange_wait_budget_ns();
    for (int d = 0; d < kExchangeMaxWorld; ++d) p.peer[d] = nullptr;
    if (a.exchange) {
        const ExchangeArgs& x = *a.exchange;
        if (x.world < 1 || x.world > kExchangeMaxWorld || x.rank < 0 || x.rank >= x.world) return W4A16_ERR_BAD_SHAPE;
        if (a.tokens > 8) return W4A16_ERR_TOO_LARGE;
        if ((long long)a.tokens * a.N > x.capacity) return W4A16_ERR_TOO_LARGE;
        for (int d = 0; d < x.world; ++d) {
            if (!x.peer[d]) return W4A16_ERR_NULL_POINTER;
            p.peer[d] = x.peer[d];
        }
        p.world = x.world; p.rank = x.rank; p.capacity = x.capacity; p.self = x.peer[x.rank];
    }
    p.tokens = a.tokens; p.N = a.N; p.K = a.K;
    p.tn_shift = 0;
    while ((1 << p.tn_shift) < c.tn) ++p.tn_shift;
    p.splits = c.splits;
    p.inv_splits = c.splits > 1 ? (unsigned)(((1ull << 32) + c.splits - 1) / c.splits) : 0u;
    p.depth = c.depth; p.ahead = c.ahead; p.rp = c.rp; p.swizzled = c.swizzled;
    p.x_offset = c.x_offset; p.w_offset = c.w_offset;
    p.relu = a.relu ? 1 : 0; p.pdl = a.static_weights ? 1 : 0;
    p.residual = a.residual; p.silu_mul = a.silu_mul ? 1 : 0;
    p.timeline = g_timeline;

    const int n_tiles = a.N / kTileN;
    p.real_x = (n_tiles + c.tn - 1) / c.tn;
    int grid_x = p.real_x;
    const int passes = (a.tokens + 7) / 8;
    // Under programmatic launch, with two CTAs per SM and a single pass, the grid is padded with CTAs that have no
    // work up to one CTA per SM (see the kernel): the next grid of the stream then also lands one CTA per SM.
    if (p.pdl && passes == 1 && c.smem <= kSmemBudget) {
        const int per_wave = sm_count() / c.splits;
        if (per_wave > grid_x) grid_x = per_wave;
    }
    dim3 grid(grid_x, c.splits, passes);
    if (grid.z > 65535) return W4A16_ERR_BAD_SHAPE;
    if (a.exchange && grid.z != 1) return W4A16_ERR_TOO_LARGE;
    if (a.plan_only) return (a.g == 128 || a.g == 64 || a.g == 32) ? W4A16_OK : W4A16_ERR_GROUP_SIZE;
    CUtensorMap wmap, xmap;
    {
        // the packed matrix as a 2-D tensor of 32-bit words: [K/32 rows][N/32 * 128 words], box = 4 rows x 128 words
        const uint64_t dims[2] = {(uint64_t)n_tiles * 128, (uint64_t)(a.K / kTileK)};
        const uint32_t box[2] = {128, (uint32_t)kUnitTiles};
        int s = encode_tensor_map_2d(&wmap, a.qw, /*u32*/ 4, dims, (uint64_t)n_tiles * 512, box, /*swizzle128*/ false);
        if (s != W4A16_OK) return s;
        // the activations [tokens][K] fp16: boxes of rp rows x 64 halfs (128 bytes, the swizzle span) or, for one or
        // two rows, one box of rp rows x 128 halfs without swizzle
        const uint64_t xdims[2] = {(uint64_t)a.K, (uint64_t)a.tokens};
        const uint32_t xbox[2] = {c.swizzled ? 64u : 128u, (uint32_t)c.rp};
        s = encode_tensor_map_2d(&xmap, a.x, /*f16*/ 2, xdims, (uint64_t)a.K * 2, xbox, c.swizzled != 0);
        if (s != W4A16_OK) return s;
    }
    switch (a.g) {
        case 128: return launch_instance<128>(wmap, xmap, p, grid, c.smem, st);
        case 64:  return launch_instance<64>(wmap, xmap, p, grid, c.smem, st);
        case 32:  return launch_instance<32>(wmap, xmap, p, grid, c.smem, st);
        default:  return W4A16_ERR_GROUP_SIZE;
    }
}

}  // namespace w4a16
