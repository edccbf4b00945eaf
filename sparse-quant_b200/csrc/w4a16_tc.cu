// Prefill kernel: W4A16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
//   out[t, n] = fp16( sum_k fp32( dq(W)[n, k] * x[t, k] ) ) (+ bias[n])
//
// Replaces the large-token instantiations of gemm_s4_f16_nn (gemm_template.h:358-464 of the
// reference: mma.sync + cp.async + ldmatrix, dequantisation re-done in the MMA issue slots).
// Role assignment follows the packed format: the weights are the MMA "A" operand (M = 128
// out-features per CTA tile), the activations are "B" (N = 64/128/256 tokens), the fp32
// accumulator D[out-feature lane][token column] lives in tensor memory.
//
// One persistent CTA per SM, warp specialised (warp numbers: 0-3 and 6.. dequantisers, 4 and the last one TMA, 5 MMA;
// 352 threads with the 256-token tile, 608 with the smaller ones, which have two more dequantiser groups).
//
// What set the pace of earlier versions was the ISSUE cost of the tensor-core instructions in the one thread that may
// issue them (measured on B200 with a loop of nothing but MMAs, 148 CTAs): from a loop that a single lane enters a
// tcgen05.mma issues every 94 cycles whatever its N (it executes in N/2 cycles) and a tcgen05.commit adds about 205;
// from a loop walked by the whole warp with an elected issuer (see elect_one) 45 / 73.5 / 137.5 cycles per MMA at
// N = 64 / 128 / 256 with the commit hidden at N = 256.  Hence: stages of 128 k (eight MMAs per pair of commits), the
// warp-wide loop, and barrier probes issued ahead of the MMAs in front of them.  With 64-k stages, a single issuing
// lane and one or two commits per stage the same kernel ran at 750 to 790 cycles per 512 cycles of tensor time,
// whatever the token tile, and no change to the other roles moved it.
//
// Rings (a stage = 128 k):
//   x ring   (shared memory, 128-byte swizzle, K-major): the activation tile as two 64-k sub-tiles, each with its own
//            mbarrier, filled by warp 4 with one tensor copy each, read only by the MMA.  The first sub-tile is
//            released by a commit of its own after the stage's first four MMAs, so that its refill starts half a
//            stage earlier (with whole-stage release the MMA warp waited for activations 10 % of its time at 256
//            tokens; with this 1 %).
//   A ring   (tensor memory, 64 columns per slot, same depth and index as the x ring): the dequantised fp16 weights
//            of the stage, written by the dequantisers, read by the MMA.  The commit at the end of a stage releases
//            the second x sub-tile and the A slot together (barrier `consumed`, waited on by warp 4 and by the
//            dequantisers).
//   W ring   (shared memory, own depth): the stage's packed weight tiles (a k-tile row of the format is contiguous:
//            plain bulk copies) and the (zero, scale) row(s), filled by the last warp, read only by the dequantisers and
//            released as soon as they hold the words in registers.
//   warps0-3,6.. dequantisers (groups of four; a pair of groups takes the two 64-k halves of a stage; with the 64- and
//            128-token tiles, whose stages are shorter than a pair's latency chain, two pairs take stages in turn -
//            measured 3-7 % there): read 16 B per lane per 32x32 tile from shared memory, expand the nibbles in
//            registers, (t - z) * s with
//            sub.ftz/mul.ftz (bit-exact with the reference), and write the fp16 result straight into tensor memory
//            with tcgen05.st.16x128b - the packed layout is already that fragment order - so the dequantised weights
//            never touch shared memory.
//   warp 5   MMA issuer: tcgen05.mma kind::f16 with A from tensor memory and B from the swizzled shared-memory
//            tile, eight K=16 instructions and two commits per stage; the barriers needed next are probed before
//            the MMAs in front of them are issued, so that in steady state no barrier round trip sits between them.
//   warps0-3,6-9 epilogue (the first pair of groups, after their last dequant step of the tile): tcgen05.ld the accumulator,
//            fp32 -> fp16, bias add, transposed store to out[token, out-feature].
// No cluster fan-out is used anywhere.  Every mbarrier wait is bounded; on a timeout the CTA raises an error word
// in global memory, drains and frees its tensor memory, and returns.
#include <mutex>

#include <cuda.h>

#include "w4a16_common.cuh"
#include "w4a16_sm100.cuh"

namespace w4a16 {

using namespace sm100;

namespace {

constexpr int kBlockN   = 128;                 // out-features per CTA tile (4 packed tiles)
constexpr int kBlockK   = 128;                 // k per pipeline stage (4 packed tiles, eight MMAs, one commit)
constexpr int kSubK     = 64;                  // k per swizzled activation sub-tile (128 bytes of fp16)
// GROUPS = groups of four dequantiser warps: 2 (one per 64-k half of every stage) for the 256-token tile, 4 (two
// pairs taking stages in turn) for the smaller tiles, whose stages are shorter than one pair's latency chain.
// Warps 0-3, 6.. : dequantisers; 4: x TMA; 5: MMA; the last warp: W TMA.
__host__ __device__ constexpr int w_producer_warp(int groups) { return 2 + 4 * groups; }
__host__ __device__ constexpr int tc_threads(int groups) { return 32 * (w_producer_warp(groups) + 1); }
#ifndef W4A16_TC_GROUPS_SMALL
#define W4A16_TC_GROUPS_SMALL 4
#endif
__host__ __device__ constexpr int tc_groups(int tok) { return tok == 256 ? 2 : W4A16_TC_GROUPS_SMALL; }
constexpr int kTmemCols = 512;
constexpr uint64_t kWaitBudgetNs = 400ull * 1000 * 1000;   // 0.4 s: far above any legitimate wait

template <int TOK>
struct TcCfg {
    static constexpr int kXSubBytes = TOK * kSubK * 2;                // one 64-k sub-tile (multiple of 8 KB)
    static constexpr int kXBytes   = 2 * kXSubBytes;                  // activation tile of a stage
    static constexpr int kWBytes   = 4 * 4 * 512;                     // four k-tile rows of four packed tiles
    static constexpr int kWStageBytes = kWBytes + 1024;               // + up to two (zero, scale) rows of 128 out-features
    static constexpr int kWStages  = TOK == 256 ? 3 : 4;
    static constexpr int kStages   = TOK == 256 ? 3 : (TOK == 128 ? 5 : 6);   // x ring == A ring
    static constexpr int kBarrierBytes = 1024;
    static constexpr int kACol     = TOK;                             // first TMEM column of the A ring
    static constexpr int kWRingOff = kStages * kXBytes;
    static constexpr int kBarOff   = kWRingOff + kWStages * kWStageBytes;
    static constexpr size_t kSmemBytes = 1024 /*align slack*/ + (size_t)kBarOff + kBarrierBytes;
    static constexpr int kBarriers = 5 * kStages + 2 * kWStages + 3;
    static_assert(8 * kBarriers + 12 <= kBarrierBytes, "barrier area");
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
    static_assert(kACol + 64 * kStages <= kTmemCols, "TMEM budget");
};

struct TcParams {
    const uint4*    qw;
    const uint32_t* zs;
    const __half*   bias;
    __half*         out;
    int*            error;          // device word, set non-zero on a wait timeout
    int tokens, N, K, g;
    int n_blocks, t_blocks;
    int relu;                       // clamp the outputs at zero after the bias add
    const __half* residual;         // [tokens, N] added after bias / ReLU (fp16 add), or null
    int split;                      // K parts per output tile (1 = no split)
    float* partial;                 // split > 1: fp32 partial tiles [split][tokens][N]
    int*   counters;                // split > 1: arrivals per output tile (zero on entry, reset by the last arriver)
    long long* account;             // debug builds: cycle accounting of CTA 0's MMA warp (8 words), or null
};

template <int TOK>
__global__ void __launch_bounds__(tc_threads(tc_groups(TOK)), 1) tc_kernel(const __grid_constant__ CUtensorMap x_map, const TcParams p)
{
    using Cfg = TcCfg<TOK>;
    constexpr int S = Cfg::kStages, SW = Cfg::kWStages;
    extern __shared__ unsigned char smem_raw[];

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + Cfg::kBarOff;
    // barrier layout (8 B each): xfull[2S] (one per 64-k half), afull[S], consumed[S], xhalf[S], wfull[SW], wempty[SW],
    // dfull, dempty, epi ; then tmem ptr, abort flag, last flag
    auto xfull_bar    = [&](int h) { return bar_base + 8u * h; };                     // h = 2 * stage + half
    auto afull_bar    = [&](int s) { return bar_base + 8u * (2 * S + s); };
    auto consumed_bar = [&](int s) { return bar_base + 8u * (3 * S + s); };           // A slot and second x half free
    auto xhalf_bar    = [&](int s) { return bar_base + 8u * (4 * S + s); };           // first x half free
    auto wfull_bar    = [&](int s) { return bar_base + 8u * (5 * S + s); };
    auto wempty_bar   = [&](int s) { return bar_base + 8u * (5 * S + SW + s); };
    const uint32_t dfull_bar = bar_base + 8u * (Cfg::kBarriers - 3), dempty_bar = dfull_bar + 8u, epi_bar = dfull_bar + 16u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Cfg::kBarOff + 8 * Cfg::kBarriers);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* last_flag = abort_flag + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(xfull_bar(2 * s), 1); mbar_init(xfull_bar(2 * s + 1), 1);
            mbar_init(afull_bar(s), 8); mbar_init(consumed_bar(s), 1); mbar_init(xhalf_bar(s), 1);
        }
        for (int s = 0; s < SW; ++s) { mbar_init(wfull_bar(s), 1); mbar_init(wempty_bar(s), 8); }
        mbar_init(dfull_bar, 1);
        mbar_init(dempty_bar, 8);
        mbar_init(epi_bar, 8);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32((const void*)tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    if (warp == 4 && lane == 0) prefetch_tmap(&x_map);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int n_tiles = p.N / kTileN;
    const int k_steps = (p.K + kBlockK - 1) / kBlockK;        // K % 128 == 64: the last stage carries one 64-k half
    const bool k_tail = (p.K % kBlockK) != 0;
    const int total_tiles = p.n_blocks * p.t_blocks * p.split;      // work items: (output tile, K part)
    auto k_range = [&](int item, int& ks0, int& ks1) {
        const int kp = item % p.split;
        ks0 = (int)((long long)k_steps * kp / p.split);
        ks1 = (int)((long long)k_steps * (kp + 1) / p.split);
    };
    // after a failed wait: give copies already in flight time to land before the CTA releases its shared memory
    auto drain_copies = [&]() {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000) { }
    };

    if (warp == 4) {
        // ------------------------------ TMA producer of the activation tiles ------------------------------
        if (lane == 0) {
            int st = 0; uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
                const int tb = (item / p.split) / p.n_blocks;
                int ks0, ks1;
                k_range(item, ks0, ks1);
                int kcoord = ks0 * kBlockK;
                for (int ks = ks0; ks < ks1; ++ks) {
                    // the two 64-k halves of a stage are released one after the other (the first one by a commit in
                    // the middle of the stage's MMAs): each refill starts half a stage earlier than a whole-stage
                    // release would allow
                    const uint32_t dst = smem_base + st * Cfg::kXBytes;
                    ok = mbar_wait(xhalf_bar(st), phase ^ 1u, abort_flag, kWaitBudgetNs);
                    if (!ok) break;
                    mbar_arrive_expect_tx(xfull_bar(2 * st), Cfg::kXSubBytes);
                    tma_load_2d(dst, &x_map, kcoord, tb * TOK, xfull_bar(2 * st));
                    ok = mbar_wait(consumed_bar(st), phase ^ 1u, abort_flag, kWaitBudgetNs);
                    if (!ok) break;
                    mbar_arrive_expect_tx(xfull_bar(2 * st + 1), Cfg::kXSubBytes);
                    tma_load_2d(dst + Cfg::kXSubBytes, &x_map, kcoord + kSubK, tb * TOK, xfull_bar(2 * st + 1));
                    kcoord += kBlockK;
                    if (++st == S) { st = 0; phase ^= 1u; }
                }
            }
            if (!ok) drain_copies();
        }
    } else if (warp == w_producer_warp(tc_groups(TOK))) {
        // ------------------------------ TMA producer of the packed weights ------------------------------
        // Three lanes share the copies of a stage (an issued copy holds its thread for about a hundred cycles).  A
        // copy that completes before lane 0 has armed the barrier only drives its byte count negative for a moment;
        // the phase cannot complete before lane 0's arrival.
        if (lane < 3) {
            int sw = 0; uint32_t wphase = 0;
            bool ok = true;
            const uint32_t row_words = (uint32_t)n_tiles * 32u;                 // uint4 per k-tile row of the packed matrix
            const int zs_rows = kBlockK / p.g;                                  // 1 (g = 128) or 2 (g = 64) per stage
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
                const int nb = (item / p.split) % p.n_blocks;
                const int nb_tiles = min(4, n_tiles - nb * 4);
                int ks0, ks1;
                k_range(item, ks0, ks1);
                const uint32_t w_bytes = nb_tiles * 512u, zs_bytes = nb_tiles * 128u;
                const uint4* wsrc = p.qw + (size_t)(ks0 * 4) * row_words + nb * 4 * 32;
                const uint32_t* zsrc = p.zs + (size_t)(ks0 * zs_rows) * p.N + nb * kBlockN;
                for (int ks = ks0; ks < ks1; ++ks) {
                    ok = mbar_wait(wempty_bar(sw), wphase ^ 1u, abort_flag, kWaitBudgetNs);
                    if (!ok) break;
                    const uint32_t dst = smem_base + Cfg::kWRingOff + sw * Cfg::kWStageBytes;
                    const uint32_t bar = wfull_bar(sw);
                    const bool tail = k_tail && ks == k_steps - 1;                  // only the first half exists (g = 64)
                    if (lane == 0) {
                        mbar_arrive_expect_tx(bar, tail ? 2 * w_bytes + zs_bytes : 4 * w_bytes + zs_rows * zs_bytes);
                        bulk_load(dst, wsrc, w_bytes, bar);
                        bulk_load(dst + 2048, wsrc + row_words, w_bytes, bar);
                    } else if (lane == 1) {
                        if (!tail) {
                            bulk_load(dst + 4096, wsrc + 2 * row_words, w_bytes, bar);
                            bulk_load(dst + 6144, wsrc + 3 * row_words, w_bytes, bar);
                        }
                    } else {
                        bulk_load(dst + Cfg::kWBytes, zsrc, zs_bytes, bar);
                        if (zs_rows == 2 && !tail) bulk_load(dst + Cfg::kWBytes + 512, zsrc + p.N, zs_bytes, bar);
                    }
                    wsrc += 4 * row_words;
                    zsrc += (size_t)zs_rows * p.N;
                    if (++sw == SW) { sw = 0; wphase ^= 1u; }
                }
            }
            if (!ok && lane == 0) drain_copies();
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer ------------------------------
        // The whole warp walks the loop and an elected lane issues, so that descriptors and addresses stay in uniform
        // registers (see elect_one).
        constexpr uint32_t idesc = idesc_f16_m128(TOK);
        const uint64_t bdesc0 = smem_desc_sw128(smem_base);            // the start-address field advances in 16-byte units
        int st = 0; uint32_t phase = 0, dphase = 0;
        bool ok = true;
        // Whatever this warp does between the last MMA of a stage and the first of the next is idle tensor time, and
        // a barrier wait that succeeds at once still costs a round trip of about a hundred cycles.  The coming stage's
        // two barriers are therefore probed before this stage's MMAs; in steady state both are complete (every other
        // role runs ahead of the MMA) and the next iteration starts issuing at once.
        bool ready = false;
#ifdef W4A16_SKINNY_DEBUG
        // where this warp's cycles go: [0] total, [1] waiting for the A slot, [2] for the x stage, [3] for the
        // accumulator, [4] / [5] stages whose A / x probe missed, [6] stages
        long long acct[7] = {0, 0, 0, 0, 0, 0, 0};
        const long long t_begin = clock64();
#define TC_ACCT(i, v) acct[i] += (v)
#else
#define TC_ACCT(i, v)
#endif
        for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
#ifdef W4A16_SKINNY_DEBUG
            const long long cd0 = clock64();
#endif
            ok = __all_sync(0xffffffffu, mbar_wait(dempty_bar, dphase ^ 1u, abort_flag, kWaitBudgetNs));   // epilogue drained D
            if (!ok) break;
            TC_ACCT(3, clock64() - cd0);
            tc_fence_after_sync();
            int ks0, ks1;
            k_range(item, ks0, ks1);
            for (int ks = ks0; ks < ks1; ++ks) {
                TC_ACCT(6, 1);
                if (!ready) {
#ifdef W4A16_SKINNY_DEBUG
                    const long long c0 = clock64();
                    ok = __all_sync(0xffffffffu, mbar_wait(afull_bar(st), phase, abort_flag, kWaitBudgetNs));
                    const long long c1 = clock64();
                    ok = ok && __all_sync(0xffffffffu, mbar_wait(xfull_bar(2 * st), phase, abort_flag, kWaitBudgetNs));
                    acct[1] += c1 - c0; acct[2] += clock64() - c1;
#else
                    ok = __all_sync(0xffffffffu, mbar_wait(afull_bar(st), phase, abort_flag, kWaitBudgetNs) &&
                                                 mbar_wait(xfull_bar(2 * st), phase, abort_flag, kWaitBudgetNs));
#endif
                    if (!ok) break;
                }
                tc_fence_after_sync();
                const uint64_t bdesc = bdesc0 + (uint64_t)((uint32_t)(st * Cfg::kXBytes) >> 4);
                const uint32_t a_tmem = tmem_base + Cfg::kACol + 64 * st;
                const int cur = st;
                const uint32_t cur_phase = phase;
                // first 64-k half: its activation sub-tile is released by a commit of its own
                const bool second_x = mbar_test_wait(xfull_bar(2 * cur + 1), cur_phase);
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        mma_f16_ts(tmem_base, a_tmem + 8 * kk, bdesc + (uint64_t)(2 * kk), idesc, ((ks - ks0) | kk) != 0);
                    tc_commit(xhalf_bar(cur));
                }
                __syncwarp();
                if (!__all_sync(0xffffffffu, second_x)) {
#ifdef W4A16_SKINNY_DEBUG
                    const long long c1 = clock64();
#endif
                    ok = __all_sync(0xffffffffu, mbar_wait(xfull_bar(2 * cur + 1), cur_phase, abort_flag, kWaitBudgetNs));
                    TC_ACCT(2, clock64() - c1);
                    TC_ACCT(5, 1);
                    if (!ok) break;
                    tc_fence_after_sync();
                }
                if (++st == S) { st = 0; phase ^= 1u; }
                const bool next_a = mbar_test_wait(afull_bar(st), phase);
                const bool next_x = mbar_test_wait(xfull_bar(2 * st), phase);
                if (elect_one()) {
#pragma unroll
                    for (int kk = 4; kk < 8; ++kk)
                        mma_f16_ts(tmem_base, a_tmem + 8 * kk, bdesc + (uint64_t)((Cfg::kXSubBytes >> 4) + 2 * (kk & 3)), idesc, 1);
                    tc_commit(consumed_bar(cur));
                }
                __syncwarp();
                ready = __all_sync(0xffffffffu, next_a && next_x);
#ifdef W4A16_SKINNY_DEBUG
                if (!__all_sync(0xffffffffu, next_a)) acct[4] += 1;
                if (!__all_sync(0xffffffffu, next_x)) acct[5] += 1;
#endif
            }
            if (!ok) break;
            if (elect_one()) tc_commit(dfull_bar);
            __syncwarp();
            dphase ^= 1u;
        }
#ifdef W4A16_SKINNY_DEBUG
        if (p.account && blockIdx.x == 0 && lane == 0) {
            acct[0] = clock64() - t_begin;
            for (int i = 0; i < 7; ++i) p.account[i] = acct[i];
        }
#endif
    } else {
        // ------------------------------ dequant + epilogue (warps 0..3 and 6..9) ------------------------------
        // Two groups of four warps; a warp may only touch the TMEM lane quarter (warp index % 4), which is also the
        // packed tile column it dequantises.  Group g takes the g-th 64-k half of every stage: a half keeps a warp
        // busy for a chain of dependent latencies (shared-memory load, unpack, sub/mul, tcgen05.st, its completion),
        // which the ring depth covers.  Both groups also drain the accumulator (half of the columns each) in the
        // epilogue.
        int st = 0, sw = 0; uint32_t phase = 0, wphase = 0, dphase = 0;
        bool ok = true;
        const int r = lane >> 2;
        constexpr int GROUPS = tc_groups(TOK);
        const int quarter = warp & 3;
        const int wgroup = warp < 4 ? 0 : (warp - 2) / 4;              // 0 .. GROUPS-1
        const int dgroup = wgroup & 1;                                 // which 64-k half of a stage
        const int turn = wgroup >> 1;                                  // GROUPS == 4: which stages (even / odd)
        uint32_t step_mod = 0;
        uint32_t epi_phase = 0;
        // bounded rendezvous of the eight dequant/epilogue warps (split-K finalisation)
        auto epi_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_bar);
            const bool done = __all_sync(0xffffffffu, mbar_wait(epi_bar, epi_phase, abort_flag, kWaitBudgetNs));
            epi_phase ^= 1u;
            return done;
        };
        const uint32_t lane_field = (uint32_t)(quarter * 32) << 16;
        const int zs_row = p.g == 64 ? dgroup : 0;                     // (zero, scale) row of this group's half
        for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
            const int tile = item / p.split, kp = item % p.split;
            const int nb = tile % p.n_blocks, tb = tile / p.n_blocks;
            const bool has_tile = nb * 4 + quarter < n_tiles;
            int ks0, ks1;
            k_range(item, ks0, ks1);
            for (int ks = ks0; ks < ks1; ++ks, step_mod ^= 1u) {
                if (GROUPS == 4 && step_mod != (uint32_t)turn) {               // the other pair's stage
                    if (++sw == SW) { sw = 0; wphase ^= 1u; }
                    if (++st == S) { st = 0; phase ^= 1u; }
                    continue;
                }
                ok = __all_sync(0xffffffffu, mbar_wait(wfull_bar(sw), wphase, abort_flag, kWaitBudgetNs));
                if (!ok) break;
                const unsigned char* wst = smem + Cfg::kWRingOff + sw * Cfg::kWStageBytes;
                const uint4* wq = reinterpret_cast<const uint4*>(wst) + dgroup * 256;
                const uint32_t* zsp = reinterpret_cast<const uint32_t*>(wst + Cfg::kWBytes + zs_row * 512) + quarter * 32 + r;
                uint4 q0 = make_uint4(0, 0, 0, 0), q1 = q0;
                uint32_t zsw[4] = {0, 0, 0, 0};
                // a missing second half (K % 128 == 64) dequantises to zeros: codes 0 with zero point and scale 0
                if (has_tile && !(dgroup == 1 && k_tail && ks == k_steps - 1)) {
                    q0 = wq[quarter * 32 + lane]; q1 = wq[128 + quarter * 32 + lane];
#pragma unroll
                    for (int j = 0; j < 4; ++j) zsw[j] = zsp[8 * j];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(wempty_bar(sw));                // the words are in registers: the stage may refill
                ok = __all_sync(0xffffffffu, mbar_wait(consumed_bar(st), phase ^ 1u, abort_flag, kWaitBudgetNs));
                if (!ok) break;
                if (has_tile) {
                    tc_fence_after_sync();
                    const uint32_t words[2][4] = {{q0.x, q0.y, q0.z, q0.w}, {q1.x, q1.y, q1.z, q1.w}};
#pragma unroll
                    for (int nh = 0; nh < 2; ++nh) {
                        uint32_t z0, s0, z1, s1;
                        split_zs(zsw[nh * 2], z0, s0);
                        split_zs(zsw[nh * 2 + 1], z1, s1);
                        uint32_t a[16];
#pragma unroll
                        for (int j = 0; j < 2; ++j)
#pragma unroll
                            for (int kh = 0; kh < 2; ++kh) {
                                uint32_t h[4];
                                unpack_s4x8(words[j][kh * 2 + nh], h);
                                uint32_t* d = a + j * 8 + kh * 4;
                                d[0] = dequant_h2(h[0], z0, s0);
                                d[1] = dequant_h2(h[1], z1, s1);
                                d[2] = dequant_h2(h[2], z0, s0);
                                d[3] = dequant_h2(h[3], z1, s1);
                            }
                        tmem_st_16x128b_x8(tmem_base + lane_field + ((uint32_t)(nh * 16) << 16) + Cfg::kACol + 64 * st + 32 * dgroup, a);
                    }
                    tmem_wait_st();
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(afull_bar(st));
                if (++sw == SW) { sw = 0; wphase ^= 1u; }
                if (++st == S) { st = 0; phase ^= 1u; }
            }
            if (!ok) break;
            if (wgroup >= 2) continue;                                       // only the first pair drains the accumulator

            // epilogue: thread = out-feature (TMEM lane), registers = tokens.  The per-element loops carry no branch
            // (measured: with the bias / ReLU / residual / ragged-tile tests inside them a tile took 15 000 cycles to
            // drain, without them 5 000): the common case - full token tile, no ReLU, no residual - has its own loop,
            // and a missing bias is added as -0.0, which changes no value.
            ok = __all_sync(0xffffffffu, mbar_wait(dfull_bar, dphase, abort_flag, kWaitBudgetNs));
            if (!ok) break;
            dphase ^= 1u;
            tc_fence_after_sync();
            const int n = nb * kBlockN + quarter * 32 + lane;
            const bool n_ok = n < p.N;
            const __half bias = (p.bias && n_ok) ? p.bias[n] : __ushort_as_half((unsigned short)0x8000u);
            const int tok0 = tb * TOK;
            const bool full_tile = tok0 + TOK <= p.tokens;
            const bool plain = full_tile && !p.relu && !p.residual;
            const int c_begin = dgroup * (TOK / 2), c_end = (dgroup + 1) * (TOK / 2);
            // the accumulator is free again once this warp's columns are in registers: the MMA of the next tile
            // starts while the values are still being converted and stored
            auto release_accumulator = [&]() {
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(dempty_bar);
            };
            auto finish = [&](float acc, int t) {                                // general path: one output element
                __half h = __hadd(__float2half_rn(acc), bias);
                if (p.relu) h = __hmax(h, __half());
                if (p.residual) h = __hadd(h, p.residual[(size_t)t * p.N + n]);
                p.out[(size_t)t * p.N + n] = h;
            };
            if (p.split == 1) {
#pragma unroll 1
                for (int c0 = c_begin; c0 < c_end; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_base + lane_field + c0, v);
                    tmem_wait_ld();
                    if (c0 + 32 >= c_end) release_accumulator();
                    if (!n_ok) continue;
                    if (plain) {
                        __half* dst = p.out + (size_t)(tok0 + c0) * p.N + n;
#pragma unroll
                        for (int j = 0; j < 32; ++j) dst[(size_t)j * p.N] = __hadd(__float2half_rn(__uint_as_float(v[j])), bias);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (tok0 + c0 + j < p.tokens) finish(__uint_as_float(v[j]), tok0 + c0 + j);
                    }
                }
            } else {
                // split-K: park the fp32 partial tile in the workspace; the CTA that completes the tile (the last
                // of `split` arrivals, found with one atomic per CTA) adds the parts in a fixed order - deterministic.
                float* mine = p.partial + (size_t)kp * p.tokens * p.N;
#pragma unroll 1
                for (int c0 = c_begin; c0 < c_end; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_base + lane_field + c0, v);
                    tmem_wait_ld();
                    if (c0 + 32 >= c_end) release_accumulator();
                    if (!n_ok) continue;
                    float* dst = mine + (size_t)(tok0 + c0) * p.N + n;
                    if (full_tile) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) dst[(size_t)j * p.N] = __uint_as_float(v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (tok0 + c0 + j < p.tokens) dst[(size_t)j * p.N] = __uint_as_float(v[j]);
                    }
                }
                __threadfence();
                if (!(ok = epi_sync())) break;                               // every warp's part of the tile is in the workspace
                if (warp == 0 && lane == 0) {
                    const int old = atomicAdd(p.counters + tile, 1);
                    const int last = old == p.split - 1;
                    if (last) p.counters[tile] = 0;                          // ready for the next launch
                    *last_flag = last;
                }
                if (!(ok = epi_sync())) break;
                if (*last_flag) {
                    __threadfence();
                    if (n_ok) {
                        // 32 tokens per batch: part 0, then one part at a time added to it (fixed order, up to 32
                        // loads in flight per thread - the reduction is a chain of L2 round trips otherwise)
                        const int c_last = min(c_end, p.tokens - tok0);      // ragged tile: stop at the last token
#pragma unroll 1
                        for (int c = c_begin; c < c_last; c += 32) {
                            const float* src = p.partial + (size_t)(tok0 + c) * p.N + n;
                            const bool whole = c + 32 <= c_last;
                            float sum[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) sum[j] = (whole || c + j < c_last) ? __ldcg(src + (size_t)j * p.N) : 0.f;
                            for (int q = 1; q < p.split; ++q) {
                                const float* sq = src + (size_t)q * p.tokens * p.N;
                                float part[32];
#pragma unroll
                                for (int j = 0; j < 32; ++j) part[j] = (whole || c + j < c_last) ? __ldcg(sq + (size_t)j * p.N) : 0.f;
#pragma unroll
                                for (int j = 0; j < 32; ++j) sum[j] += part[j];
                            }
                            if (whole && plain) {
                                __half* dst = p.out + (size_t)(tok0 + c) * p.N + n;
#pragma unroll
                                for (int j = 0; j < 32; ++j) dst[(size_t)j * p.N] = __hadd(__float2half_rn(sum[j]), bias);
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                    if (c + j < c_last) finish(sum[j], tok0 + c + j);
                            }
                        }
                    }
                }
                if (!(ok = epi_sync())) break;                               // last_flag may be rewritten by the next item
            }
        }
    }

    // ------------------------------ teardown ------------------------------
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) atomicExch(p.error, 1);
    if (warp == 5) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}


// Hardware self-check of the tensor-memory fragment mapping the dequantisers rely on: every warp
// stores tagged words with tcgen05.st.16x128b.x8 (both 16-lane halves) and reads its 32 lanes back
// with tcgen05.ld.32x32b.x32, which has the trivial mapping (thread i = lane i, register = column).
__global__ void __launch_bounds__(128, 1) tmem_layout_probe_kernel(uint32_t* out)
{
    __shared__ uint32_t slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        tmem_alloc(smem_u32(&slot), 32);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t base = slot;
    const uint32_t lane_field = (uint32_t)(warp * 32) << 16;
    for (int nh = 0; nh < 2; ++nh) {
        uint32_t r[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = ((uint32_t)warp << 24) | ((uint32_t)nh << 20) | ((uint32_t)lane << 8) | (uint32_t)j;
        tmem_st_16x128b_x8(base + lane_field + ((uint32_t)(nh * 16) << 16), r);
    }
    tmem_wait_st();
    uint32_t v[32];
    tmem_ld_32x32b_x32(base + lane_field, v);
    tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < 32; ++c) out[(warp * 32 + lane) * 32 + c] = v[c];
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(base, 32);
}

int g_force_tok = 0, g_force_split = 0;
long long* g_tc_account = nullptr;

struct TcPlan { int tok, split; };

// Token tile and K split by a cost model in SM clocks, fitted to measurements on B200: a work item costs
// k-steps x step + epilogue, where a 128-k step costs the larger of its tensor time (4 x tokens) and the issue time of
// its eight MMAs and one commit, items run in waves of one per SM, and split-K adds the round trip of the fp32
// partial tiles through L2/HBM at about 650 bytes per clock.
TcPlan pick_plan(int tokens, int N, int K, bool allow_split, int force_split = 0)
{
    const int n_blocks = (N + kBlockN - 1) / kBlockN;
    const long long k_steps = (K + kBlockK - 1) / kBlockK;
    TcPlan best = {256, 1};
    double best_cost = -1;
    const int cands[3] = {256, 128, 64};
    for (int i = 0; i < 3; ++i) {
        const int t = cands[i];
        if (g_force_tok && t != g_force_tok) continue;
        for (int sp = 1; sp <= 4; sp *= 2) {
            if (g_force_split && !force_split ? sp != g_force_split : (sp > 1 && !allow_split)) continue;
            if (sp > 1 && k_steps / sp < 4) continue;
            if (sp > 1 && K < 8192 && !g_force_split && !force_split) continue;      // measured: no gain from splitting a short K
            if (force_split && sp != force_split) continue;
            const long long items = (long long)n_blocks * ((tokens + t - 1) / t) * sp;
            const long long waves = (items + 147) / 148;
            const double issue = 8 * 94.0 + 205.0 + 60.0;           // eight MMAs, one commit, the loop around them
            const double step = 4.0 * t > issue ? 4.0 * t : issue;
            double cost = waves * ((double)(k_steps / sp) * step + 6.0 * t + 2000);
            if (sp > 1) cost += (double)sp * tokens * N * 8.0 / 650.0 + 3000;        // partials written + read back
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = {t, sp}; }
        }
    }
    return best;
}

size_t split_workspace_bytes(int tokens, int N, int split, int tiles)
{
    return (size_t)split * tokens * N * sizeof(float) + (((size_t)tiles * sizeof(int) + 255) / 256) * 256;
}

template <int TOK>
int launch_tok(const CUtensorMap& map, const TcParams& p, int grid, cudaStream_t st)
{
    static int configured[64] = {0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev >= 64 || !configured[dev]) {
        e = cudaFuncSetAttribute(tc_kernel<TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcCfg<TOK>::kSmemBytes);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev < 64) configured[dev] = 1;
    }
    tc_kernel<TOK><<<grid, tc_threads(tc_groups(TOK)), TcCfg<TOK>::kSmemBytes, st>>>(map, p);
    count_launch();
    e = cudaGetLastError();
    return e == cudaSuccess ? W4A16_OK : record_cuda_error(e);
}

}  // namespace

void tc_force_config(int tile_tokens, int split_k) { g_force_tok = tile_tokens; g_force_split = split_k; }
void tc_set_account(unsigned long long* buf) { g_tc_account = reinterpret_cast<long long*>(buf); }

bool tc_supported(int tokens, int N, int K, int g)
{
    return tokens > 0 && (g == 64 || g == 128) && (K % 64) == 0 && (N % kTileN) == 0;
}

size_t tc_workspace_bytes(int tokens, int N, int K, int g)
{
    if (!tc_supported(tokens, N, K, g)) return 0;
    const TcPlan pl = pick_plan(tokens, N, K, true);
    if (pl.split == 1) return 0;
    const int tiles = ((N + kBlockN - 1) / kBlockN) * ((tokens + pl.tok - 1) / pl.tok);
    return split_workspace_bytes(tokens, N, pl.split, tiles);
}

int launch_tc(const GemmArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t st, int* err_word, int force_split)
{
    int* err = err_word ? err_word : device_error_word();
    if (!err) return W4A16_ERR_CUDA;
    // split-K needs the caller's workspace; without one the best unsplit plan is used
    TcPlan pl = pick_plan(a.tokens, a.N, a.K, workspace != nullptr, force_split);
    const int tok = pl.tok;

    CUtensorMap map;
    {
        const uint64_t dims[2] = {(uint64_t)a.K, (uint64_t)a.tokens};
        const uint32_t box[2] = {(uint32_t)kSubK, (uint32_t)tok};
        int s = encode_tensor_map_2d(&map, a.x, 2, dims, (uint64_t)a.K * sizeof(__half), box, /*swizzle128*/ true);
        if (s != W4A16_OK) return s;
    }

    TcParams p;
    p.qw = reinterpret_cast<const uint4*>(a.qw); p.zs = a.zs; p.bias = a.bias; p.out = a.out; p.error = err;
    p.tokens = a.tokens; p.N = a.N; p.K = a.K; p.g = a.g; p.relu = a.relu ? 1 : 0; p.residual = a.residual; p.account = g_tc_account;
    p.n_blocks = (a.N + kBlockN - 1) / kBlockN;
    p.t_blocks = (a.tokens + tok - 1) / tok;
    const long long tiles = (long long)p.n_blocks * p.t_blocks;
    p.split = pl.split; p.partial = nullptr; p.counters = nullptr;
    if (pl.split > 1) {
        const size_t need = split_workspace_bytes(a.tokens, a.N, pl.split, (int)tiles);
        if (!workspace || workspace_bytes < need) return W4A16_ERR_WORKSPACE;
        if (((uintptr_t)workspace & 255)) return W4A16_ERR_MISALIGNED;
        p.partial = reinterpret_cast<float*>(workspace);
        p.counters = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + (size_t)pl.split * a.tokens * a.N * sizeof(float));
        cudaError_t e = cudaMemsetAsync(p.counters, 0, (size_t)tiles * sizeof(int), st);   // arrival counters start at zero
        if (e != cudaSuccess) return record_cuda_error(e);
    }
    int sms = 148;
    {
        static int cached[64] = {0};
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && dev < 64) {
            if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
            if (cached[dev] > 0) sms = cached[dev];
        }
    }
    const long long items = tiles * pl.split;
    const int grid = (int)(items < sms ? items : sms);
    switch (tok) {
        case 256: return launch_tok<256>(map, p, grid, st);
        case 128: return launch_tok<128>(map, p, grid, st);
        default:  return launch_tok<64>(map, p, grid, st);
    }
}

}  // namespace w4a16

// ---------------------------------------------------------------------------------------------------------------
// Entry point for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at all: code running between cudaStreamBeginCapture and
// EndCapture, plug-ins living inside another runtime's memory pool that forbids side allocations, and services
// that pin their whole memory budget at start-up.  The split-K flavour of the tcgen05 kernel needs global scratch
// (fp32 partial tiles, arrival counters) and every GEMM kernel needs an error word; here all three live in ONE
// file-scope device array that is part of the loaded library image: every GPU that loads the library carries
// these kStaticScratchBytes until the process exits, and nothing is ever allocated or freed.
//   * capacity: 2 K parts x tokens x N fp32 <= kStaticPartialBytes (16 MiB, e.g. 512 x 4096) and at most
//     kStaticMaxTiles output tiles; larger problems are refused with W4A16_ERR_TOO_LARGE;
//   * all calls on a device share the array and it keeps the previous call's contents: the counters are cleared
//     at the start of every call, the partial tiles are fully rewritten before they are read, and two calls whose
//     kernels overlap on the GPU (different streams) race on it - serialise them;
//   * in host code the array's name is only a handle: the device address comes from cudaGetSymbolAddress, looked
//     up once per device (with that device current) by the first call on that device.  Make that first call
//     outside stream capture.
constexpr size_t kStaticPartialBytes = 16u << 20;
constexpr int    kStaticMaxTiles     = 4096;
constexpr size_t kStaticScratchBytes = kStaticPartialBytes + kStaticMaxTiles * sizeof(int) + 256;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

extern "C" int w4a16_gemm_static_scratch(const void* x, const void* qweight, const void* zeros_scales, const void* bias,
                                         void* out, int tokens, int N, int K, int group_size, void* stream)
{
    using namespace w4a16;
    if (group_size != 64 && group_size != 128) return W4A16_ERR_GROUP_SIZE;
    if (tokens <= 0 || N <= 0 || K <= 0 || (N % 32) || (K % group_size) || K < 1024) return W4A16_ERR_BAD_SHAPE;
    if (!x || !qweight || !zeros_scales || !out) return W4A16_ERR_NULL_POINTER;
    if (((uintptr_t)x & 15) || ((uintptr_t)qweight & 15) || ((uintptr_t)zeros_scales & 15) || ((uintptr_t)out & 15))
        return W4A16_ERR_MISALIGNED;
    if ((size_t)2 * tokens * N * sizeof(float) > kStaticPartialBytes) return W4A16_ERR_TOO_LARGE;
    if ((long long)((N + kBlockN - 1) / kBlockN) * ((tokens + 63) / 64) > kStaticMaxTiles) return W4A16_ERR_TOO_LARGE;

    // once per device: resolve the device address of the file-scope array (the host-side name is not an address).
    // Host threads making their first call on a device together take turns here, so the set-up runs once.
    static unsigned char* base[64] = {nullptr};
    static std::mutex setup_lock;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= 64) return W4A16_ERR_UNSUPPORTED_GPU;
    std::lock_guard<std::mutex> guard(setup_lock);
    if (!base[dev]) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (major != 10) return W4A16_ERR_UNSUPPORTED_GPU;
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) return record_cuda_error(e == cudaSuccess ? cudaErrorInvalidSymbol : e);
        e = cudaMemsetAsync(ptr + kStaticScratchBytes - 256, 0, 256, (cudaStream_t)stream);     // error word starts clear
        if (e != cudaSuccess) return record_cuda_error(e);
        base[dev] = ptr;
    }
    unsigned char* scratch = base[dev];
    int* err_word = reinterpret_cast<int*>(scratch + kStaticScratchBytes - 256);

    GemmArgs a;
    a.x = (const __half*)x; a.qw = (const uint32_t*)qweight; a.zs = (const uint32_t*)zeros_scales;
    a.bias = (const __half*)bias; a.out = (__half*)out;
    a.tokens = tokens; a.N = N; a.K = K; a.g = group_size; a.static_weights = false;
    // workspace handed to the kernel = the static array minus the error word; launch_tc clears the counters
    return launch_tc(a, scratch, kStaticScratchBytes - 256, (cudaStream_t)stream, err_word, /*force_split=*/2);
}

// Reads the error word of the static-scratch entry point on the current device (0 = no barrier wait ever timed
// out there; also 0 if the entry point was never used on this device).  Synchronises the device.
extern "C" int w4a16_static_scratch_error_flag(int* flag)
{
    if (!flag) return W4A16_ERR_NULL_POINTER;
    unsigned char* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
    if (e != cudaSuccess) return w4a16::record_cuda_error(e);
    e = cudaMemcpy(flag, ptr + kStaticScratchBytes - 256, sizeof(int), cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? W4A16_OK : w4a16::record_cuda_error(e);
}

// Debug aid: fills out[128][32] (device, uint32) with the tags read back by the probe kernel above.
extern "C" int w4a16_debug_tmem_layout(void* out, void* stream)
{
    if (!out) return W4A16_ERR_NULL_POINTER;
    w4a16::tmem_layout_probe_kernel<<<1, 128, 0, (cudaStream_t)stream>>>((uint32_t*)out);
    w4a16::count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? W4A16_OK : w4a16::record_cuda_error(e);
}
