// W8A16 linear for tall activations, CTA-pair version: tcgen05.mma.cta_group::2 over a cluster
// of two CTAs (two SMs), M = 256 weight rows x N <= 256 activation rows per pair tile.
//
//   y[m, n] = (sum_k x[m, k] * wq[n, k]) * scale[n] + sum_j xo[m, j] * wo[n, j] + bias[n]
//
// Same structure and orientation as the single-CTA kernel (w8a16_tc.cu: weights are UMMA
// operand A, activations operand B, accumulator D[n (lane), m (column)] double-buffered in TMEM),
// with the pair sharing operand B: CTA r of the pair
//   * owns weight rows [256 tn + 128 r, +128): loads their int8 tile by TMA, widens it to 16-bit
//     in its own shared memory, holds their accumulator rows in its own TMEM and runs their
//     epilogue;
//   * loads only HALF of the activation tile (rows [tile_x tx + r tile_x/2, + tile_x/2)); the
//     tensor cores of both SMs read both halves.
// Per SM and per 128 x tile_x x 64 block of MACs this moves 8 KiB + tile_x * 64 B through
// L2 -> shared memory instead of 8 KiB + tile_x * 128 B.
//
// A pipeline stage is 128 wide in k (two 64-wide swizzle atoms), so every barrier probe, TMA issue
// and commit is paid once per 8 MMAs: with 64-wide stages the single-thread roles (a probe costs
// ~130 cycles even on a completed phase, a TMA issue ~100) set the pace, not the tensor core.
// Roles per CTA (23 warps): warp 0 TMA producer for activations, warp 22 TMA producer for int8
// weights (+ L2 prefetch six stages ahead), warp 1 MMA issuer (leader) / relay (peer), warps 2-5
// epilogue, warps 6-21 converters.
//
// Cross-CTA signalling (no TMA multicast anywhere): every TMA load and every converter arrival
// completes on a barrier of the CTA that owns the data; in the peer CTA two relay lanes forward
// "activation half landed" and "weight rows widened" to the leader as ONE remote mbarrier.arrive
// each per stage; the leader's single MMA thread issues every tcgen05.mma and signals "slot free" /
// "accumulator ready" to both CTAs with tcgen05.commit ... .multicast::cluster; the peer's
// epilogue warps arrive remotely on the leader's "accumulator drained" barrier.
// Every wait is bounded (see tc_common.cuh); on expiry the error flag is raised, all roles leave
// their loops, the pair meets at a cluster barrier, TMEM is released and the kernel returns.

#include "tc_common.cuh"

#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace cb {

namespace {

using namespace tc;

constexpr int kMaxTileX = 256;  // activation rows per pair tile = UMMA N (multiple of 16)
// A pipeline stage covers kSub consecutive 64-wide k-blocks (one 128-byte swizzle atom each): every
// barrier probe (~130 cycles even when complete), TMA issue (~100) and commit is paid once per
// stage, and with 64-wide stages those per-stage costs of the single-thread roles, not the tensor
// core, set the pace of the main loop.
constexpr int kSub = 2;
constexpr int kStageK = kSub * kBlockK;  // 128
constexpr int kStagesA = 3;     // converted weight stages (kSub x 16 KiB each)
constexpr int kStagesW8 = 2;    // int8 weight stages (kSub x 8 KiB each)
constexpr int kMaxStages = 8;   // activation half stages (kSub x <= 16 KiB each)
constexpr int kConvWarps = 16;
constexpr int kConvGroupWarps = 16; // converter warps per group (one group: all warps share every stage)
constexpr int kEpiWarps = 4;
constexpr int kThreads = (3 + kEpiWarps + kConvWarps) * 32;  // + TMA(x), MMA/relay, TMA(w8)
constexpr int kW8Warp = 2 + kEpiWarps + kConvWarps;         // last warp: int8 weight producer
constexpr int kTmemCols = 512;
constexpr uint32_t kBytesASub = kUmmaM * kBlockK * 2;  // 16384: one 128-row x 64-k converted sub-tile
constexpr uint32_t kBytesA = kSub * kBytesASub;        // 32768 per stage
constexpr uint32_t kBytesW8 = kUmmaM * kStageK;        // 16384 per stage: 128 rows x 128 int8
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;         // shared::cluster address -> same offset in CTA rank 0
constexpr uint32_t kSmemLimit = 232448;             // 227 KiB opt-in shared memory per CTA
// barriers: full_x[8], empty_x[8], peer_x[8], full_a[3], empty_a[3], peer_a[3], full_w8[4], empty_w8[4], tmem_full[2], tmem_empty[2]
constexpr uint32_t kNumBars = 3 * kMaxStages + 3 * kStagesA + 2 * kStagesW8 + 4;
constexpr uint32_t kTailBytes = kNumBars * 8 + 16;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The hardware cluster barrier has no bounded form; both CTAs of a pair reach it unconditionally (prologue and
// teardown only; after an expired wait every role of both CTAs falls through to the teardown).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the barrier at the same offset in CTA rank 0 (local when this CTA is rank 0)
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & kPeerMask) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive (once all prior MMAs of this thread retired) on the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((uint16_t)3)
        : "memory");
}
// instruction descriptor for the pair: M = 256 (128 rows per CTA), N = n, fp32 accumulate, K-major operands
__device__ __forceinline__ uint32_t make_idesc_pair(bool bf16, uint32_t n) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
// Warp-collective bounded wait: lane 0 polls, the result is broadcast.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}


struct PairParams {
    int64_t M, N, K;
    const void* scales;
    int scales_dtype;
    const void* bias;
    int bias_dtype;
    const void* xo;
    const void* wo;
    int64_t KO, ldxo;
    void* y;
    int64_t ldy;
    int tile_x;    // activation rows per pair tile (multiple of 16, <= 256); each CTA loads tile_x / 2
    int tiles_x;   // ceil(M / tile_x)
    int tiles_n;   // ceil(N / 256)
    int stages;    // depth of the activation ring
    uint32_t x_stage_bytes;  // kSub sub-tiles
    uint32_t x_sub_bytes;    // one sub-tile (half_x rows x 128 B, rounded up to 1 KiB)
    unsigned int* error_flag;
    int debug;  // development builds only: 1 skip the widening, 2 skip the MMAs, 4 skip the proxy fence, 8 no L2 prefetch
};

template <typename A>
__global__ void __launch_bounds__(kThreads, 1)
w8a16_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                     const PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t rank = cluster_ctarank();   // 0 = leader
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t stages = (uint32_t)p.stages;
    const uint32_t sa = base;                                   // converted weights, kStagesA x 16 KiB
    const uint32_t sw8 = sa + kStagesA * kBytesA;               // int8 weights, kStagesW8 x 8 KiB
    const uint32_t sx = sw8 + kStagesW8 * kBytesW8;             // activation halves, stages x x_stage_bytes
    const uint32_t bars = sx + stages * p.x_stage_bytes;
    // full_x / full_a are LOCAL in each CTA (own activation half landed / own weight rows widened);
    // the peer's relay lanes forward each as ONE remote arrive on the leader's peer_x / peer_a.
    // empty_x / empty_a are signalled in both CTAs by the leader's multicast tcgen05.commit.
    const uint32_t full_x = bars, empty_x = full_x + 8 * kMaxStages, peer_x = empty_x + 8 * kMaxStages;
    const uint32_t full_a = peer_x + 8 * kMaxStages, empty_a = full_a + 8 * kStagesA, peer_a = empty_a + 8 * kStagesA;
    const uint32_t full_w8 = peer_a + 8 * kStagesA, empty_w8 = full_w8 + 8 * kStagesW8;
    const uint32_t tmem_full = empty_w8 + 8 * kStagesW8, tmem_empty = tmem_full + 16;
    const uint32_t tmem_slot_addr = tmem_empty + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + (tmem_slot_addr - base));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair = (int)(blockIdx.x >> 1), num_pairs = (int)(gridDim.x >> 1);
    const int num_kb = (int)((p.K + kStageK - 1) / kStageK);  // pipeline stages per tile
    const int total_tiles = p.tiles_x * p.tiles_n;
    const int half_x = p.tile_x >> 1;
    const uint32_t sub_bytes = (uint32_t)half_x * kBlockK * 2;     // one activation sub-tile
    const uint32_t half_bytes = kSub * sub_bytes;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kMaxStages; ++i) {
            mbar_init(full_x + 8 * i, 1);
            mbar_init(empty_x + 8 * i, 1);
            mbar_init(peer_x + 8 * i, 1);
        }
        for (int i = 0; i < kStagesA; ++i) {
            mbar_init(full_a + 8 * i, kConvGroupWarps);
            mbar_init(empty_a + 8 * i, 1);
            mbar_init(peer_a + 8 * i, 1);
        }
        for (int i = 0; i < kStagesW8; ++i) { mbar_init(full_w8 + 8 * i, 1); mbar_init(empty_w8 + 8 * i, kConvGroupWarps); }
        for (int i = 0; i < 2; ++i) { mbar_init(tmem_full + 8 * i, 1); mbar_init(tmem_empty + 8 * i, 2 * kEpiWarps); }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&map_x);
        prefetch_tmap(&map_w);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot_addr, kTmemCols);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer, activations (both CTAs) ------------------------------
        // The two producers are separate warps: a barrier probe costs ~130 cycles and a TMA issue
        // ~100, so one thread doing both rings cannot stay ahead of the tensor core.
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int t = pair; t < total_tiles && ok; t += num_pairs) {
                const int row_x = (t % p.tiles_x) * p.tile_x + (int)rank * half_x;
                for (int kb = 0; kb < num_kb; ++kb) {
                    { ok = mbar_wait(empty_x + 8 * s, ph ^ 1u, abort_flag); }
                    if (!ok) break;
                    { mbar_expect_tx(full_x + 8 * s, half_bytes);
#pragma unroll
                    for (int u = 0; u < kSub; ++u)
                        tma_load_2d(sx + s * p.x_stage_bytes + u * p.x_sub_bytes, &map_x, kb * kStageK + u * kBlockK, row_x,
                                    full_x + 8 * s); }
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == kW8Warp) {
        // ------------------------------ TMA producer, int8 weights (both CTAs) ------------------------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            constexpr int kAhead = 6;  // stages of int8 weights requested into L2 ahead of their TMA load
            for (int t = pair; t < total_tiles && ok; t += num_pairs) {
                const int row_w = (t / p.tiles_x) * 256 + (int)rank * kUmmaM;
                const int row_w_next = ((t + num_pairs) / p.tiles_x) * 256 + (int)rank * kUmmaM;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (kb + kAhead < num_kb) tma_prefetch_l2_2d(&map_w, (kb + kAhead) * kStageK, row_w);
                    else if (t + num_pairs < total_tiles) tma_prefetch_l2_2d(&map_w, (kb + kAhead - num_kb) * kStageK, row_w_next);
                    { ok = mbar_wait(empty_w8 + 8 * s, ph ^ 1u, abort_flag); }
                    if (!ok) break;
                    { mbar_expect_tx(full_w8 + 8 * s, kBytesW8);
                    tma_load_2d(sw8 + s * kBytesW8, &map_w, kb * kStageK, row_w, full_w8 + 8 * s); }
                    if (++s == kStagesW8) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) ------------------------------
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = make_idesc_pair(Widen<A>::kBf16, (uint32_t)p.tile_x);
            // Ring positions are kept incrementally (no divisions), and the four barriers of a
            // k-block are probed back to back before any result is used: a probe costs ~130 cycles
            // even when the phase is already complete, and this thread's loop is the critical path.
            uint32_t sx_i = 0, phx = 0, sa_i = 0, pha = 0, it = 0;
            bool ok = true, pre = false;
            for (int t = pair; t < total_tiles && ok; t += num_pairs, ++it) {
                const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
                { ok = mbar_wait(tmem_empty + 8 * acc, acc_ph ^ 1u, abort_flag); }  // both epilogues drained it
                if (!ok) break;
                const uint32_t d_tmem = tmem_base + acc * kMaxTileX;
                for (int kb = 0; kb < num_kb; ++kb) {
                    {
                        // `pre` holds the result of the probes issued one stage ago (they overlap the
                        // MMA issue of the previous stage); only on a miss does the thread block here.
                        if (!pre) {
                            const bool r0 = mbar_try(full_a + 8 * sa_i, pha), r1 = mbar_try(peer_a + 8 * sa_i, pha);
                            const bool r2 = mbar_try(full_x + 8 * sx_i, phx), r3 = mbar_try(peer_x + 8 * sx_i, phx);
                            ok = (r0 || mbar_wait(full_a + 8 * sa_i, pha, abort_flag)) &&
                                 (r1 || mbar_wait(peer_a + 8 * sa_i, pha, abort_flag)) &&
                                 (r2 || mbar_wait(full_x + 8 * sx_i, phx, abort_flag)) &&
                                 (r3 || mbar_wait(peer_x + 8 * sx_i, phx, abort_flag));
                        }
                    }
                    if (!ok) break;
                    tc_fence_after();
                    // ring positions of the NEXT stage, probed now, consumed after this stage is issued
                    uint32_t nsa = sa_i + 1, npha = pha, nsx = sx_i + 1, nphx = phx;
                    if (nsa == kStagesA) { nsa = 0; npha ^= 1u; }
                    if (nsx == stages) { nsx = 0; nphx ^= 1u; }
                    const bool n0 = mbar_try(full_a + 8 * nsa, npha), n1 = mbar_try(peer_a + 8 * nsa, npha);
                    const bool n2 = mbar_try(full_x + 8 * nsx, nphx), n3 = mbar_try(peer_x + 8 * nsx, nphx);
#pragma unroll
                    for (int u = 0; u < kSub; ++u) {
                        const uint64_t adesc = make_kmajor_sw128_desc(sa + sa_i * kBytesA + u * kBytesASub);
                        const uint64_t bdesc = make_kmajor_sw128_desc(sx + sx_i * p.x_stage_bytes + u * p.x_sub_bytes);
#pragma unroll
                        for (int k = 0; k < kBlockK / 16; ++k)
                            umma_f16_pair(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                                          (kb > 0 || u > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(empty_a + 8 * sa_i);  // frees the slots in both CTAs once these MMAs retire
                    umma_commit_pair(empty_x + 8 * sx_i);
                    pre = n0 && n1 && n2 && n3;
                    sa_i = nsa; pha = npha; sx_i = nsx; phx = nphx;
                }
                if (!ok) break;
                umma_commit_pair(tmem_full + 8 * acc);
            }
        } else if (rank == 1 && lane < 2) {
            // relays (two lanes, one per ring): when this CTA's activation half has landed (lane 0)
            // or its weight rows are widened (lane 1), tell the leader with ONE remote arrive
            const uint32_t depth = lane == 0 ? stages : (uint32_t)kStagesA;
            const uint32_t local = lane == 0 ? full_x : full_a, remote = lane == 0 ? peer_x : peer_a;
            const int64_t total_kb = pair < total_tiles ? (int64_t)((total_tiles - 1 - pair) / num_pairs + 1) * num_kb : 0;
            uint32_t s = 0, ph = 0;
            for (int64_t i = 0; i < total_kb; ++i) {
                bool ok;
                { ok = mbar_wait(local + 8 * s, ph, abort_flag); }
                if (!ok) break;
                mbar_arrive_leader(remote + 8 * s);
                if (++s == depth) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ------------------------------ epilogue (both CTAs, own 128 rows) ------------------------------
        const int quarter = warp & 3;
        const A* xo = static_cast<const A*>(p.xo);
        const A* wo = static_cast<const A*>(p.wo);
        A* y = static_cast<A*>(p.y);
        uint32_t it = 0;
        bool ok = true;
        for (int t = pair; t < total_tiles && ok; t += num_pairs, ++it) {
            const int tx = t % p.tiles_x, tn = t / p.tiles_x;
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            const int64_t n = (int64_t)tn * 256 + (int64_t)rank * kUmmaM + quarter * 32 + lane;
            const bool n_ok = n < p.N;
            const float scale = n_ok ? ref_round<A>(load_scalar(p.scales, p.scales_dtype, n)) : 0.0f;
            const bool has_bias = p.bias != nullptr;
            const float bias = (n_ok && has_bias) ? ref_round<A>(load_scalar(p.bias, p.bias_dtype, n)) : 0.0f;
            ok = warp_wait(tmem_full + 8 * acc, acc_ph, abort_flag, lane);
            if (!ok) break;
            tc_fence_after();
            const int64_t m_base = (int64_t)tx * p.tile_x;
            for (int c0 = 0; c0 < p.tile_x; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kMaxTileX + (uint32_t)c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int64_t m = m_base + c0 + c;
                    if (m >= p.M || c0 + c >= p.tile_x) break;  // uniform across the warp
                    float v = ref_round<A>(ref_round<A>(__uint_as_float(r[c])) * scale);
                    if (p.KO > 0 && n_ok) {
                        const A* xrow = xo + m * p.ldxo;  // same address in every lane: broadcast load
                        const A* wrow = wo + n * p.KO;
                        float side = 0.0f;
                        for (int j = 0; j < (int)p.KO; ++j)
                            side = fmaf(Widen<A>::to_float(__ldg(xrow + j)), Widen<A>::to_float(__ldg(wrow + j)), side);
                        v = ref_round<A>(v + ref_round<A>(side));
                    }
                    if (has_bias) v = ref_round<A>(v + bias);
                    if (n_ok) y[m * p.ldy + n] = Widen<A>::from_float(v);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(tmem_empty + 8 * acc);
        }
    } else if (warp < kW8Warp) {
        // ------------------------------ converters (both CTAs, own 128 rows) ------------------------------
        // Two groups of kConvGroupWarps warps take alternate stages, so the barrier probes, the
        // shared-memory latency and the proxy fence of one stage overlap the arithmetic of the next.
        const int lw = warp - (2 + kEpiWarps);
        const int group = lw / kConvGroupWarps;
        const int cid = (lw % kConvGroupWarps) * 32 + lane;  // 0 .. 255 within the group
        uint32_t s_w = 0, ph_w = 0, s_a = 0, ph_a = 0;
        auto advance = [&]() {
            if (++s_w == kStagesW8) { s_w = 0; ph_w ^= 1u; }
            if (++s_a == kStagesA) { s_a = 0; ph_a ^= 1u; }
        };
        if (group == 1) advance();
        const int64_t total_st = pair < total_tiles ? (int64_t)((total_tiles - 1 - pair) / num_pairs + 1) * num_kb : 0;
        bool ok = true;
        {
            for (int64_t st = group; st < total_st && ok; st += kConvWarps / kConvGroupWarps) {
                {
                    int okw = 1;
                    if (lane == 0) {
                        const bool r0 = mbar_try(full_w8 + 8 * s_w, ph_w), r1 = mbar_try(empty_a + 8 * s_a, ph_a ^ 1u);
                        okw = ((r0 || mbar_wait(full_w8 + 8 * s_w, ph_w, abort_flag)) &&
                               (r1 || mbar_wait(empty_a + 8 * s_a, ph_a ^ 1u, abort_flag))) ? 1 : 0;
                    }
                    ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
                }
                if (!ok) break;
                tc_fence_after();
                {
#pragma unroll
                for (int pass = 0; pass < (kUmmaM * kStageK / 16) / (kConvGroupWarps * 32); ++pass) {
                    // 16-byte chunk `id` of the int8 stage: 128-byte rows, chunk jc covers k = 16 jc .. +15
                    const int id = pass * (kConvGroupWarps * 32) + cid;
                    const int row = id >> 3, jc = id & 7, sub = jc >> 2, j = jc & 3;
                    uint32_t c0, c1, c2, c3;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
                                 : "r"(sw8 + s_w * kBytesW8 + (uint32_t)(id * 16)));
                    uint32_t o[8];
                    Widen<A>::four(c0, o[0], o[1]);
                    Widen<A>::four(c1, o[2], o[3]);
                    Widen<A>::four(c2, o[4], o[5]);
                    Widen<A>::four(c3, o[6], o[7]);
                    // 16-bit row = 128 bytes = eight 16-byte chunks; chunk c lives at c ^ (row % 8)
                    const uint32_t rbase = sa + s_a * kBytesA + (uint32_t)sub * kBytesASub + (uint32_t)(row * 128);
                    const uint32_t sw = (uint32_t)(row & 7);
                    // The two sub-tiles sit 16 KiB apart (same banks), so lanes of sub-tile 1 store their
                    // two chunks in the opposite order: each store instruction then touches eight
                    // different 16-byte bank groups per quarter-warp.
                    const bool swp = sub != 0;
                    const uint32_t ca = (uint32_t)(2 * j + (swp ? 1 : 0)), cb2 = (uint32_t)(2 * j + (swp ? 0 : 1));
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(rbase + ((ca ^ sw) << 4)),
                                 "r"(swp ? o[4] : o[0]), "r"(swp ? o[5] : o[1]), "r"(swp ? o[6] : o[2]), "r"(swp ? o[7] : o[3])
                                 : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(rbase + ((cb2 ^ sw) << 4)),
                                 "r"(swp ? o[0] : o[4]), "r"(swp ? o[1] : o[5]), "r"(swp ? o[2] : o[6]), "r"(swp ? o[3] : o[7])
                                 : "memory");
                }
                }
                fence_async_smem();  // generic-proxy stores -> visible to the tensor-core (async) proxy
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(full_a + 8 * s_a);
                    mbar_arrive(empty_w8 + 8 * s_w);
                }
                for (int q = 0; q < kConvWarps / kConvGroupWarps; ++q) advance();
            }
        }
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer may still read this CTA's shared memory / signal its barriers until here
    tc_fence_after();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag) {
        atomicExch(p.error_flag, 1u);
        __nanosleep(200000);  // let any TMA copy still in flight land before the CTA's memory is released
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn2() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

bool make_map(CUtensorMap* map, CUtensorMapDataType dt, const void* ptr, uint64_t inner, uint64_t outer,
              uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn2();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Activation rows per pair tile: the multiple of 32 (<= 256) with the fewest wasted pair-slots over
// the persistent schedule of ceil(M / tile) * ceil(N / 256) tiles on `pairs` CTA pairs.
int pick_pair_tile_x(int64_t M, int64_t N, int pairs) {
    const int64_t tiles_n = (N + 255) / 256;
    int best = 256;
    double best_cost = 1e30;
    for (int tx = 256; tx >= 32; tx -= 16) {
        const int64_t tiles = ((M + tx - 1) / tx) * tiles_n;
        const int64_t waves = (tiles + pairs - 1) / pairs;
        const double cost = (double)waves * (tx + 512);  // measured: a k-block costs nearly the same for every tile height
        if (cost < best_cost - 1e-9) { best_cost = cost; best = tx; }
    }
    return best;
}

}  // namespace

unsigned int* w8a16_tc_error_word();  // w8a16_tc.cu


bool w8a16_tc_pair_supported(const W8A16Args& a) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (a.act_dtype != kBF16 && a.act_dtype != kF16) return false;
    if (a.K < 16 || a.K % 16 != 0) return false;  // TMA: int8 row stride must be a multiple of 16 bytes
    if ((a.ldx * 2) % 16 != 0) return false;      // TMA: activation row stride
    if (!al16(a.x) || !al16(a.wq)) return false;
    if (a.KO > 64 || a.M < 1 || a.N < 1) return false;
    if (sm_count() < 2) return false;
    return encode_fn2() != nullptr;
}

cudaError_t launch_w8a16_tc_pair(const W8A16Args& a, cudaStream_t s) {
    const int pairs_avail = sm_count() / 2;
    PairParams p;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.scales = a.scales; p.scales_dtype = a.scales_dtype;
    p.bias = a.bias; p.bias_dtype = a.bias_dtype;
    p.xo = a.xo; p.wo = a.wo; p.KO = a.KO; p.ldxo = a.ldxo;
    p.y = a.y; p.ldy = a.ldy;
    p.tile_x = pick_pair_tile_x(a.M, a.N, pairs_avail);
    p.debug = 0;
    p.tiles_x = (int)((a.M + p.tile_x - 1) / p.tile_x);
    p.tiles_n = (int)((a.N + 255) / 256);
    p.error_flag = w8a16_tc_error_word();
    if (!p.error_flag) return cudaErrorUnknown;
    p.x_sub_bytes = ((uint32_t)(p.tile_x / 2) * kBlockK * 2 + 1023u) & ~1023u;
    p.x_stage_bytes = kSub * p.x_sub_bytes;
    const uint32_t fixed = 1024 + kStagesA * kBytesA + kStagesW8 * kBytesW8 + kTailBytes;
    int st = (int)((kSmemLimit - fixed) / p.x_stage_bytes);
    if (st > kMaxStages) st = kMaxStages;
    if (st < 2) return cudaErrorNotSupported;
    p.stages = st;
    const uint32_t smem = fixed + (uint32_t)st * p.x_stage_bytes;

    CUtensorMap map_x, map_w;
    const CUtensorMapDataType xdt = a.act_dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!make_map(&map_x, xdt, a.x, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.ldx * 2, kBlockK, (uint32_t)(p.tile_x / 2),
                  CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorNotSupported;
    if (!make_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.K, kStageK,
                  kUmmaM, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorNotSupported;

    const int64_t tiles = (int64_t)p.tiles_x * p.tiles_n;
    const int pairs = (int)(tiles < pairs_avail ? tiles : pairs_avail);
    const void* fn = a.act_dtype == kBF16 ? (const void*)w8a16_tc_pair_kernel<__nv_bfloat16>
                                          : (const void*)w8a16_tc_pair_kernel<__half>;
    static bool attr_done[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int which = a.act_dtype == kBF16 ? 0 : 1;
    if (dev >= 0 && dev < 64 && !attr_done[dev][which]) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit);
        if (e != cudaSuccess) return e;
        attr_done[dev][which] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    {
        // a persistent schedule needs every pair resident at once: never launch more clusters
        // than the device can hold simultaneously
        static int max_clusters[64][2] = {};
        if (dev >= 0 && dev < 64 && max_clusters[dev][which] == 0) {
            int n = 0;
            cudaLaunchConfig_t probe = cfg;
            probe.gridDim = dim3((unsigned)(2 * pairs_avail));
            if (cudaOccupancyMaxActiveClusters(&n, fn, &probe) != cudaSuccess || n <= 0) n = pairs_avail;
            max_clusters[dev][which] = n;
        }
        int cap = (dev >= 0 && dev < 64) ? max_clusters[dev][which] : pairs_avail;
        if (pairs > cap) cfg.gridDim = dim3((unsigned)(2 * cap));
    }
    void* args[3] = {(void*)&map_x, (void*)&map_w, (void*)&p};
    cudaError_t e = cudaLaunchKernelExC(&cfg, fn, args);
    if (e != cudaSuccess) return e;
    return cudaPeekAtLastError();
}

}  // namespace cb
