// W8A16 linear for tall activations on PAIRS of CTAs: tcgen05.mma.cta_group::2 over a cluster of two CTAs
// (two SMs).  A pair's work item is 256 output features x two activation tiles of up to 208 rows.
//
//   y[m, n] = r(r(sum_k x[m, k] * wq[n, k]) * r(scale[n])) (+ r(bias[n]), rounded)      r = round to the activation type
//
// What pairs change.  With cta_group::2 the tensor cores of both SMs read operand B (the activations) from BOTH CTAs'
// shared memory, so each CTA loads only HALF of every activation tile: 2 x 13 KB + 8 KB = 34 KB per k-block for 128
// features x 416 rows, against 61 KB in the single-CTA two-tile mode.  Each CTA keeps what is its own: the int8 tile of
// its 128 weight rows (TMA), their widening into its own tensor memory (operand A is read from tensor memory,
// tcgen05.st by the converter warps), their two accumulators (2 x 208 columns + 3 A stages x 32 = 512 columns) and
// their epilogue.  Measured on B200 (N = 14336, K = 4096): 55 / 211 / 932 us at M = 416 / 2048 / 8192 against 51 / 200 /
// 906 us for the single-CTA kernel -- halving the ingest does not pay, that kernel is not bound by it -- so the
// dispatcher keeps this kernel for path = 2 only.
//
// Roles per CTA (15 warps): warp 0 TMA producer of this CTA's activation halves; warp 14 TMA producer of its int8
// tiles (+ L2 prefetch); warp 1 MMA issuer (leader CTA only: one thread issues every tcgen05.mma of the pair);
// warps 2-5 epilogue; warps 6-13 converters, two groups of four warps on alternate k-blocks.
//
// Signalling.  Ring slot s of the LEADER carries the "full" barrier the MMA thread waits on: the activation
// loads of both CTAs complete on it (the .cta_group::2 form of the TMA load may name a barrier of the peer CTA;
// no multicast is involved, every load is a plain per-CTA load) and the converter warps of both CTAs arrive on
// it (one arrival per CTA and k-block, after the group's four warps met at a named barrier).  The int8 tile of a CTA completes on a local
// barrier its own converters wait on.  The leader frees a slot in both CTAs, and publishes the finished
// accumulators to both, with tcgen05.commit ... multicast::cluster (an mbarrier arrive, not a load); the epilogue
// warps of both CTAs arrive on the leader's "accumulator drained" barriers.  The accumulators are not
// double-buffered: the next item's MMAs into an accumulator wait until both CTAs have drained it.
// Every wait is bounded (tc_common.cuh); on expiry the error flag is raised, all roles leave their loops, the
// pair meets at the cluster barrier, tensor memory is released and the kernel returns.
//
// Not served here (the single-CTA kernel takes these): outlier columns, K % 16 != 0, fewer than 256 features.

#include "tc_common.cuh"

#include <mutex>

namespace cb {

namespace {

using namespace tc;

constexpr int kTileN = 128;        // weight rows per CTA
constexpr int kMaxTileX = 208;     // rows of one activation tile = UMMA N (a multiple of 16)
constexpr int kHalves = 2;         // activation tiles per work item
constexpr int kStages = 6;         // ring slots (activation halves + int8 tile)
constexpr int kTmemAStages = 3;    // widened-weight stages in tensor memory: slot s uses stage s % 3
constexpr int kConvWarps = 8;
constexpr int kEpiWarps = 4;
constexpr int kThreads = (3 + kEpiWarps + kConvWarps) * 32;
constexpr int kW8Warp = 2 + kEpiWarps + kConvWarps;  // 14: int8 weight producer
constexpr int kTmemCols = 512;
constexpr int kAccStride = kMaxTileX;       // columns between the two accumulators
constexpr int kACol = kHalves * kMaxTileX;  // first column of the A stages
constexpr int kAColsPerStage = kBlockK / 2; // two 16-bit k per 32-bit column
constexpr int kPfBlocks = 4;                // k-blocks of weights per L2 prefetch
constexpr uint32_t kBytesXHalf = (kMaxTileX / 2) * kBlockK * 2;  // 13312: this CTA's half of one activation tile
constexpr uint32_t kBytesX = kHalves * kBytesXHalf;              // 26624 per slot
constexpr uint32_t kBytesW8 = kTileN * kBlockK;                  // 8192 per slot
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;  // shared::cluster address -> same offset in CTA rank 0
static_assert(kACol + kTmemAStages * kAColsPerStage <= kTmemCols, "tensor memory map");
static_assert(kBytesXHalf % 1024 == 0, "swizzle atoms need 1024-byte aligned tiles");

struct Smem {
    static constexpr uint32_t x = 0;
    static constexpr uint32_t w8 = x + kStages * kBytesX;
    static constexpr uint32_t bars = w8 + kStages * kBytesW8;
    // full[kStages], empty[kStages], full_w8[kStages], tmem_full, tmem_empty[2]
    static constexpr uint32_t n_bars = 3 * kStages + 3;
    static constexpr uint32_t tmem_slot = bars + n_bars * 8;
    static constexpr uint32_t abort_flag = tmem_slot + 4;
    static constexpr uint32_t total = abort_flag + 4;
};
constexpr uint32_t kSmemBytes = Smem::total + 1024;
static_assert(kSmemBytes <= 232448, "shared memory map");

struct PairParams {
    int64_t M, N, K;
    const void* scales;
    int scales_dtype;
    const void* bias;
    int bias_dtype;
    void* y;
    int64_t ldy;
    int tile_x;   // rows of one activation tile (multiple of 16, <= 208)
    int tiles_x;  // ceil(M / (2 * tile_x))
    int tiles_n;  // ceil(N / 256)
    unsigned int* error_flag;
};

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
__device__ __forceinline__ void mbar_expect_tx_leader(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar & kPeerMask), "r"(bytes) : "memory");
}
// TMA tile load into THIS CTA's shared memory whose bytes are counted on the leader's barrier (no multicast)
__device__ __forceinline__ void tma_load_2d_to_leader_bar(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar & kPeerMask)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// M = 256 over the pair, operand A (this CTA's 128 rows x 16 k) from tensor memory, operand B from both CTAs'
// shared memory (each holds N / 2 rows at the descriptor's offset)
__device__ __forceinline__ void umma_f16_pair_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                                     uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive (once all prior MMAs of this thread retired) on the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// kind::f16, fp32 accumulate, both operands K-major, M = 256 over the pair, N = n
__device__ __forceinline__ uint32_t make_idesc_pair(bool bf16, uint32_t n) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <typename A>
__global__ void __launch_bounds__(kThreads, 1)
w8a16_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                     const __grid_constant__ CUtensorMap map_pf, const __grid_constant__ PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sx = base + Smem::x, sw8 = base + Smem::w8;
    const uint32_t full = base + Smem::bars, empty = full + 8 * kStages, full_w8 = empty + 8 * kStages;
    const uint32_t tmem_full = full_w8 + 8 * kStages, tmem_empty = tmem_full + 8;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + Smem::tmem_slot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gbase + Smem::abort_flag);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (int)((p.K + kBlockK - 1) / kBlockK);
    const int total_items = p.tiles_x * p.tiles_n;  // items of 256 features x 2 activation tiles
    const int pair = (int)(blockIdx.x >> 1), num_pairs = (int)(gridDim.x >> 1);
    const int half_rows = p.tile_x / 2;
    const uint32_t half_bytes = (uint32_t)half_rows * kBlockK * 2;  // one CTA's half of one activation tile, one k-block

    if (threadIdx.x == 0) {
        // full (used on the leader): one arrive.expect_tx per CTA + one arrive per CTA for its converter group;
        // empty / tmem_full: the leader's multicast commit; tmem_empty (leader): the epilogue warps of both CTAs
        for (int i = 0; i < kStages; ++i) {
            mbar_init(full + 8 * i, 2 + 2);
            mbar_init(empty + 8 * i, 1);
            mbar_init(full_w8 + 8 * i, 1);
        }
        mbar_init(tmem_full, 1);
        for (int i = 0; i < 2; ++i) mbar_init(tmem_empty + 8 * i, 2 * kEpiWarps);
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&map_x);
        prefetch_tmap(&map_w);
        prefetch_tmap(&map_pf);
    }
    if (warp == 1) tmem_alloc_pair(base + Smem::tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer: this CTA's halves of the two activation tiles ------------------------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int t = pair; t < total_items && ok; t += num_pairs) {
                const int row_x = (t % p.tiles_x) * p.tile_x * kHalves + (int)rank * half_rows;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(empty + 8 * s, ph ^ 1u, abort_flag);  // local copy: freed by the leader's multicast commit
                    if (!ok) break;
                    mbar_expect_tx_leader(full + 8 * s, kHalves * half_bytes);
                    tma_load_2d_to_leader_bar(sx + s * kBytesX, &map_x, kb * kBlockK, row_x, full + 8 * s);
                    // second activation tile of the item (rows beyond M arrive as zeros)
                    tma_load_2d_to_leader_bar(sx + s * kBytesX + kBytesXHalf, &map_x, kb * kBlockK, row_x + p.tile_x, full + 8 * s);
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == kW8Warp) {
        // ------------------------------ TMA producer: this CTA's int8 weight tile (local barrier) ------------------------------
        if (lane == 0) {
            constexpr int kAhead = 12;  // k-blocks of weights requested into L2 ahead of their TMA load
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int t = pair; t < total_items && ok; t += num_pairs) {
                const int row_w = (t / p.tiles_x) * 256 + (int)rank * kTileN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if ((kb & (kPfBlocks - 1)) == 0 && kb + kAhead < num_kb)
                        tma_prefetch_l2_2d(&map_pf, (kb + kAhead) * kBlockK, row_w);
                    // the int8 staging buffer of a slot is free when the slot is: the MMAs that retired consumed what
                    // the converters made of it
                    ok = mbar_wait(empty + 8 * s, ph ^ 1u, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(full_w8 + 8 * s, kBytesW8);
                    tma_load_2d(sw8 + s * kBytesW8, &map_w, kb * kBlockK, row_w, full_w8 + 8 * s);
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) ------------------------------
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = make_idesc_pair(Widen<A>::kBf16, (uint32_t)p.tile_x);
            uint32_t s = 0, ph = 0, it = 0;
            bool ok = true;
            for (int t = pair; t < total_items && ok; t += num_pairs, ++it) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_spin(full + 8 * s, ph, abort_flag);  // bytes and converter arrivals come from both CTAs
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_tmem = tmem_base + kACol + (s % (uint32_t)kTmemAStages) * kAColsPerStage;
                    const uint64_t bdesc0 = make_kmajor_sw128_desc(sx + s * kBytesX);
                    const uint64_t bdesc1 = make_kmajor_sw128_desc(sx + s * kBytesX + kBytesXHalf);
                    if (kb == 0) {  // both CTAs' epilogues have drained the first accumulator of the previous item
                        ok = mbar_spin(tmem_empty, (it & 1u) ^ 1u, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                    }
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k)  // 16 k = 8 columns of A, 32 bytes of every B row
                        umma_f16_pair_tmem_a(tmem_base, a_tmem + (uint32_t)(8 * k), bdesc0 + (uint64_t)(2 * k), idesc,
                                             (kb > 0 || k > 0) ? 1u : 0u);
                    if (kb == 0) {
                        ok = mbar_spin(tmem_empty + 8, (it & 1u) ^ 1u, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                    }
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k)  // the same widened weights against the second activation tile
                        umma_f16_pair_tmem_a(tmem_base + kAccStride, a_tmem + (uint32_t)(8 * k), bdesc1 + (uint64_t)(2 * k), idesc,
                                             (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty + 8 * s);  // the slot is free in both CTAs once these MMAs retire
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                umma_commit_pair(tmem_full);  // both accumulators complete -> the epilogues of both CTAs
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ------------------------------ epilogue (each CTA: its own 128 features, both activation tiles) ------------------------------
        const int quarter = warp & 3;  // a warp may only touch tensor-memory lanes 32 * (warp % 4) .. + 31
        uint16_t* y = static_cast<uint16_t*>(p.y);
        uint32_t it = 0;
        bool ok = true;
        for (int t = pair; t < total_items && ok; t += num_pairs, ++it) {
            const int tx = t % p.tiles_x, tn = t / p.tiles_x;
            const int64_t n = (int64_t)tn * 256 + (int64_t)rank * kTileN + quarter * 32 + lane;
            const bool n_ok = n < p.N;
            const float scale = n_ok ? load_scalar(p.scales, p.scales_dtype, n) : 0.0f;
            const bool has_bias = p.bias != nullptr;
            const float bias = (n_ok && has_bias) ? load_scalar(p.bias, p.bias_dtype, n) : 0.0f;
            const uint32_t scale2 = Widen<A>::pack2(scale, scale), bias2 = Widen<A>::pack2(bias, bias);  // rounded to A
            {
                int okw = 1;
                if (lane == 0) okw = mbar_wait(tmem_full, it & 1u, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
            }
            if (!ok) break;
            tc_fence_after();
            for (int half = 0; half < kHalves; ++half) {
                const int64_t m_base = ((int64_t)tx * kHalves + half) * p.tile_x;
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)half * kAccStride;
                for (int c0 = 0; c0 < p.tile_x && m_base + c0 < p.M; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(taddr + (uint32_t)c0, r);
                    tmem_ld_wait();
                    // rows of this block that exist; no control flow per row (predicated stores), two rows per step
                    // in packed 16-bit arithmetic, every step rounded as the reference's chain of kernels rounds
                    const int64_t rows_left = p.M - (m_base + c0);
                    int nrows = rows_left < 32 ? (int)rows_left : 32;
                    if (nrows > p.tile_x - c0) nrows = p.tile_x - c0;
                    uint16_t* yrow = y + (m_base + c0) * p.ldy + n;
                    const int64_t ystep = p.ldy;
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        uint32_t v = Widen<A>::mul2(Widen<A>::pack2(__uint_as_float(r[c]), __uint_as_float(r[c + 1])), scale2);
                        v = has_bias ? Widen<A>::add2(v, bias2) : v;
                        if (n_ok && c < nrows) yrow[(int64_t)c * ystep] = (uint16_t)(v & 0xffffu);
                        if (n_ok && c + 1 < nrows) yrow[(int64_t)(c + 1) * ystep] = (uint16_t)(v >> 16);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_leader(tmem_empty + 8 * half);
            }
        }
    } else if (warp < kW8Warp) {
        // ------------------------------ converters: two groups of four warps on alternate k-blocks ------------------------------
        // A thread owns weight row 32 * quarter + lane = its tensor-memory lane.  The int8 tile arrived with the 64-byte
        // TMA swizzle, so the eight lanes of a quarter-warp hit eight different bank groups.
        const int cw = warp - (2 + kEpiWarps);  // 0 .. 7
        const uint32_t group = (uint32_t)(cw >> 2);
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t swz = (uint32_t)((row >> 1) & 3);  // chunk c of row r sits at c ^ ((r >> 1) & 3)
        uint32_t s = 0, ph = 0, g = 0;
        bool ok = true;
        for (int t = pair; t < total_items && ok; t += num_pairs) {
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                if (g == group) {
                    int okw = 1;
                    if (lane == 0) {
                        okw = mbar_wait(full_w8 + 8 * s, ph, abort_flag) ? 1 : 0;
                        // the tensor-memory stage is shared with the slot kTmemAStages back: its MMAs must have retired
                        // (same ring round for the upper slots, the round before for the lower ones)
                        if (okw) {
                            const uint32_t back = s >= (uint32_t)kTmemAStages ? s - kTmemAStages : s + kTmemAStages;
                            okw = mbar_wait(empty + 8 * back, s >= (uint32_t)kTmemAStages ? ph : ph ^ 1u, abort_flag) ? 1 : 0;
                        }
                    }
                    if (__shfl_sync(0xffffffffu, okw, 0) == 0) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_stage = s % (uint32_t)kTmemAStages;
                    const uint32_t rbase = sw8 + s * kBytesW8 + (uint32_t)(row * 64);
#pragma unroll
                    for (int khalf = 0; khalf < 2; ++khalf) {
                        uint32_t c[8];
#pragma unroll
                        for (int j = 0; j < 2; ++j)
                            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                         : "=r"(c[4 * j]), "=r"(c[4 * j + 1]), "=r"(c[4 * j + 2]), "=r"(c[4 * j + 3])
                                         : "r"(rbase + ((((uint32_t)(2 * khalf + j)) ^ swz) << 4)));
                        uint32_t o[16];
#pragma unroll
                        for (int j = 0; j < 8; ++j) Widen<A>::four(c[j], o[2 * j], o[2 * j + 1]);
                        tmem_st16(tmem_base + ((uint32_t)(quarter * 32) << 16) +
                                      (uint32_t)(kACol + a_stage * kAColsPerStage + khalf * 16), o);
                    }
                    tmem_st_wait();
                    tc_fence_before();
                    // the group's four warps meet at a named barrier; one of them tells the leader (one remote arrive
                    // per CTA and k-block: the tensor-memory writes are complete, nothing in memory has to be released)
                    asm volatile("bar.sync %0, 128;" ::"r"(1 + (int)group) : "memory");
                    if ((cw & 3) == 0 && lane == 0) mbar_arrive_leader(full + 8 * s);
                }
                g ^= 1u;
                if (++s == kStages) { s = 0; ph ^= 1u; }
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

}  // namespace

unsigned int* w8a16_tc_error_word();  // w8a16_tc.cu

// Rows of one activation tile (a multiple of 16, <= 208) and the modelled length of the schedule in units of
// k-blocks x rows: ceil(M / (2 tile)) * ceil(N / 256) items on `pairs` CTA pairs.
double w8a16_tc_pair_plan(int64_t M, int64_t N, int64_t K, int pairs, int* tile_x) {
    const int64_t tiles_n = (N + 255) / 256;
    const int64_t num_kb = (K + kBlockK - 1) / kBlockK;
    int best = kMaxTileX;
    double best_cost = 1e300;
    for (int tx = kMaxTileX; tx >= 32; tx -= 16) {
        const int64_t items = ((M + 2 * tx - 1) / (2 * tx)) * tiles_n;
        const int64_t rounds = (items + pairs - 1) / pairs;
        const double cost = (double)rounds * (double)num_kb * (2 * tx + 512);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = tx; }
    }
    if (tile_x) *tile_x = best;
    return best_cost;
}

bool w8a16_tc_pair_supported(const W8A16Args& a) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (a.act_dtype != kBF16 && a.act_dtype != kF16) return false;
    if (a.K < 16 || a.K % 16 != 0) return false;  // TMA: int8 row stride must be a multiple of 16 bytes
    if ((a.ldx * 2) % 16 != 0) return false;      // TMA: activation row stride
    if (!al16(a.x) || !al16(a.wq)) return false;
    if (a.KO > 0 || a.M < 1 || a.N < 1) return false;
    if (sm_count() < 2) return false;
    return encode_fn2() != nullptr;
}

cudaError_t launch_w8a16_tc_pair(const W8A16Args& a, cudaStream_t s) {
    const int pairs_avail = sm_count() / 2;
    PairParams p;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.scales = a.scales; p.scales_dtype = a.scales_dtype;
    p.bias = a.bias; p.bias_dtype = a.bias_dtype;
    p.y = a.y; p.ldy = a.ldy;
    w8a16_tc_pair_plan(a.M, a.N, a.K, pairs_avail, &p.tile_x);
    p.tiles_x = (int)((a.M + 2 * p.tile_x - 1) / (2 * p.tile_x));
    p.tiles_n = (int)((a.N + 255) / 256);
    p.error_flag = w8a16_tc_error_word();
    if (!p.error_flag) return cudaErrorUnknown;

    CUtensorMap map_x, map_w, map_pf;
    const CUtensorMapDataType xdt = a.act_dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!make_map(&map_x, xdt, a.x, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.ldx * 2, kBlockK, (uint32_t)(p.tile_x / 2),
                  CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorNotSupported;
    // the int8 tile is read by the converters' generic loads, one row per lane: 64-byte swizzle
    if (!make_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.K, kBlockK, kTileN,
                  CU_TENSOR_MAP_SWIZZLE_64B))
        return cudaErrorNotSupported;
    // the same tensor with a box of kPfBlocks k-blocks, for L2 prefetches only
    if (!make_map(&map_pf, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.K,
                  a.K >= kPfBlocks * kBlockK ? kPfBlocks * kBlockK : kBlockK, kTileN, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorNotSupported;

    const int64_t items = (int64_t)p.tiles_x * p.tiles_n;
    const int pairs = (int)(items < pairs_avail ? items : pairs_avail);
    const void* fn = a.act_dtype == kBF16 ? (const void*)w8a16_tc_pair_kernel<__nv_bfloat16>
                                          : (const void*)w8a16_tc_pair_kernel<__half>;
    static bool attr_done[64][2] = {};
    static int max_clusters[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    const int which = a.act_dtype == kBF16 ? 0 : 1;
    if (!attr_done[dev][which]) {
        const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev][which] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (max_clusters[dev][which] == 0) {
        // a persistent schedule needs every pair resident at once: never launch more clusters than the device
        // holds simultaneously
        int n = 0;
        cudaLaunchConfig_t probe = cfg;
        probe.gridDim = dim3((unsigned)(2 * pairs_avail));
        if (cudaOccupancyMaxActiveClusters(&n, fn, &probe) != cudaSuccess || n <= 0) n = pairs_avail;
        max_clusters[dev][which] = n;
    }
    if (pairs > max_clusters[dev][which]) cfg.gridDim = dim3((unsigned)(2 * max_clusters[dev][which]));
    void* args[4] = {(void*)&map_x, (void*)&map_w, (void*)&map_pf, (void*)&p};
    const cudaError_t e = cudaLaunchKernelExC(&cfg, fn, args);
    return e != cudaSuccess ? e : cudaPeekAtLastError();
}

}  // namespace cb
