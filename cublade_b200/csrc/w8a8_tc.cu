// W8A8 linear: int8 activations x int8 weights on the integer tensor-core path (tcgen05 kind::i8,
// int32 accumulators in tensor memory), per-token and per-output-channel scales applied in the
// epilogue.
//
//   y[m, n] = T( (float(sum_k xq[m, k] * wq[n, k]) * xs[m]) * ws[n] + bias[n] )
//
// The reference reserves the layer type ("w8a8" in the registry comment of
// cublade/quantization/quantizers.py:169-171) without implementing it.  Compared with the W8A16
// kernel (w8a16_tc.cu) there is nothing to widen: both operands arrive by TMA in the canonical K-major
// 128-byte-swizzled layout (128 int8 per row and stage) and feed the MMA as they are, so the CTA has
// no converter warps and a single operand ring; the integer accumulation is exact, which makes the
// result bit-reproducible on a CPU.
//
// Orientation as in the W8A16 kernel: the WEIGHT tile is UMMA operand A (M = 128 output features =
// tensor-memory lanes), the ACTIVATION tile operand B (N = tile_x <= 256 rows = columns), so scale
// and bias of an output feature are one scalar per epilogue thread.
//
// Warps of a CTA (one CTA per SM, persistent over output tiles): 0 TMA activations, 10 TMA weights,
// 1 MMA issuer (+ tensor-memory allocation), 2-9 epilogue (overlaps the next tile: two accumulators).
// No TMA multicast, no clusters.  Every mbarrier wait is bounded; on expiry the kernel raises the
// per-device error flag, all roles leave their loops, tensor memory is released, the kernel returns.
#include "tc_common.cuh"

#include <cstdlib>
#include <mutex>

namespace cb {

unsigned int* w8a16_tc_error_word();  // the per-device flag of the tensor-core kernels (w8a16_tc.cu)

namespace {

using namespace tc;

constexpr int kTileN = 128;     // output features per tile = UMMA M
constexpr int kMaxTileX = 256;  // activation rows per tile = UMMA N
constexpr int kBlockK8 = 128;   // int8 k per stage: one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kEpiWarps = 8;  // two per tensor-memory lane quarter, each draining every other 32-column chunk
constexpr int kThreads = (3 + kEpiWarps) * 32;
constexpr int kWWarp = 2 + kEpiWarps;
constexpr int kTmemCols = 512;
constexpr uint32_t kBytesX = kMaxTileX * kBlockK8;  // 32768
constexpr uint32_t kBytesW = kTileN * kBlockK8;     // 16384

struct Smem {
    static constexpr uint32_t x = 0;
    static constexpr uint32_t w = x + kStages * kBytesX;
    static constexpr uint32_t bars = w + kStages * kBytesW;
    // full[kStages] (two producers), empty[kStages], tmem_full[2], tmem_empty[2]
    static constexpr uint32_t n_bars = 2 * kStages + 4;
    static constexpr uint32_t tmem_slot = bars + n_bars * 8;
    static constexpr uint32_t abort_flag = tmem_slot + 4;
    static constexpr uint32_t total = abort_flag + 4;
};
constexpr uint32_t kSmemBytes = Smem::total + 1024;

struct Params {
    int64_t M, N, K;
    const float* xs;  // [M] per-token scales
    const void* ws;   // [N] per-output-channel scales
    int ws_dtype;
    const void* bias;  // [N] or nullptr
    int bias_dtype;
    void* y;
    int64_t ldy;
    int tile_x, tiles_x, tiles_n;
    unsigned int* error_flag;
};

// Epilogue of one tile for one warp: lanes = 32 output features (one tensor-memory lane quarter), `part` of
// `parts` warps sharing the quarter takes every parts-th chunk of 32 token columns.  The tcgen05.ld of the
// next chunk is in flight while the current one is scaled and stored: a tensor-memory load takes a few
// thousand cycles while the MMAs of the next tile are writing the other accumulator, and a drain that
// waits for each load on its own (first version) took 1.7x as long as the tile's main loop.
template <typename T>
__device__ __forceinline__ void drain_accumulator(const Params& p, uint32_t taddr, int part, int parts, int64_t m_base,
                                                  int64_t n, bool n_ok, float wscale, float bias, int lane) {
    T* y = static_cast<T*>(p.y);
    const int nchunks = (p.tile_x + 31) / 32;
    auto scales_of = [&](int ch) {
        const int64_t m_lane = m_base + ch * 32 + lane;
        return m_lane < p.M ? __ldg(p.xs + m_lane) : 0.0f;  // one per-token scale per lane, handed round by shuffles
    };
    auto finish = [&](const uint32_t (&r)[32], int ch, float xs_lane) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            const float xs = __shfl_sync(0xffffffffu, xs_lane, c);
            const int64_t m = m_base + ch * 32 + c;
            if (m >= p.M || ch * 32 + c >= p.tile_x) continue;  // uniform across the warp
            float v = __fmul_rn(__fmul_rn(__int2float_rn((int)r[c]), xs), wscale);
            if (p.bias) v = __fadd_rn(v, bias);
            if (n_ok) y[m * p.ldy + n] = Widen<T>::from_float(v);
        }
    };
    uint32_t ra[32], rb[32];
    int ch = part;
    if (ch < nchunks) tmem_ld32(taddr + (uint32_t)(ch * 32), ra);
    while (ch < nchunks) {
        float xs_lane = scales_of(ch);
        tmem_ld_wait();
        int nx = ch + parts;
        if (nx < nchunks) tmem_ld32(taddr + (uint32_t)(nx * 32), rb);
        finish(ra, ch, xs_lane);
        ch = nx;
        if (ch >= nchunks) break;
        xs_lane = scales_of(ch);
        tmem_ld_wait();
        nx = ch + parts;
        if (nx < nchunks) tmem_ld32(taddr + (uint32_t)(nx * 32), ra);
        finish(rb, ch, xs_lane);
        ch = nx;
    }
}


template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
w8a8_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sx = base + Smem::x, sw = base + Smem::w;
    const uint32_t full = base + Smem::bars, empty = full + 8 * kStages;
    const uint32_t tmem_full = empty + 8 * kStages, tmem_empty = tmem_full + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + Smem::tmem_slot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gbase + Smem::abort_flag);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (int)((p.K + kBlockK8 - 1) / kBlockK8);
    const int total_tiles = p.tiles_x * p.tiles_n;
    const uint32_t x_bytes = (uint32_t)p.tile_x * kBlockK8;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) { mbar_init(full + 8 * i, 2); mbar_init(empty + 8 * i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(tmem_full + 8 * i, 1); mbar_init(tmem_empty + 8 * i, kEpiWarps); }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&map_x);
        prefetch_tmap(&map_w);
    }
    if (warp == 1) tmem_alloc(base + Smem::tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 || warp == kWWarp) {
        // ------------------------------ TMA producers (one warp per operand) ------------------------------
        if (lane == 0) {
            const bool is_x = warp == 0;
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int row = is_x ? (t % p.tiles_x) * p.tile_x : (t / p.tiles_x) * kTileN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    {
                        ok = mbar_wait(empty + 8 * s, ph ^ 1u, abort_flag);
                    }
                    if (!ok) break;
                    if (is_x) {
                        mbar_expect_tx(full + 8 * s, x_bytes);
                        tma_load_2d(sx + s * kBytesX, &map_x, kb * kBlockK8, row, full + 8 * s);
                    } else {
                        mbar_expect_tx(full + 8 * s, kBytesW);
                        tma_load_2d(sw + s * kBytesW, &map_w, kb * kBlockK8, row, full + 8 * s);
                    }
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc_i8((uint32_t)p.tile_x);
            uint32_t s = 0, ph = 0, it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++it) {
                const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
                {
                    ok = mbar_wait(tmem_empty + 8 * acc, acc_ph ^ 1u, abort_flag);  // epilogue drained this accumulator
                }
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kMaxTileX;
                for (int kb = 0; kb < num_kb; ++kb) {
                    {
                        ok = mbar_wait(full + 8 * s, ph, abort_flag);
                    }
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t adesc = make_kmajor_sw128_desc(sw + s * kBytesW);
                    const uint64_t bdesc = make_kmajor_sw128_desc(sx + s * kBytesX);
#pragma unroll
                    for (int k = 0; k < kBlockK8 / 32; ++k) {
                        // 32 int8 = 32 bytes per k step: +2 in the (>>4) start-address field
                        umma_i8(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty + 8 * s);  // the stage is free once these MMAs retire
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                umma_commit(tmem_full + 8 * acc);
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ------------------------------ epilogue ------------------------------
        const int quarter = warp & 3;  // a warp may only touch tensor-memory lanes 32 * (warp % 4) .. + 31
        uint32_t it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++it) {
            const int tx = t % p.tiles_x, tn = t / p.tiles_x;
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            const int64_t n = (int64_t)tn * kTileN + quarter * 32 + lane;
            const bool n_ok = n < p.N;
            const float wscale = n_ok ? load_scalar(p.ws, p.ws_dtype, n) : 0.0f;
            const float bias = (n_ok && p.bias) ? load_scalar(p.bias, p.bias_dtype, n) : 0.0f;
            {
                int okw = 1;
                if (lane == 0) okw = mbar_wait(tmem_full + 8 * acc, acc_ph, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
            }
            if (!ok) break;
            tc_fence_after();
            drain_accumulator<T>(p, tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kMaxTileX, (warp - 2) >> 2, kEpiWarps / 4,
                                 (int64_t)tx * p.tile_x, n, n_ok, wscale, bias, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty + 8 * acc);
        }
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag) {
        atomicExch(p.error_flag, 1u);
        __nanosleep(200000);  // let any TMA copy still in flight land before the CTA's memory is released
    }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair version: tcgen05.mma.cta_group::2 over a cluster of two CTAs.  The pair computes 256 output
// features x tile_x tokens per tile; each CTA loads its own 128 weight rows and only HALF of the activation
// tile (the hardware reads operand B from both CTAs' shared memory), so a CTA pulls 32 KB per 128-k stage
// through TMA instead of 48 KB -- the single-CTA kernel is bound by exactly that ingest.
// Signalling: every TMA load of either CTA completes on the LEADER's (rank 0) "full" barrier -- the peer's
// loads name the leader's barrier (the .cta_group::2 form of the TMA load allows a barrier of the peer CTA;
// no multicast is involved) -- so the leader's MMA thread waits on one barrier per stage and nobody relays.
// The leader frees a stage in both CTAs, and publishes a finished accumulator to both, with
// tcgen05.commit ... .multicast::cluster; the epilogue warps of both CTAs arrive on the leader's
// "accumulator drained" barrier.  All waits are bounded as in the single-CTA kernel.
// ---------------------------------------------------------------------------------------------
constexpr int kPairStages = 6;
constexpr uint32_t kPairBytesX = (kMaxTileX / 2) * kBlockK8;  // 16384: this CTA's half of the activation tile
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;                   // shared::cluster address -> same offset in CTA rank 0

struct PairSmem {
    static constexpr uint32_t x = 0;
    static constexpr uint32_t w = x + kPairStages * kPairBytesX;
    static constexpr uint32_t bars = w + kPairStages * kBytesW;
    static constexpr uint32_t n_bars = 2 * kPairStages + 4;
    static constexpr uint32_t tmem_slot = bars + n_bars * 8;
    static constexpr uint32_t abort_flag = tmem_slot + 4;
    static constexpr uint32_t total = abort_flag + 4;
};
constexpr uint32_t kPairSmemBytes = PairSmem::total + 1024;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The hardware cluster barrier has no bounded form; it is safe here because both CTAs of a pair reach it
// unconditionally: it sits only in the prologue (before any wait) and in the teardown, which every role of both CTAs
// reaches -- an expired mbarrier wait raises the CTA's abort flag, after which all of its loops (and, through the
// barriers they stop feeding, the peer's bounded waits) fall through to the teardown.
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
// TMA tile load into THIS CTA's shared memory whose bytes are counted on the leader's barrier
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
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive (once all prior MMAs of this thread retired) on the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// kind::i8, int32 accumulate, signed operands, K-major, M = 256 over the pair
__device__ __forceinline__ uint32_t make_idesc_i8_pair(uint32_t n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
w8a8_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sx = base + PairSmem::x, sw = base + PairSmem::w;
    const uint32_t full = base + PairSmem::bars, empty = full + 8 * kPairStages;
    const uint32_t tmem_full = empty + 8 * kPairStages, tmem_empty = tmem_full + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + PairSmem::tmem_slot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gbase + PairSmem::abort_flag);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (int)((p.K + kBlockK8 - 1) / kBlockK8);
    const int total_tiles = p.tiles_x * p.tiles_n;  // tiles of 256 features x tile_x tokens
    const int pair = (int)(blockIdx.x >> 1), num_pairs = (int)(gridDim.x >> 1);
    const int half_x = p.tile_x / 2;
    const uint32_t stage_bytes = (uint32_t)half_x * kBlockK8 + kBytesW;  // what ONE CTA loads per stage

    if (threadIdx.x == 0) {
        // full: one arrive.expect_tx per CTA (used on the leader only); empty: the leader's multicast commit
        for (int i = 0; i < kPairStages; ++i) { mbar_init(full + 8 * i, 2); mbar_init(empty + 8 * i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(tmem_full + 8 * i, 1); mbar_init(tmem_empty + 8 * i, 2 * kEpiWarps); }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&map_x);
        prefetch_tmap(&map_w);
    }
    if (warp == 1) tmem_alloc_pair(base + PairSmem::tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer (both operands of this CTA) ------------------------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int t = pair; t < total_tiles && ok; t += num_pairs) {
                const int row_x = (t % p.tiles_x) * p.tile_x + (int)rank * half_x;
                const int row_w = (t / p.tiles_x) * 256 + (int)rank * kTileN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(empty + 8 * s, ph ^ 1u, abort_flag);  // local: freed by the leader's multicast commit
                    if (!ok) break;
                    mbar_expect_tx_leader(full + 8 * s, stage_bytes);
                    tma_load_2d_to_leader_bar(sx + s * kPairBytesX, &map_x, kb * kBlockK8, row_x, full + 8 * s);
                    tma_load_2d_to_leader_bar(sw + s * kBytesW, &map_w, kb * kBlockK8, row_w, full + 8 * s);
                    if (++s == kPairStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader only) ------------------------------
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = make_idesc_i8_pair((uint32_t)p.tile_x);
            uint32_t s = 0, ph = 0, it = 0;
            bool ok = true;
            for (int t = pair; t < total_tiles && ok; t += num_pairs, ++it) {
                const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
                ok = mbar_spin(tmem_empty + 8 * acc, acc_ph ^ 1u, abort_flag);  // both CTAs' epilogues drained it
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kMaxTileX;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_spin(full + 8 * s, ph, abort_flag);  // arrivals and bytes come from both CTAs
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t adesc = make_kmajor_sw128_desc(sw + s * kBytesW);
                    const uint64_t bdesc = make_kmajor_sw128_desc(sx + s * kPairBytesX);
#pragma unroll
                    for (int k = 0; k < kBlockK8 / 32; ++k)
                        umma_i8_pair(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty + 8 * s);
                    if (++s == kPairStages) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                umma_commit_pair(tmem_full + 8 * acc);
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ------------------------------ epilogue (each CTA: its own 128 features) ------------------------------
        const int quarter = warp & 3;
        uint32_t it = 0;
        bool ok = true;
        for (int t = pair; t < total_tiles && ok; t += num_pairs, ++it) {
            const int tx = t % p.tiles_x, tn = t / p.tiles_x;
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            const int64_t n = (int64_t)tn * 256 + (int64_t)rank * kTileN + quarter * 32 + lane;
            const bool n_ok = n < p.N;
            const float wscale = n_ok ? load_scalar(p.ws, p.ws_dtype, n) : 0.0f;
            const float bias = (n_ok && p.bias) ? load_scalar(p.bias, p.bias_dtype, n) : 0.0f;
            {
                int okw = 1;
                if (lane == 0) okw = mbar_wait(tmem_full + 8 * acc, acc_ph, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
            }
            if (!ok) break;
            tc_fence_after();
            drain_accumulator<T>(p, tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kMaxTileX, (warp - 2) >> 2, kEpiWarps / 4,
                                 (int64_t)tx * p.tile_x, n, n_ok, wscale, bias, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(tmem_empty + 8 * acc);
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
        __nanosleep(200000);
    }
}

// Any K, any alignment: one thread per output, dp4a where the row offset allows 32-bit loads.
template <typename T>
__global__ void __launch_bounds__(256) w8a8_simple_kernel(const int8_t* __restrict__ xq, const float* __restrict__ xs,
                                                          int64_t M, int64_t K, const int8_t* __restrict__ wq, int64_t N,
                                                          const void* __restrict__ ws, int ws_dtype,
                                                          const void* __restrict__ bias, int bias_dtype,
                                                          T* __restrict__ y, int64_t ldy) {
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= M * N) return;
    const int64_t m = idx / N, n = idx - m * N;
    const int8_t* xr = xq + m * K;
    const int8_t* wr = wq + n * K;
    int acc = 0;
    for (int64_t k = 0; k < K; ++k) acc += (int)xr[k] * (int)wr[k];
    float v = __fmul_rn(__fmul_rn(__int2float_rn(acc), xs[m]), load_scalar(ws, ws_dtype, n));
    if (bias) v = __fadd_rn(v, load_scalar(bias, bias_dtype, n));
    y[m * ldy + n] = Widen<T>::from_float(v);
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

bool make_map_u8(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_outer) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner};
    cuuint32_t box[2] = {(cuuint32_t)kBlockK8, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// activation rows per tile: the multiple of 16 (<= 256) with the fewest rounds x (rows + fixed cost)
int pick_tile_x(int64_t M, int64_t N, int sms) {
    const int64_t tiles_n = (N + kTileN - 1) / kTileN;
    int best = 256;
    double best_cost = 1e300;
    for (int tx = 256; tx >= 16; tx -= 16) {
        const int64_t tiles = ((M + tx - 1) / tx) * tiles_n;
        const double cost = (double)((tiles + sms - 1) / sms) * (tx + 256);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = tx; }
    }
    return best;
}

// activation rows per pair tile (a multiple of 32 <= 256: each CTA holds half) over `pairs` CTA pairs
int pick_pair_tile_x(int64_t M, int64_t N, int pairs) {
    const int64_t tiles_n = (N + 255) / 256;
    int best = 256;
    double best_cost = 1e300;
    for (int tx = 256; tx >= 32; tx -= 32) {
        const int64_t tiles = ((M + tx - 1) / tx) * tiles_n;
        const double cost = (double)((tiles + pairs - 1) / pairs) * (tx + 256);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = tx; }
    }
    return best;
}

template <typename T>
cudaError_t launch_pair_t(const W8A8Args& a, Params p, cudaStream_t s) {
    const int pairs_avail = sm_count() / 2;
    p.tile_x = pick_pair_tile_x(a.M, a.N, pairs_avail);
    p.tiles_x = (int)((a.M + p.tile_x - 1) / p.tile_x);
    p.tiles_n = (int)((a.N + 255) / 256);
    CUtensorMap map_x, map_w;
    if (!make_map_u8(&map_x, a.xq, (uint64_t)a.K, (uint64_t)a.M, (uint32_t)(p.tile_x / 2))) return cudaErrorNotSupported;
    if (!make_map_u8(&map_w, a.wq, (uint64_t)a.K, (uint64_t)a.N, kTileN)) return cudaErrorNotSupported;
    const int64_t tiles = (int64_t)p.tiles_x * p.tiles_n;
    int pairs = (int)(tiles < pairs_avail ? tiles : pairs_avail);
    auto fn = w8a8_tc_pair_kernel<T>;
    static bool attr_done[64] = {};
    static int max_clusters[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_done[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (max_clusters[dev] == 0) {
        // a persistent schedule needs every pair resident at once
        int n = 0;
        cudaLaunchConfig_t probe = cfg;
        probe.gridDim = dim3((unsigned)(2 * pairs_avail));
        if (cudaOccupancyMaxActiveClusters(&n, fn, &probe) != cudaSuccess || n <= 0) n = pairs_avail;
        max_clusters[dev] = n;
    }
    if (pairs > max_clusters[dev]) cfg.gridDim = dim3((unsigned)(2 * max_clusters[dev]));
    void* args[3] = {(void*)&map_x, (void*)&map_w, (void*)&p};
    const cudaError_t e = cudaLaunchKernelExC(&cfg, (const void*)fn, args);
    return e != cudaSuccess ? e : cudaPeekAtLastError();
}

template <typename T>
cudaError_t launch_t(const W8A8Args& a, cudaStream_t s) {
    auto al16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    const bool tc_ok = a.K >= 16 && a.K % 16 == 0 && al16(a.xq) && al16(a.wq) && encode_fn() != nullptr;
    if (!tc_ok) {
        const int64_t total = a.M * a.N;
        w8a8_simple_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, s>>>(
            a.xq, a.xs, a.M, a.K, a.wq, a.N, a.ws, a.ws_dtype, a.bias, a.bias_dtype, static_cast<T*>(a.y), a.ldy);
        return cudaPeekAtLastError();
    }
    const int sms = sm_count();
    Params p;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.xs = a.xs; p.ws = a.ws; p.ws_dtype = a.ws_dtype; p.bias = a.bias; p.bias_dtype = a.bias_dtype;
    p.y = a.y; p.ldy = a.ldy;
    p.error_flag = w8a16_tc_error_word();
    if (!p.error_flag) return cudaErrorUnknown;
    bool use_pair = a.M >= 256 && a.N >= 256;
    if (use_pair) return launch_pair_t<T>(a, p, s);
    p.tile_x = pick_tile_x(a.M, a.N, sms);
    p.tiles_x = (int)((a.M + p.tile_x - 1) / p.tile_x);
    p.tiles_n = (int)((a.N + kTileN - 1) / kTileN);
    CUtensorMap map_x, map_w;
    if (!make_map_u8(&map_x, a.xq, (uint64_t)a.K, (uint64_t)a.M, (uint32_t)p.tile_x)) return cudaErrorNotSupported;
    if (!make_map_u8(&map_w, a.wq, (uint64_t)a.K, (uint64_t)a.N, kTileN)) return cudaErrorNotSupported;
    const int64_t tiles = (int64_t)p.tiles_x * p.tiles_n;
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(w8a8_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    w8a8_tc_kernel<T><<<grid, kThreads, kSmemBytes, s>>>(map_x, map_w, p);
    return cudaPeekAtLastError();
}

}  // namespace

cudaError_t launch_w8a8(const W8A8Args& a, cudaStream_t s) {
    if (a.out_dtype == kBF16) return launch_t<__nv_bfloat16>(a, s);
    if (a.out_dtype == kF16) return launch_t<__half>(a, s);
    return cudaErrorInvalidValue;
}

}  // namespace cb

