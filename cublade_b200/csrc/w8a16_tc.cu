// W8A16 linear for tall activations: a tcgen05 / TMEM GEMM fed by TMA that widens int8 weight
// tiles to 16-bit floats on the way to the tensor core.
//
//   y[m, n] = (sum_k x[m, k] * wq[n, k]) * scale[n] + sum_j xo[m, j] * wo[n, j] + bias[n]
//
// Replaces the reference's per-call chain "cast the whole weight to bf16, transpose it, Triton
// tl.dot GEMM, multiply by scales, add bias" (cublade/quantization/linear.py:123-135,
// cublade/kernels/triton/matmul_kernel.py:9-99) with one persistent kernel.
//
// Orientation ("swap-AB"): the WEIGHT tile is the 128-row UMMA operand A and the ACTIVATION tile
// is the (up to) 256-row operand B, so the accumulator in TMEM is D[n_local (lane), m_local
// (column)].  Consequences: (1) the int8 -> 16-bit conversion work per flop is halved compared
// with putting the weights on the 256 side; (2) the per-output-channel scale and bias are one
// scalar per TMEM lane, i.e. per epilogue thread; (3) for a fixed column m the 32 lanes of an
// epilogue warp store 32 consecutive n of y[m, :], a 64-byte contiguous segment.
//
// Warp roles in a CTA of 15 warps (one CTA per SM, persistent over output tiles):
//   warp 0      TMA producer: activation tile (bf16/f16, 128-byte swizzle) per k-block
//   warp 14     TMA producer: int8 weight tile per k-block, plus an L2 prefetch 12 k-blocks ahead
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma (M=128, N=tile_x, K=16) x4 per
//               k-block and commits to the "slot free" / "accumulator ready" barriers; also owns
//               the TMEM allocation (512 columns = two accumulators)
//   warps 2-5   epilogue: tcgen05.ld the accumulator, * scale, + outlier side product, + bias,
//               round once, store; overlaps the next tile's main loop (double-buffered TMEM)
//   warps 6-13  converters: int8 tile (shared) -> registers -> 16-bit operand A, either in shared
//               memory (canonical K-major 128-byte-swizzled UMMA layout, fence.proxy.async) or,
//               for M <= 208, straight in tensor memory (tcgen05.st), then barrier arrive
//
// One operand ring: stage s carries the activation tile, the int8 tile and the widened tile of a k-block.
// The MMA thread waits on ONE "full" barrier per k-block (TMA bytes of the activations + the eight
// converter warps) and commits to ONE "empty" barrier, which both TMA producers wait on; the converters wait
// on the int8 tile's barrier only (its producer has already waited for the stage).  The MMA thread's loop is
// the critical path: an isolated test shows ~200 cycles of other work per group of four MMAs is all the
// tensor core's queue hides, and a barrier probe costs ~100 cycles even on a completed phase.
//
// Schedule: tile t of round r goes to CTA t - r * gridDim.x.  A schedule without one full round
// (fewer tiles than SMs) splits its tiles along K over the idle CTAs: every split stores its fp32
// partial accumulator to its own slab of the workspace, and a small second kernel adds the slabs
// of a tile in a fixed order and applies the ordinary epilogue (scale, outlier side product, bias,
// each rounded as the reference rounds).  Nobody waits for anybody, nothing is zeroed, and the result is deterministic.
//
// No TMA multicast, no clusters, no peer memory.  Every mbarrier wait is bounded: on expiry the
// kernel raises an error flag in global memory, every role leaves its loop, TMEM is released and
// the kernel returns.

#include "tc_common.cuh"

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <type_traits>

namespace cb {

namespace {

using namespace tc;



constexpr int kTileN = 128;  // weight rows (output features) per tile = UMMA M
constexpr int kConvWarps = 8;
constexpr int kEpiWarps = 4;
constexpr int kThreads = (4 + kEpiWarps + kConvWarps) * 32;  // + TMA(x), MMA, TMA(w8), second MMA issuer
constexpr int kW8Warp = 2 + kEpiWarps + kConvWarps;         // int8 weight producer
constexpr int kPfBlocks = 4;                                // k-blocks of weights per L2 prefetch
constexpr int kMma2Warp = kW8Warp + 1;                      // second MMA issuer (kTmemA128 only, idle otherwise)
constexpr int kTmemCols = 512;
constexpr uint32_t kBytesW8 = kTileN * kBlockK;  // 8192

// Where the widened weight tile (UMMA operand A) lives.
//   kSmemA: converters write it to shared memory in the canonical K-major 128-byte-swizzled layout;
//           activation tiles up to 256 rows, two 256-column accumulators fill tensor memory.
//   kTmemA: converters write it straight into tensor memory (tcgen05.st) and the MMA reads A from
//           there.  Shared memory then carries only the two TMA rings and one read of the int8 tile:
//           80 KiB of shared-memory traffic per k-block instead of 112 KiB -- at full tensor rate the
//           shared-memory path, not the tensor core, is what saturates.  Tensor memory holds two
//           208-column accumulators plus three 32-column A stages, so activation tiles stop at 208 rows.
//   kTmemA128: kTmemA for activation tiles of at most 128 rows: two 128-column accumulators leave room for eight
//           A stages, so the operand ring is eight k-blocks deep -- with one tile per CTA (M <= 128) the kernel is
//           a weight stream whose pace is set by how many k-blocks are in flight, not by the tensor core.
//   kTmemA64: the same for tiles of at most 64 rows: twelve stages.
//   kTmemA2: kTmemA with TWO activation tiles of up to 208 rows per work item: a widened weight k-block in tensor
//           memory is used by two MMAs, one per activation tile, each into its own accumulator: the widening and
//           the int8 tile's trip through shared memory are per weight k-block, so a second activation tile halves
//           them per output row (ALU pipe 52 -> 34 %), and the larger items fill the rounds better.
//           The two accumulators fill tensor memory beside three A stages, so they are not double-buffered: the
//           next work item's MMAs into an accumulator wait until the epilogue has drained it (a few microseconds
//           per ~30 us item).
enum AMode : int { kSmemA = 0, kTmemA = 1, kTmemA128 = 2, kTmemA64 = 3, kTmemA2 = 4 };

template <int MODE>
struct Cfg {
    static constexpr int kMaxTileX = MODE == kSmemA ? 256 : (MODE == kTmemA || MODE == kTmemA2 ? 208 : (MODE == kTmemA128 ? 128 : 64));  // activation rows per tile = UMMA N
    static constexpr int kHalves = MODE == kTmemA2 ? 2 : 1;  // activation tiles (and accumulators) per work item
    // ONE operand ring: stage s holds the activation tile and the widened weight tile of a k-block, one
    // "full" barrier (TMA bytes + the eight converter warps) and one "empty" barrier (one tcgen05.commit) per
    // stage -- the MMA thread's loop is the critical path of the kernel, and every barrier it probes or
    // commits to costs it time the tensor core spends idle.
    static constexpr int kStages = MODE == kSmemA ? 4 : (MODE == kTmemA ? 6 : (MODE == kTmemA128 ? 8 : (MODE == kTmemA64 ? 12 : 3)));
    // kTmemA: only three 32-column A stages fit beside two 208-column accumulators, but shared memory holds six
    // activation + int8 stages: ring slot s uses tensor-memory A stage s % 3, and a converter waits, besides the int8
    // tile, for the MMAs of the k-block three slots back (the `empty` barrier of that slot) before it overwrites the stage.
    static constexpr int kTmemAStages = MODE == kTmemA ? 3 : kStages;
    // kTmemA128 has TWO MMA issuers: a thread needs ~350 cycles to issue the four MMAs of a k-block and commit
    // them, whatever their size, so with short activation tiles one issuer, not the tensor core, sets the pace.
    // Issuer i takes the k-blocks of parity i of a work item and accumulates into accumulator i; the epilogue adds
    // the two (the accumulators then do not alternate between tiles: short tiles drain in a few hundred cycles).
    static constexpr bool kDual = MODE == kTmemA128 || MODE == kTmemA64;
    // ... and THREE converter groups of four warps (one warp per tensor-memory lane quarter, the whole 64 k of
    // its 32 weight rows), each taking every third k-block: a warp's chain per k-block -- barrier probe, shared-
    // memory loads, widening, tcgen05.st, wait::st, fence, arrive -- is ~600 cycles of mostly latency, and with all
    // eight converter warps working on the SAME k-block that chain, not the memory system, paced the kernel
    // (timing floors: no change with 8 or 128 weight rows per TMA box, 12 instead of 8 stages, or no MMAs).
    // The third group are the epilogue warps, idle during a tile's main loop in these modes.
    static constexpr int kConvGroups = kDual ? 3 : 2;  // kTmemA: the two groups of converter warps
    static constexpr int kFullArrivals = MODE == kSmemA ? 1 + kConvWarps : 1 + 4;  // TMA expect_tx + converter warps per stage
    static constexpr int kStagesX = kStages;
    static constexpr int kStagesA = kStages;
    static constexpr int kStagesW8 = kStages;                      // int8 weight tiles (8 KiB each), part of the same ring
    static constexpr int kAccStride = kMaxTileX;                   // columns between the two accumulators
    static constexpr int kACol = 2 * kMaxTileX;                    // first tensor-memory column of the A stages (kTmemA)
    static constexpr int kAColsPerStage = kBlockK / 2;             // two 16-bit k per 32-bit column
    static constexpr uint32_t kBytesXHalf = kMaxTileX * kBlockK * 2;  // 32768 / 26624, both multiples of 1024
    static constexpr uint32_t kBytesX = kHalves * kBytesXHalf;
    static constexpr uint32_t kBytesA = MODE == kSmemA ? kTileN * kBlockK * 2 : 0;
    // shared memory map
    static constexpr uint32_t x = 0;
    static constexpr uint32_t a = x + kStagesX * kBytesX;
    static constexpr uint32_t w8 = a + kStagesA * kBytesA;
    static constexpr uint32_t bars = w8 + kStagesW8 * kBytesW8;
    // barriers: full[kStages], empty[kStages], full_w8[kStages], tmem_full[2], tmem_empty[2]
    static constexpr uint32_t n_bars = 3 * kStages + 4;
    static constexpr uint32_t tmem_slot = bars + n_bars * 8;
    static constexpr uint32_t abort_flag = tmem_slot + 4;
    // Scratch of the epilogue warps for the outlier side product on the warp-level tensor-core path (see the epilogue):
    // 32 features x 32 activation rows of fp32 per warp, 33 floats per feature so that a lane reading its own feature's
    // row and its neighbours reading theirs hit 32 different banks.  kSmemA's four 56 KB stages leave no room for it.
    static constexpr bool kSideMma = MODE != kSmemA;
    static constexpr uint32_t kSideBytes = 32 * 33 * 4;
    static constexpr uint32_t side = (abort_flag + 4 + 15u) & ~15u;
    static constexpr uint32_t total = side + (kSideMma ? kEpiWarps * kSideBytes : 4);
    static constexpr uint32_t kSmemBytes = total + 1024;  // + slack to align the base to 1024 B
    static_assert(kACol + kTmemAStages * kAColsPerStage <= kTmemCols || MODE == kSmemA, "tensor memory map");
    static_assert(kSmemBytes <= 232448, "shared memory map");
};

struct TcParams {
    int64_t M, N, K;
    const void* scales;
    int scales_dtype;
    const void* bias;
    int bias_dtype;
    const void* xo;  // [M, KO] 16-bit
    const void* wo;  // [N, KO] 16-bit
    int64_t KO, ldxo;
    int weights_ready;  // 1: the int8 weights were not written by the kernel ahead in the stream (see W8A16Args)
    int side_vec;    // 1: KO % 8 == 0, ldxo % 8 == 0, xo and wo 16-byte aligned -> the side product reads 16-byte chunks
    void* y;
    int64_t ldy;
    int tile_x;      // activation rows per tile (multiple of 16, <= 256)
    int tiles_x;     // ceil(M / (tile_x * activation tiles per work item))
    int tiles_n;     // ceil(N / 128)
    unsigned int* error_flag;  // global; set to 1 when a bounded wait expired
    // schedule (see work_item)
    int full_rounds;  // rounds in which every CTA owns a whole tile
    int rem_tiles;    // tiles of the last, partly filled round
    int splits;       // K-splits per tile of that round (1 = whole tiles)
    float* partial;   // [rem_tiles][splits][tile_x][128] fp32 partial products (splits > 1)
};

// One unit of work of a CTA: k-blocks [kb0, kb1) of an output tile.  split_slot >= 0 marks a
// partial product that goes to slab split_slot of the workspace.
struct WorkItem {
    int tile, kb0, kb1, split_slot;
};

// idx-th item of this CTA; every warp role walks the same sequence.
__device__ __forceinline__ bool work_item(const TcParams& p, int num_kb, int idx, WorkItem& w) {
    const int P = (int)gridDim.x, b = (int)blockIdx.x;
    if (idx < p.full_rounds) {
        w.tile = b + idx * P; w.kb0 = 0; w.kb1 = num_kb; w.split_slot = -1;
        return true;
    }
    if (idx > p.full_rounds || b >= p.rem_tiles * p.splits) return false;
    const int j = b / p.splits, sp = b - j * p.splits;
    w.tile = p.full_rounds * P + j;
    w.kb0 = (int)((int64_t)sp * num_kb / p.splits);
    w.kb1 = (int)((int64_t)(sp + 1) * num_kb / p.splits);
    w.split_slot = p.splits > 1 ? b : -1;  // slab index = j * splits + sp
    return true;
}

// Outlier columns handled by the epilogue's CUDA-core side product.  The loop serves any count; it costs
// M * N * KO fused multiply-adds on four warps per SM, so it is meant for the LLM.int8 regime (up to ~1 % of
// the input features).  Beyond this bound the call falls back to the streaming kernel.
constexpr int kMaxKO = 512;


// d += a (16 x 16, row-major fragments) . b (16 x 8, column-major fragments), fp32 accumulation, on the warp-level
// tensor-core path: the outlier side product of a 32 x 32 block of outputs is eight of these instead of ~20 CUDA-core
// instructions per output.
template <typename A>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (Widen<A>::kBf16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// side += sum over the eight 16-bit pairs of two 16-byte chunks (activation chunk x, weight chunk w), in order
template <typename A>
__device__ __forceinline__ float dot8(const uint4& x, const uint4& w, float side) {
    const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float2 a, b;
        if constexpr (Widen<A>::kBf16) {
            a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[k]));
            b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ww[k]));
        } else {
            a = __half22float2(*reinterpret_cast<const __half2*>(&xw[k]));
            b = __half22float2(*reinterpret_cast<const __half2*>(&ww[k]));
        }
        side = fmaf(a.x, b.x, side);
        side = fmaf(a.y, b.y, side);
    }
    return side;
}

// Epilogue of one K-split of a tile (one warp = 32 output features x tile_x rows): store the fp32
// partial accumulator to this split's slab, [row][feature] so that a warp writes 128 contiguous
// bytes per row.  Kept out of line: the code of the ordinary epilogue is not affected by it.
// second_offset > 0: the partial product is the sum of two accumulators that many columns apart.
__device__ __noinline__ void epilogue_split(const TcParams& p, uint32_t taddr, uint32_t second_offset, int slab, int n_local,
                                            int64_t m_base) {
    float* part = p.partial + (size_t)slab * ((size_t)p.tile_x * kTileN) + n_local;
    for (int c0 = 0; c0 < p.tile_x; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + (uint32_t)c0, r);
        if (second_offset) {
            uint32_t r2[32];
            tmem_ld32(taddr + second_offset + (uint32_t)c0, r2);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) + __uint_as_float(r2[c]));
        }
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            if (m_base + c0 + c >= p.M || c0 + c >= p.tile_x) break;  // uniform across the warp
            __stcg(part + (size_t)(c0 + c) * kTileN, __uint_as_float(r[c]));
        }
    }
}

// Second kernel of a call whose last round was split: one warp per output row of a split tile adds
// the slabs in split order and finishes the row (scale, outlier side product, bias, each rounded as the reference rounds).
template <typename A>
__global__ void __launch_bounds__(256) w8a16_tc_fixup_kernel(const __grid_constant__ TcParams p, int grid_main) {
    pdl_wait();  // the slabs come from the kernel ahead
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blocks_per_tile = (p.tile_x + 7) / 8;
    const int j = blockIdx.x / blocks_per_tile;                      // tile of the split round
    const int row = (blockIdx.x - j * blocks_per_tile) * 8 + warp;  // row inside the tile
    const int tile = p.full_rounds * grid_main + j;
    const int tx = tile % p.tiles_x, tn = tile / p.tiles_x;
    const int64_t m = (int64_t)tx * p.tile_x + row;
    if (row >= p.tile_x || m >= p.M) return;
    const size_t slab_elems = (size_t)p.tile_x * kTileN;
    const float* part = p.partial + (size_t)j * p.splits * slab_elems + (size_t)row * kTileN + lane;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int sp = 0; sp < p.splits; ++sp) {
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q] += __ldcg(part + sp * slab_elems + q * 32);
    }
    const A* xrow = static_cast<const A*>(p.xo) + m * p.ldxo;
    A* y = static_cast<A*>(p.y);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int64_t n = (int64_t)tn * kTileN + q * 32 + lane;
        if (n >= p.N) continue;
        // the reference's rounding order (see ref_round in tc_common.cuh)
        float v = ref_round<A>(ref_round<A>(acc[q]) * ref_round<A>(load_scalar(p.scales, p.scales_dtype, n)));
        if (p.KO > 0) {
            const A* wrow = static_cast<const A*>(p.wo) + n * p.KO;
            float side = 0.0f;
            for (int k = 0; k < (int)p.KO; ++k)
                side = fmaf(Widen<A>::to_float(__ldg(xrow + k)), Widen<A>::to_float(__ldg(wrow + k)), side);
            v = ref_round<A>(v + ref_round<A>(side));
        }
        if (p.bias) v = ref_round<A>(v + ref_round<A>(load_scalar(p.bias, p.bias_dtype, n)));
        y[m * p.ldy + n] = Widen<A>::from_float(v);
    }
}

template <typename A, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
w8a16_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ CUtensorMap map_pf,
                const __grid_constant__ TcParams p) {
    using C = Cfg<MODE>;
    constexpr int kStagesX = C::kStagesX, kStagesA = C::kStagesA, kStagesW8 = C::kStagesW8;
    constexpr uint32_t kBytesX = C::kBytesX, kBytesA = C::kBytesA;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte aligned base (the 128-byte swizzle pattern repeats every 1024 bytes)
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sx = base + C::x, sa = base + C::a, sw8 = base + C::w8;
    const uint32_t bars = base + C::bars;
    const uint32_t full_x = bars, empty_x = full_x + 8 * kStagesX;  // the operand ring's full / empty barriers
    const uint32_t full_a = full_x, empty_a = empty_x;              // (the converters and the activation TMA share them)
    const uint32_t full_w8 = empty_x + 8 * kStagesX;
    const uint32_t tmem_full = full_w8 + 8 * kStagesW8, tmem_empty = tmem_full + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + C::tmem_slot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gbase + C::abort_flag);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (int)((p.K + kBlockK - 1) / kBlockK);
    const uint32_t x_bytes = (uint32_t)p.tile_x * kBlockK * 2;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStagesX; ++i) { mbar_init(full_x + 8 * i, C::kFullArrivals); mbar_init(empty_x + 8 * i, 1); }
        for (int i = 0; i < kStagesW8; ++i) mbar_init(full_w8 + 8 * i, 1);
        for (int i = 0; i < 2; ++i) { mbar_init(tmem_full + 8 * i, 1); mbar_init(tmem_empty + 8 * i, kEpiWarps); }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&map_x);
        prefetch_tmap(&map_w);
        prefetch_tmap(&map_pf);
    }
    if (warp == 1) tmem_alloc(base + C::tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic launch edge.  This CTA may be running while the kernel ahead of it in the stream has not finished:
    // barriers, tensor memory and the weight stream (weights_ready) are set up under that kernel's tail, and every warp
    // that touches what that kernel may have written -- the activation producer, the epilogue (outlier activations,
    // the output, the K-split slabs) -- waits for it first.  The kernel behind this one may be set up in turn.
    if (p.weights_ready) pdl_trigger();

    // Tensor-memory modes: widen the k-blocks of work item w that belong to converter group `group` (every
    // kConvGroups-th k-block of the CTA's running count) into their tensor-memory stages.  A thread owns weight row
    // 32 * quarter + lane = its tensor-memory lane; the int8 tile arrived with the 64-byte TMA swizzle, so the eight
    // lanes of a quarter-warp hit eight different bank groups.  State of the calling warp: ring stage,
    // phase and the running count modulo kConvGroups.  Returns false when a wait gave up.
    uint32_t cv_s = 0, cv_ph = 0, cv_g = 0;
    auto convert_item_tmem = [&](const WorkItem& w, uint32_t group) -> bool {
        const int quarter = warp & 3;  // a warp may only touch tensor-memory lanes 32 * (warp % 4) .. + 31
        const int row = quarter * 32 + lane;
        const uint32_t swz = (uint32_t)((row >> 1) & 3);  // 64-byte TMA swizzle: chunk c of row r sits at c ^ ((r >> 1) & 3)
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
            if (cv_g == group) {
                int okw = 1;
                if (lane == 0) okw = mbar_wait(full_w8 + 8 * cv_s, cv_ph, abort_flag) ? 1 : 0;
                if constexpr (C::kTmemAStages != C::kStages) {
                    // the tensor-memory stage is shared with the slot kTmemAStages back: its MMAs must have retired
                    // (same ring round for the upper slots, the round before for the lower ones)
                    if (lane == 0 && okw) {
                        const uint32_t back = cv_s >= (uint32_t)C::kTmemAStages ? cv_s - C::kTmemAStages : cv_s + C::kTmemAStages;
                        okw = mbar_wait(empty_a + 8 * back, cv_s >= (uint32_t)C::kTmemAStages ? cv_ph : cv_ph ^ 1u, abort_flag) ? 1 : 0;
                    }
                }
                if (__shfl_sync(0xffffffffu, okw, 0) == 0) return false;
                tc_fence_after();
                const uint32_t a_stage = C::kTmemAStages == C::kStages ? cv_s : cv_s % (uint32_t)C::kTmemAStages;
                const uint32_t rbase = sw8 + cv_s * kBytesW8 + (uint32_t)(row * 64);
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
                                  (uint32_t)(C::kACol + a_stage * C::kAColsPerStage + khalf * 16), o);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(full_a + 8 * cv_s);
            }
            if (++cv_g == (uint32_t)C::kConvGroups) cv_g = 0;
            if (++cv_s == (uint32_t)C::kStages) { cv_s = 0; cv_ph ^= 1u; }
        }
        return true;
    };

    if (warp == 0) {
        // ------------------------------ TMA producer, activations ------------------------------
        // The two producers are separate warps: probing a barrier costs ~130 cycles even when its
        // phase is complete and issuing a TMA ~100, so one thread feeding both rings cannot stay
        // ahead of the tensor core.
        if (lane == 0) {
            pdl_wait();
            if (!p.weights_ready) pdl_trigger();
            uint32_t s = 0, ph = 0;
            bool ok = true;
            WorkItem w;
            for (int idx = 0; ok && work_item(p, num_kb, idx, w); ++idx) {
                const int row_x = (w.tile % p.tiles_x) * p.tile_x * C::kHalves;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    {
                        ok = mbar_wait(empty_x + 8 * s, ph ^ 1u, abort_flag);
                    }
                    if (!ok) break;
                    mbar_expect_tx(full_x + 8 * s, x_bytes * C::kHalves);
                    tma_load_2d(sx + s * kBytesX, &map_x, kb * kBlockK, row_x, full_x + 8 * s);
                    // second activation tile of the item (rows beyond M arrive as zeros)
                    if constexpr (C::kHalves == 2)
                        tma_load_2d(sx + s * kBytesX + C::kBytesXHalf, &map_x, kb * kBlockK, row_x + p.tile_x, full_x + 8 * s);
                    if (++s == kStagesX) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == kW8Warp) {
        // ------------------------------ TMA producer, int8 weights ------------------------------
        if (lane == 0) {
            if (!p.weights_ready) pdl_wait();
            constexpr int kAhead = 12;  // k-blocks of weights requested into L2 ahead of their TMA load
            uint32_t s = 0, ph = 0;
            bool ok = true;
            WorkItem w, nx;
            for (int idx = 0; ok && work_item(p, num_kb, idx, w); ++idx) {
                const int row_w = (w.tile / p.tiles_x) * kTileN;
                const bool has_next = work_item(p, num_kb, idx + 1, nx);
                const int row_w_next = has_next ? (nx.tile / p.tiles_x) * kTileN : 0;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    // One prefetch covers kPfBlocks k-blocks (a wider box of the same tensor): every instruction
                    // of this thread costs 100-250 cycles of issue, and with a prefetch per k-block its loop
                    // (~600 cycles) paced the whole kernel for short activation tiles.
                    if (((kb - w.kb0) & (kPfBlocks - 1)) == 0) {
                        if (kb + kAhead < w.kb1) tma_prefetch_l2_2d(&map_pf, (kb + kAhead) * kBlockK, row_w);
                        else if (has_next && nx.kb0 + (kb + kAhead - w.kb1) < nx.kb1)
                            tma_prefetch_l2_2d(&map_pf, (nx.kb0 + kb + kAhead - w.kb1) * kBlockK, row_w_next);
                    }
                    {
                        // the int8 staging buffer of a stage is free when the stage is: the MMAs that retired
                        // consumed what the converters made of it
                        ok = mbar_wait(empty_a + 8 * s, ph ^ 1u, abort_flag);
                    }
                    if (!ok) break;
                    mbar_expect_tx(full_w8 + 8 * s, kBytesW8);
                    tma_load_2d(sw8 + s * kBytesW8, &map_w, kb * kBlockK, row_w, full_w8 + 8 * s);
                    if (++s == kStagesW8) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1 || (C::kDual && warp == kMma2Warp)) {
        // ------------------------------ MMA issuer(s) ------------------------------
        if (lane == 0) {
            const uint32_t me = warp == 1 ? 0u : 1u;  // kDual: issuer `me` owns accumulator `me` and the k-blocks of parity `me`
            const uint32_t idesc = make_idesc(Widen<A>::kBf16, (uint32_t)p.tile_x);
            // This thread's loop is the critical path of the kernel: tcgen05.mma issue is not free-running
            // (cycle counters: the four issues of a k-block take about as long as their execution), so
            // whatever else the loop does -- barrier probes, commits -- is time the tensor core idles.
            // Hence one wait and one commit per k-block.
            uint32_t s_a = 0, ph_a = 0, it = 0;
            bool ok = true;
            WorkItem w;
            for (int idx = 0; ok && work_item(p, num_kb, idx, w); ++idx, ++it) {
                // kHalves == 2: both accumulators belong to the item (one per activation tile), neither alternates
                const uint32_t acc = C::kDual ? me : (C::kHalves == 2 ? 0u : (it & 1u));
                const uint32_t acc_ph = (C::kDual || C::kHalves == 2) ? (it & 1u) : ((it >> 1) & 1u);
                {
                    ok = mbar_wait(tmem_empty + 8 * acc, acc_ph ^ 1u, abort_flag);  // epilogue drained this accumulator
                }
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * C::kAccStride;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    if (C::kDual && (uint32_t)((kb - w.kb0) & 1) != me) {  // the other issuer's k-block: only keep step with the ring
                        if (++s_a == kStagesA) { s_a = 0; ph_a ^= 1u; }
                        continue;
                    }
                    const int kb_first = C::kDual ? w.kb0 + (int)me : w.kb0;  // first k-block into this accumulator
                    {
                        ok = mbar_wait(full_a + 8 * s_a, ph_a, abort_flag);  // activation bytes landed and weights widened
                    }
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t bdesc = make_kmajor_sw128_desc(sx + s_a * kBytesX);
                    if constexpr (MODE == kSmemA) {
                        const uint64_t adesc = make_kmajor_sw128_desc(sa + s_a * kBytesA);
#pragma unroll
                        for (int k = 0; k < kBlockK / 16; ++k) {
                            // +32 bytes per 16-element k step: +2 in the (>>4) start-address field
                            umma_f16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                                     (kb > kb_first || k > 0) ? 1u : 0u);
                        }
                    } else {
                        const uint32_t a_tmem = tmem_base + C::kACol + (s_a % (uint32_t)C::kTmemAStages) * C::kAColsPerStage;
#pragma unroll
                        for (int k = 0; k < kBlockK / 16; ++k) {
                            // 16 k = 8 columns of A, 32 bytes of every B row
                            umma_f16_tmem_a(d_tmem, a_tmem + (uint32_t)(8 * k), bdesc + (uint64_t)(2 * k), idesc,
                                            (kb > kb_first || k > 0) ? 1u : 0u);
                        }
                        if constexpr (C::kHalves == 2) {
                            // the same widened weights against the second activation tile, into the second accumulator
                            if (kb == w.kb0) {
                                ok = mbar_wait(tmem_empty + 8, acc_ph ^ 1u, abort_flag);
                                if (!ok) break;
                                tc_fence_after();
                            }
                            const uint64_t bdesc1 = make_kmajor_sw128_desc(sx + s_a * kBytesX + C::kBytesXHalf);
#pragma unroll
                            for (int k = 0; k < kBlockK / 16; ++k)
                                umma_f16_tmem_a(d_tmem + C::kAccStride, a_tmem + (uint32_t)(8 * k), bdesc1 + (uint64_t)(2 * k), idesc,
                                                (kb > kb_first || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(empty_a + 8 * s_a);  // the stage is free once these MMAs retire
                    if (++s_a == kStagesA) { s_a = 0; ph_a ^= 1u; }
                }
                if (!ok) break;
                // accumulator complete -> epilogue (an issuer whose parity had no k-block in this item commits nothing
                // pending: the barrier completes at once and the epilogue ignores that accumulator)
                umma_commit(tmem_full + 8 * acc);
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ------------------------------ epilogue ------------------------------
        const int quarter = warp & 3;  // a warp may only touch TMEM lanes 32*(warp%4) .. +31
        const A* xo = static_cast<const A*>(p.xo);
        pdl_wait();
        const A* wo = static_cast<const A*>(p.wo);
        A* y = static_cast<A*>(p.y);
        uint32_t it = 0;
        bool ok = true;
        WorkItem w;
        for (int idx = 0; ok && work_item(p, num_kb, idx, w); ++idx, ++it) {
            if constexpr (C::kDual) {
                // third converter group during the tile's main loop, epilogue afterwards
                if (!convert_item_tmem(w, 2u)) { ok = false; break; }
            }
            const int tx = w.tile % p.tiles_x, tn = w.tile / p.tiles_x;
            // kDual: both accumulators belong to this tile (one per MMA issuer), the same barrier phase on both
            const uint32_t acc = (C::kDual || C::kHalves == 2) ? 0u : (it & 1u);
            const uint32_t acc_ph = (C::kDual || C::kHalves == 2) ? (it & 1u) : ((it >> 1) & 1u);
            const uint32_t second = (C::kDual && w.kb1 - w.kb0 >= 2) ? (uint32_t)C::kAccStride : 0u;  // issuer 1 had work
            const int n_local = quarter * 32 + lane;
            const int64_t n = (int64_t)tn * kTileN + n_local;
            const bool n_ok = n < p.N;
            const float scale = n_ok ? ref_round<A>(load_scalar(p.scales, p.scales_dtype, n)) : 0.0f;
            const bool has_bias = p.bias != nullptr;
            const float bias = (n_ok && has_bias) ? ref_round<A>(load_scalar(p.bias, p.bias_dtype, n)) : 0.0f;
            const uint32_t scale2 = Widen<A>::pack2(scale, scale), bias2 = Widen<A>::pack2(bias, bias);
            // Outlier side product (see side_vec): 16-byte chunks of eight columns.  Up to kSideRegs chunks (16 outlier
            // columns) stay in registers: this lane's weight chunks are fetched once per tile, and the activation chunks
            // of a 32-row block are fetched by ONE load per chunk -- lane l takes row l -- right after the block's
            // tensor-memory load is issued, then handed round the warp by shuffles.  A global load per output row, even
            // eight at a time, left the epilogue longer than the tile's main loop (M = 2048: 371 against 240 us).
            constexpr int kSideRegs = 2;
            const int side_chunks = p.side_vec ? (int)(p.KO >> 3) : 0;
            const bool side_fast = side_chunks > 0 && side_chunks <= kSideRegs;
            const uint4* wrow4 = reinterpret_cast<const uint4*>(wo + (n_ok ? n : 0) * p.KO);
            // With room for the scratch (every mode but kSmemA) the side product of a 32 x 32 block runs as eight
            // mma.m16n8k16: operand A = this warp's 32 outlier-weight rows (two 16-row tiles; fragments fetched once per
            // work item), operand B = the block's outlier activations (four 8-row tiles), k = the <= 16 outlier columns
            // (zeros beyond KO).  The products land in the MMA's own layout -- feature 16 i + g (+ 8), row 8 j + 2 t (+ 1)
            // -- and go through the warp's scratch so that lane l reads the 32 values of ITS feature.  fp32 throughout,
            // rounded to the activation type where the reference rounds its outlier product.
            const bool side_mma = C::kSideMma && side_fast;
            const int g8 = lane >> 2, t4 = lane & 3;
            uint32_t afr[2][4] = {{0u, 0u, 0u, 0u}, {0u, 0u, 0u, 0u}};
            uint4 wreg[kSideRegs];
            if (side_mma) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int64_t n_lo = (int64_t)tn * kTileN + quarter * 32 + 16 * i + g8, n_hi = n_lo + 8;
                    const uint32_t* r_lo = reinterpret_cast<const uint32_t*>(wo + (n_lo < p.N ? n_lo : p.N - 1) * p.KO);
                    const uint32_t* r_hi = reinterpret_cast<const uint32_t*>(wo + (n_hi < p.N ? n_hi : p.N - 1) * p.KO);
                    afr[i][0] = __ldg(r_lo + t4);
                    afr[i][1] = __ldg(r_hi + t4);
                    if (side_chunks > 1) {
                        afr[i][2] = __ldg(r_lo + 4 + t4);
                        afr[i][3] = __ldg(r_hi + 4 + t4);
                    }
                }
            }
#pragma unroll
            for (int ch = 0; ch < kSideRegs; ++ch)
                wreg[ch] = (!side_mma && n_ok && ch < side_chunks) ? __ldg(wrow4 + ch) : make_uint4(0u, 0u, 0u, 0u);
            // Operand-B fragments (outlier activations) of a 32-row block are fetched one block ahead -- the first block's
            // before the wait for the accumulator, a tile's first block's during the last block of the tile before -- so
            // that their trip to L2 runs under other work: issued inside their own block, as they were at first, every
            // block stalled on them (M = 2048: 13 blocks per work item, +26 us).
            auto load_bfr = [&](int64_t mb, int c0, uint32_t (&b)[4][2]) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int64_t mr = mb + c0 + 8 * j + g8;
                    const uint32_t* xr32 = reinterpret_cast<const uint32_t*>(xo + (mr < p.M ? mr : p.M - 1) * p.ldxo);
                    b[j][0] = __ldg(xr32 + t4);
                    b[j][1] = side_chunks > 1 ? __ldg(xr32 + 4 + t4) : 0u;
                }
            };
            uint32_t bnext[4][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}, {0u, 0u}};
            if (side_mma) load_bfr((int64_t)tx * C::kHalves * p.tile_x, 0, bnext);
            {
                int okw = 1;
                if (lane == 0) {
                    okw = mbar_wait(tmem_full + 8 * acc, acc_ph, abort_flag) ? 1 : 0;
                    if (C::kDual && okw) okw = mbar_wait(tmem_full + 8, acc_ph, abort_flag) ? 1 : 0;
                }
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
            }
            if (!ok) break;
            tc_fence_after();
            for (int half = 0; half < C::kHalves; ++half) {  // kHalves == 2: the item's two activation tiles in turn
            const int64_t m_base = ((int64_t)tx * C::kHalves + half) * p.tile_x;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (acc + (uint32_t)half) * C::kAccStride;
            if (C::kHalves == 1 && w.split_slot >= 0) {
                // a K-split of a tile of the last round: rare path, kept out of line so that the code of
                // the ordinary epilogue below is not affected by it
                epilogue_split(p, taddr, second, w.split_slot, n_local, m_base);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(tmem_empty + 8 * acc);
                    if (C::kDual) mbar_arrive(tmem_empty + 8);
                }
                continue;
            }
            for (int c0 = 0; c0 < p.tile_x && m_base + c0 < p.M; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + (uint32_t)c0, r);
                if constexpr (C::kDual) {
                    if (second) {
                        uint32_t r2[32];
                        tmem_ld32(taddr + second + (uint32_t)c0, r2);
                        tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) + __uint_as_float(r2[c]));
                    }
                }
                // this block's outlier activations: row c0 + lane, one 16-byte chunk per register (rows beyond M re-read
                // row M - 1); issued before the wait so that the loads fly with the tensor-memory load
                uint32_t bfr[4][2];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    bfr[j][0] = bnext[j][0];
                    bfr[j][1] = bnext[j][1];
                }
                if (side_mma) {
                    if (c0 + 32 < p.tile_x && m_base + c0 + 32 < p.M) load_bfr(m_base, c0 + 32, bnext);
                    else if (half + 1 < C::kHalves && m_base + p.tile_x < p.M) load_bfr(m_base + p.tile_x, 0, bnext);
                }
                uint4 xblk[kSideRegs];
                if (side_fast && !side_mma) {
                    const int64_t mr = m_base + c0 + lane;
                    const uint4* xr = reinterpret_cast<const uint4*>(xo + (mr < p.M ? mr : p.M - 1) * p.ldxo);
#pragma unroll
                    for (int ch = 0; ch < kSideRegs; ++ch)
                        xblk[ch] = ch < side_chunks ? __ldg(xr + ch) : make_uint4(0u, 0u, 0u, 0u);
                }
                tmem_ld_wait();
                // Rows of this block that exist; the per-row work below is free of control flow (stores are predicated,
                // flags are selects) so that the compiler interleaves the 32 independent rows -- with an early exit per
                // row every row was a basic block of its own and its chain of dependent conversions ran unhidden
                // (measured: a bias cost 6 % of the whole kernel, eight outlier columns 80 %).
                const int64_t rows_left = p.M - (m_base + c0);
                const int nrows = (int)(rows_left < 32 ? rows_left : 32) < p.tile_x - c0 ? (int)(rows_left < 32 ? rows_left : 32)
                                                                                       : p.tile_x - c0;
                // Two rows at a time in packed 16-bit arithmetic: one conversion rounds both accumulators, one packed
                // multiply applies the scale, one packed add each the outlier product and the bias -- every step rounded
                // to the activation type like the reference's chain of kernels -- then two 16-bit stores.  The epilogue
                // warps share the SM's issue slots with the converter warps, which pace the main loop: an instruction
                // saved per output row here is time given back to the next tile's main loop.
                uint16_t* yrow = reinterpret_cast<uint16_t*>(y + (m_base + c0) * p.ldy + n);
                const int64_t ystep = p.ldy;
                if (p.KO == 0) {
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        uint32_t v = Widen<A>::mul2(Widen<A>::pack2(__uint_as_float(r[c]), __uint_as_float(r[c + 1])), scale2);
                        v = has_bias ? Widen<A>::add2(v, bias2) : v;
                        if (n_ok && c < nrows) yrow[(int64_t)c * ystep] = (uint16_t)(v & 0xffffu);
                        if (n_ok && c + 1 < nrows) yrow[(int64_t)(c + 1) * ystep] = (uint16_t)(v >> 16);
                    }
                    continue;
                }
                if (side_mma) {
                    if constexpr (C::kSideMma) {
                        float* scratch = reinterpret_cast<float*>(gbase + C::side) + (warp - 2) * (32 * 33);
#pragma unroll
                        for (int i = 0; i < 2; ++i)
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                                mma16816<A>(d, afr[i], bfr[j][0], bfr[j][1]);
                                float* dst = scratch + (16 * i + g8) * 33 + 8 * j + 2 * t4;
                                dst[0] = d[0];
                                dst[1] = d[1];
                                dst[8 * 33] = d[2];
                                dst[8 * 33 + 1] = d[3];
                            }
                        __syncwarp();
                        const float* mine = scratch + lane * 33;
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {
                            uint32_t v = Widen<A>::mul2(Widen<A>::pack2(__uint_as_float(r[c]), __uint_as_float(r[c + 1])), scale2);
                            v = Widen<A>::add2(v, Widen<A>::pack2(mine[c], mine[c + 1]));
                            v = has_bias ? Widen<A>::add2(v, bias2) : v;
                            if (n_ok && c < nrows) yrow[(int64_t)c * ystep] = (uint16_t)(v & 0xffffu);
                            if (n_ok && c + 1 < nrows) yrow[(int64_t)(c + 1) * ystep] = (uint16_t)(v >> 16);
                        }
                        __syncwarp();  // the scratch is rewritten by the next block
                    }
                    continue;
                }
                if (side_fast) {
                    auto rows32 = [&](auto two_chunks) {
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {
                            float side[2];
#pragma unroll
                            for (int u = 0; u < 2; ++u) {
                                uint4 xv;
                                xv.x = __shfl_sync(0xffffffffu, xblk[0].x, c + u);
                                xv.y = __shfl_sync(0xffffffffu, xblk[0].y, c + u);
                                xv.z = __shfl_sync(0xffffffffu, xblk[0].z, c + u);
                                xv.w = __shfl_sync(0xffffffffu, xblk[0].w, c + u);
                                side[u] = dot8<A>(xv, wreg[0], 0.0f);
                                if constexpr (decltype(two_chunks)::value) {
                                    xv.x = __shfl_sync(0xffffffffu, xblk[1].x, c + u);
                                    xv.y = __shfl_sync(0xffffffffu, xblk[1].y, c + u);
                                    xv.z = __shfl_sync(0xffffffffu, xblk[1].z, c + u);
                                    xv.w = __shfl_sync(0xffffffffu, xblk[1].w, c + u);
                                    side[u] = dot8<A>(xv, wreg[1], side[u]);
                                }
                            }
                            uint32_t v = Widen<A>::mul2(Widen<A>::pack2(__uint_as_float(r[c]), __uint_as_float(r[c + 1])), scale2);
                            v = Widen<A>::add2(v, Widen<A>::pack2(side[0], side[1]));
                            v = has_bias ? Widen<A>::add2(v, bias2) : v;
                            if (n_ok && c < nrows) yrow[(int64_t)c * ystep] = (uint16_t)(v & 0xffffu);
                            if (n_ok && c + 1 < nrows) yrow[(int64_t)(c + 1) * ystep] = (uint16_t)(v >> 16);
                        }
                    };
                    if (side_chunks > 1) rows32(std::true_type{});
                    else rows32(std::false_type{});
                    continue;
                }
                // more outlier columns than the registers hold, or unaligned operands: loads in the loop, eight output
                // rows at a time so that eight of them are in flight
#pragma unroll
                for (int cb = 0; cb < 32; cb += 8) {
                    if (m_base + c0 + cb >= p.M || c0 + cb >= p.tile_x) break;  // uniform across the warp
                    float side[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) side[u] = 0.0f;
                    if (p.side_vec) {
                        for (int ch = 0; ch < side_chunks; ++ch) {
                            const uint4 wv = n_ok ? __ldg(wrow4 + ch) : make_uint4(0u, 0u, 0u, 0u);
                            uint4 xv[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const int64_t mr = m_base + c0 + cb + u;
                                xv[u] = __ldg(reinterpret_cast<const uint4*>(xo + (mr < p.M ? mr : p.M - 1) * p.ldxo) + ch);
                            }
#pragma unroll
                            for (int u = 0; u < 8; ++u) side[u] = dot8<A>(xv[u], wv, side[u]);
                        }
                    } else if (n_ok) {
                        const A* wrow = wo + n * p.KO;
                        for (int j = 0; j < (int)p.KO; ++j) {
                            const float wj = Widen<A>::to_float(__ldg(wrow + j));
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const int64_t mr = m_base + c0 + cb + u;
                                side[u] = fmaf(Widen<A>::to_float(__ldg(xo + (mr < p.M ? mr : p.M - 1) * p.ldxo + j)), wj, side[u]);
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int64_t m = m_base + c0 + cb + u;
                        if (m >= p.M || c0 + cb + u >= p.tile_x) break;  // uniform across the warp
                        float v = ref_round<A>(ref_round<A>(__uint_as_float(r[cb + u])) * scale);
                        v = ref_round<A>(v + ref_round<A>(side[u]));
                        if (has_bias) v = ref_round<A>(v + bias);
                        if (n_ok) y[m * p.ldy + n] = Widen<A>::from_float(v);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(tmem_empty + 8 * (acc + (uint32_t)half));
                if (C::kDual) mbar_arrive(tmem_empty + 8);
            }
            }  // half
        }
    } else if (warp < kW8Warp) {
        // ------------------------------ converters ------------------------------
        const int cw = warp - (2 + kEpiWarps);  // 0 .. 7
        uint32_t s_w = 0, ph_w = 0, s_a = 0, ph_a = 0;
        bool ok = true;
        WorkItem w;
        if constexpr (MODE != kSmemA) {
            for (int idx = 0; ok && work_item(p, num_kb, idx, w); ++idx) ok = convert_item_tmem(w, (uint32_t)(cw >> 2));
        } else
        for (int idx = 0; ok && work_item(p, num_kb, idx, w); ++idx) {
            for (int kb = w.kb0; kb < w.kb1; ++kb) {
                {
                    // lane 0 probes both barriers back to back, the warp shares the verdict
                    // one wait: the int8 tile has landed -- its producer waited for the stage to be free, so the
                    // widened tile of this stage may be overwritten too (a probe costs ~100 cycles even on a
                    // completed phase, and the converters' loop is as long as the MMA thread's)
                    int okw = 1;
                    if (lane == 0) {
                        okw = mbar_wait(full_w8 + 8 * s_w, ph_w, abort_flag) ? 1 : 0;
                    }
                    ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
                }
                if (!ok) break;
                tc_fence_after();
                const uint32_t src = sw8 + s_w * kBytesW8;
                if constexpr (MODE == kSmemA) {
                    const int cid = cw * 32 + lane;  // 0 .. 255
                    const uint32_t dst = sa + s_a * kBytesA;
#pragma unroll
                    for (int pass = 0; pass < (kTileN * kBlockK / 16) / (kConvWarps * 32); ++pass) {
                        const int id = pass * (kConvWarps * 32) + cid;  // 16-byte chunk of the int8 tile
                        const int row = id >> 2, j = id & 3;            // row of 64 codes, chunk j = k 16j .. 16j+15
                        uint32_t c0, c1, c2, c3;
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
                                     : "r"(src + (uint32_t)(row * 64 + j * 16)));
                        uint32_t o[8];
                        Widen<A>::four(c0, o[0], o[1]);
                        Widen<A>::four(c1, o[2], o[3]);
                        Widen<A>::four(c2, o[4], o[5]);
                        Widen<A>::four(c3, o[6], o[7]);
                        // 16-bit row = 128 bytes = eight 16-byte chunks; chunk c lives at c ^ (row % 8)
                        const uint32_t rbase = dst + (uint32_t)(row * 128);
                        const uint32_t sw = (uint32_t)(row & 7);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(rbase + (((uint32_t)(2 * j) ^ sw) << 4)),
                                     "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                                     : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(rbase + (((uint32_t)(2 * j + 1) ^ sw) << 4)),
                                     "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                                     : "memory");
                    }
                    fence_async_smem();  // generic-proxy stores -> visible to the tensor-core (async) proxy
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(full_a + 8 * s_a);
                if (++s_w == kStagesW8) { s_w = 0; ph_w ^= 1u; }
                if (++s_a == kStagesA) { s_a = 0; ph_a ^= 1u; }
            }
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
// host side
// ---------------------------------------------------------------------------------------------
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

bool make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* ptr, uint64_t inner, uint64_t outer,
                 uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// One error word per device (file-scope device memory, nothing is allocated), raised by a
// kernel whose bounded wait expired.
__device__ unsigned int g_tc_error_word = 0;

unsigned int* error_word() {
    static unsigned int* words[64] = {nullptr};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return nullptr;
    if (!words[dev]) {
        void* sym = nullptr;
        if (cudaGetSymbolAddress(&sym, g_tc_error_word) != cudaSuccess) return nullptr;
        words[dev] = static_cast<unsigned int*>(sym);
    }
    return words[dev];
}

}  // namespace

unsigned int* w8a16_tc_error_word() { return error_word(); }

bool w8a16_tc_supported(const W8A16Args& a) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (a.act_dtype != kBF16 && a.act_dtype != kF16) return false;
    if (a.K < 16 || a.K % 16 != 0) return false;       // TMA: int8 row stride must be a multiple of 16 bytes
    if ((a.ldx * 2) % 16 != 0) return false;           // TMA: activation row stride
    if (!al16(a.x) || !al16(a.wq)) return false;
    if (a.KO > kMaxKO) return false;
    if (a.M < 1 || a.N < 1) return false;
    return encode_fn() != nullptr;
}

// The persistent schedule of one call.
struct TcPlan {
    int mode;         // AMode
    int tile_x;       // activation rows per tile (multiple of 16, <= 256 / 208)
    int grid;         // CTAs
    int full_rounds;  // rounds of whole tiles on every CTA
    int rem_tiles;    // tiles of the last, partly filled round
    int splits;       // K-splits of each of those (1 = none)
    size_t partial_bytes;
    size_t workspace_bytes() const { return partial_bytes; }
};

constexpr int kMaxSplits = 32;
// Modelled time of a k-block of the two-tile mode relative to (rows + 512) of the one-tile shared-memory mode.
// Measured on B200 (N = 14336, K = 4096): a k-block of a 416-row item takes 0.79 us against 0.48 us for a 256-row
// tile -- the same time per row (a CTA-pair kernel that halves the activation bytes per SM is no faster, nor is a
// second MMA issuer: the kernel sits at the power cap with the tensor pipe 65 % busy) -- so the two-tile form wins
// exactly where its larger items fill the rounds better:
// M = 320 / 416 / 832 / 2048 / 4096 / 8192: 47 / 52 / 97 / 203 / 404 / 917 us against 53 / 56 / 105 / 223 / 428 / 955 us,
// and loses at M = 256 / 512 / 1024 (45 / 82 / 132 against 41 / 72 / 115 us).
constexpr double kTwoTileCostFactor = 1.28;
constexpr int kSplitOverheadKb = 24;  // slab stores + the second kernel, expressed in k-blocks (measured order of magnitude)

static TcPlan plan_for_tile(int mode, int tx, int64_t M, int64_t N, int64_t K, int sms, bool may_split, double* cost) {
    TcPlan pl{};
    const int halves = mode == kTmemA2 ? 2 : 1;  // activation tiles per work item
    const int64_t item_rows = (int64_t)tx * halves;
    const int64_t tiles = ((M + item_rows - 1) / item_rows) * ((N + kTileN - 1) / kTileN);
    const int num_kb = (int)((K + kBlockK - 1) / kBlockK);
    pl.mode = mode;
    pl.tile_x = tx;
    pl.full_rounds = (int)(tiles / sms);
    pl.rem_tiles = (int)(tiles % sms);
    pl.splits = 1;
    // Split only a schedule that has no full round: there the idle SMs are a plain loss.  Behind full
    // rounds the kernel is bound by what all SMs together pull out of L2, a thinly populated last round
    // runs fast, and splitting it measured no gain (M = 1024 .. 4096, N = 14336, K = 4096).
    if (may_split && halves == 1 && pl.full_rounds == 0 && pl.rem_tiles > 0) {
        int sp = sms / pl.rem_tiles;
        if (sp > kMaxSplits) sp = kMaxSplits;
        if (sp > num_kb / 2) sp = num_kb / 2;
        // Worth it only with at least four splits per tile and a split round (its k-blocks + the slab
        // traffic and the second kernel) clearly shorter than a whole tile; measured on B200: 32 tiles x 4
        // splits is 23 % ahead at M = 128 and break-even at M = 256, 64 tiles x 2 splits is 14 % behind.
        if (sp >= 4 && (num_kb + sp - 1) / sp + kSplitOverheadKb < (num_kb * 4) / 5) pl.splits = sp;
    }
    pl.grid = tiles >= sms || pl.splits > 1 ? sms : (int)tiles;
    if (pl.splits > 1) pl.partial_bytes = (size_t)pl.rem_tiles * pl.splits * tx * kTileN * sizeof(float);
    const double tail_kb = pl.rem_tiles == 0 ? 0.0
                           : pl.splits > 1   ? (double)((num_kb + pl.splits - 1) / pl.splits + kSplitOverheadKb)
                                             : (double)num_kb;
    // time ~ k-blocks on the busiest CTA * (rows of the work item + a fixed per-k-block cost expressed in rows);
    // measured: a k-block costs nearly the same for every tile height
    *cost = ((double)pl.full_rounds * num_kb + tail_kb) * (item_rows + 512);
    return pl;
}

// Operand-A mode and tile height (a multiple of 16 rows) with the shortest modelled schedule.
static TcPlan make_plan(int64_t M, int64_t N, int64_t K, int sms, bool may_split) {
    // M <= 128: one short tile per CTA, the deep-ring modes.  Above: shared-memory A (tiles up to 256 rows) against
    // tensor-memory A (up to 208 rows), whichever models shorter -- measured on B200 (N = 14336, K = 4096) the
    // tensor-memory route needs ~9 % less time per k-block and row (M = 416: 65 vs 71 us, M = 1024: 118 vs 134 us),
    // which its smaller tiles give back when they cost an extra round (M = 4096: 446 vs 430 us) -- and, from two
    // activation tiles' worth of rows, the two-tile form of the tensor-memory route (kTmemA2).
    int modes[3] = {kSmemA, kTmemA, kTmemA2};
    int n_modes = M > Cfg<kTmemA>::kMaxTileX ? 3 : 2;
    if (M <= Cfg<kTmemA64>::kMaxTileX) { modes[0] = kTmemA64; n_modes = 1; }
    else if (M <= Cfg<kTmemA128>::kMaxTileX) { modes[0] = kTmemA128; n_modes = 1; }
    TcPlan best{};
    double best_cost = 1e300;
    for (int i = 0; i < n_modes; ++i) {
        const int mode = modes[i];
        const int max_tx = mode == kSmemA ? Cfg<kSmemA>::kMaxTileX
                           : mode == kTmemA || mode == kTmemA2 ? Cfg<kTmemA>::kMaxTileX
                           : mode == kTmemA128 ? Cfg<kTmemA128>::kMaxTileX
                                               : Cfg<kTmemA64>::kMaxTileX;
        for (int tx = max_tx; tx >= 32; tx -= 16) {
            double cost;
            const TcPlan pl = plan_for_tile(mode, tx, M, N, K, sms, may_split, &cost);
            if (mode == kTmemA) cost *= 0.91;
            if (mode == kTmemA2) cost *= kTwoTileCostFactor;
            if (cost < best_cost - 1e-9) { best_cost = cost; best = pl; }
        }
    }
    return best;
}

size_t w8a16_tc_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M < 1 || N < 1 || K < 1) return 0;
    return make_plan(M, N, K, sm_count(), true).workspace_bytes();
}

template <typename A, int MODE>
static cudaError_t launch_variant(const CUtensorMap& map_x, const CUtensorMap& map_w, const CUtensorMap& map_pf,
                                  const TcParams& p, unsigned grid,
                                  cudaStream_t s) {
    using C = Cfg<MODE>;
    // the opt-in shared-memory size is a per-device function attribute
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(w8a16_tc_kernel<A, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   C::kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    return launch_dependent(w8a16_tc_kernel<A, MODE>, grid, kThreads, C::kSmemBytes, s, map_x, map_w, map_pf, p);
}

cudaError_t launch_w8a16_tc(const W8A16Args& a, cudaStream_t s) {
    const int sms = sm_count();
    TcParams p;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.scales = a.scales; p.scales_dtype = a.scales_dtype;
    p.bias = a.bias; p.bias_dtype = a.bias_dtype;
    p.xo = a.xo; p.wo = a.wo; p.KO = a.KO; p.ldxo = a.ldxo;
    p.weights_ready = a.weights_ready ? 1 : 0;
    p.side_vec = a.KO > 0 && a.KO % 8 == 0 && a.ldxo % 8 == 0 && (reinterpret_cast<uintptr_t>(a.xo) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(a.wo) & 15) == 0;
    p.y = a.y; p.ldy = a.ldy;
    TcPlan pl = make_plan(a.M, a.N, a.K, sms, true);
    const bool ws_ok = a.workspace && a.workspace_bytes >= pl.workspace_bytes() &&
                       (reinterpret_cast<uintptr_t>(a.workspace) & 15) == 0;
    if (pl.splits > 1 && !ws_ok) pl = make_plan(a.M, a.N, a.K, sms, false);  // no workspace: whole tiles only
    p.tile_x = pl.tile_x;
    p.full_rounds = pl.full_rounds; p.rem_tiles = pl.rem_tiles; p.splits = pl.splits;
    p.partial = pl.splits > 1 ? static_cast<float*>(a.workspace) : nullptr;
    const int64_t item_rows = (int64_t)p.tile_x * (pl.mode == kTmemA2 ? 2 : 1);
    p.tiles_x = (int)((a.M + item_rows - 1) / item_rows);
    p.tiles_n = (int)((a.N + kTileN - 1) / kTileN);
    p.error_flag = error_word();
    if (!p.error_flag) return cudaErrorUnknown;

    uint32_t x_box_rows = (uint32_t)p.tile_x, w_box_rows = kTileN;
    CUtensorMap map_x, map_w, map_pf;
    const CUtensorMapDataType xdt = a.act_dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!make_map_2d(&map_x, xdt, a.x, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.ldx * 2, kBlockK, x_box_rows,
                     CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorNotSupported;
    // the int8 tile is read by generic loads: plain rows for kSmemA, the 64-byte swizzle for kTmemA
    if (!make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.K, kBlockK,
                     w_box_rows, pl.mode == kSmemA ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_64B))
        return cudaErrorNotSupported;
    // the same tensor with a box of kPfBlocks k-blocks, for L2 prefetches only (nothing lands in shared memory)
    if (!make_map_2d(&map_pf, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.K,
                     a.K >= kPfBlocks * kBlockK ? kPfBlocks * kBlockK : kBlockK, kTileN, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorNotSupported;

    const unsigned grid = (unsigned)pl.grid;
    const bool bf16 = a.act_dtype == kBF16;
    cudaError_t e;
    if (pl.mode == kSmemA) e = bf16 ? launch_variant<__nv_bfloat16, kSmemA>(map_x, map_w, map_pf, p, grid, s)
                                    : launch_variant<__half, kSmemA>(map_x, map_w, map_pf, p, grid, s);
    else if (pl.mode == kTmemA) e = bf16 ? launch_variant<__nv_bfloat16, kTmemA>(map_x, map_w, map_pf, p, grid, s)
                                         : launch_variant<__half, kTmemA>(map_x, map_w, map_pf, p, grid, s);
    else if (pl.mode == kTmemA2) e = bf16 ? launch_variant<__nv_bfloat16, kTmemA2>(map_x, map_w, map_pf, p, grid, s)
                                          : launch_variant<__half, kTmemA2>(map_x, map_w, map_pf, p, grid, s);
    else if (pl.mode == kTmemA128) e = bf16 ? launch_variant<__nv_bfloat16, kTmemA128>(map_x, map_w, map_pf, p, grid, s)
                                            : launch_variant<__half, kTmemA128>(map_x, map_w, map_pf, p, grid, s);
    else e = bf16 ? launch_variant<__nv_bfloat16, kTmemA64>(map_x, map_w, map_pf, p, grid, s)
                  : launch_variant<__half, kTmemA64>(map_x, map_w, map_pf, p, grid, s);
    if (e != cudaSuccess || pl.splits <= 1) return e;
    const unsigned fix_grid = (unsigned)(pl.rem_tiles * ((pl.tile_x + 7) / 8));
    count_launches(1);  // the fix-up kernel, beyond the one launch the C entry point accounts for
    if (bf16) return launch_dependent(w8a16_tc_fixup_kernel<__nv_bfloat16>, fix_grid, 256, 0, s, p, pl.grid);
    return launch_dependent(w8a16_tc_fixup_kernel<__half>, fix_grid, 256, 0, s, p, pl.grid);
}

// 0 = no kernel of this library has hit a bounded-wait expiry on the current device
cudaError_t w8a16_tc_read_error(unsigned int* host_value, cudaStream_t s) {
    unsigned int* w = error_word();
    if (!w) return cudaErrorUnknown;
    cudaError_t e = cudaMemcpyAsync(host_value, w, sizeof(unsigned int), cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return e;
    return cudaStreamSynchronize(s);
}

}  // namespace cb

