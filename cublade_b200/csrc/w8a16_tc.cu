// W8A16 linear for tall activations: a tcgen05 / TMEM GEMM fed by TMA that widens int8 weight
// tiles to 16-bit floats in shared memory.
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
//   warps 6-13  converters: int8 tile (shared) -> registers -> 16-bit in the canonical K-major
//               128-byte-swizzled UMMA layout (shared), then fence.proxy.async + barrier arrive
//
// No TMA multicast, no clusters, no peer memory.  Every mbarrier wait is bounded: on expiry the
// kernel raises an error flag in global memory, every role leaves its loop, TMEM is released and
// the kernel returns.

#include "tc_common.cuh"

#include <cstdio>
#include <mutex>

namespace cb {

namespace {

using namespace tc;

constexpr int kTileN = 128;     // weight rows (output features) per tile = UMMA M
constexpr int kMaxTileX = 256;  // activation rows per tile = UMMA N (multiple of 16)
constexpr int kStagesX = 4;     // activation tiles in flight (32 KiB each at 256 rows)
constexpr int kStagesA = 3;     // converted weight tiles (16 KiB each)
constexpr int kStagesW8 = 4;    // int8 weight tiles (8 KiB each)
constexpr int kConvWarps = 8;
constexpr int kEpiWarps = 4;
constexpr int kThreads = (3 + kEpiWarps + kConvWarps) * 32;  // + TMA(x), MMA, TMA(w8)
constexpr int kW8Warp = 2 + kEpiWarps + kConvWarps;         // last warp: int8 weight producer
constexpr int kTmemCols = 512;

constexpr uint32_t kBytesX = kMaxTileX * kBlockK * 2;  // 32768
constexpr uint32_t kBytesA = kTileN * kBlockK * 2;     // 16384
constexpr uint32_t kBytesW8 = kTileN * kBlockK;        // 8192

struct SmemLayout {
    static constexpr uint32_t x = 0;
    static constexpr uint32_t a = x + kStagesX * kBytesX;
    static constexpr uint32_t w8 = a + kStagesA * kBytesA;
    static constexpr uint32_t bars = w8 + kStagesW8 * kBytesW8;
    // barriers: full_x[kStagesX], empty_x[kStagesX], full_w8, empty_w8, full_a, empty_a, tmem_full[2], tmem_empty[2]
    static constexpr uint32_t n_bars = 2 * kStagesX + 2 * kStagesW8 + 2 * kStagesA + 4;
    static constexpr uint32_t tmem_slot = bars + n_bars * 8;
    static constexpr uint32_t abort_flag = tmem_slot + 4;
    static constexpr uint32_t total = abort_flag + 4;
};
constexpr uint32_t kSmemBytes = SmemLayout::total + 1024;  // + slack to align the base to 1024 B

struct TcParams {
    int64_t M, N, K;
    const void* scales;
    int scales_dtype;
    const void* bias;
    int bias_dtype;
    const void* xo;  // [M, KO] 16-bit
    const void* wo;  // [N, KO] 16-bit
    int64_t KO, ldxo;
    void* y;
    int64_t ldy;
    int tile_x;      // activation rows per tile (multiple of 16, <= 256)
    int tiles_x;     // ceil(M / tile_x)
    int tiles_n;     // ceil(N / 128)
    unsigned int* error_flag;  // global; set to 1 when a bounded wait expired
};

constexpr int kMaxKO = 64;  // outlier columns handled by the epilogue's CUDA-core side product

template <typename A>
__global__ void __launch_bounds__(kThreads, 1)
w8a16_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte aligned base (the 128-byte swizzle pattern repeats every 1024 bytes)
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sx = base + SmemLayout::x, sa = base + SmemLayout::a, sw8 = base + SmemLayout::w8;
    const uint32_t bars = base + SmemLayout::bars;
    const uint32_t full_x = bars, empty_x = full_x + 8 * kStagesX;
    const uint32_t full_w8 = empty_x + 8 * kStagesX, empty_w8 = full_w8 + 8 * kStagesW8;
    const uint32_t full_a = empty_w8 + 8 * kStagesW8, empty_a = full_a + 8 * kStagesA;
    const uint32_t tmem_full = empty_a + 8 * kStagesA, tmem_empty = tmem_full + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + SmemLayout::tmem_slot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gbase + SmemLayout::abort_flag);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (int)((p.K + kBlockK - 1) / kBlockK);
    const int total_tiles = p.tiles_x * p.tiles_n;
    const uint32_t x_bytes = (uint32_t)p.tile_x * kBlockK * 2;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStagesX; ++i) { mbar_init(full_x + 8 * i, 1); mbar_init(empty_x + 8 * i, 1); }
        for (int i = 0; i < kStagesW8; ++i) { mbar_init(full_w8 + 8 * i, 1); mbar_init(empty_w8 + 8 * i, kConvWarps); }
        for (int i = 0; i < kStagesA; ++i) { mbar_init(full_a + 8 * i, kConvWarps); mbar_init(empty_a + 8 * i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(tmem_full + 8 * i, 1); mbar_init(tmem_empty + 8 * i, kEpiWarps); }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&map_x);
        prefetch_tmap(&map_w);
    }
    if (warp == 1) tmem_alloc(base + SmemLayout::tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer, activations ------------------------------
        // The two producers are separate warps: probing a barrier costs ~130 cycles even when its
        // phase is complete and issuing a TMA ~100, so one thread feeding both rings cannot stay
        // ahead of the tensor core.
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int row_x = (t % p.tiles_x) * p.tile_x;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(empty_x + 8 * s, ph ^ 1u, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(full_x + 8 * s, x_bytes);
                    tma_load_2d(sx + s * kBytesX, &map_x, kb * kBlockK, row_x, full_x + 8 * s);
                    if (++s == kStagesX) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == kW8Warp) {
        // ------------------------------ TMA producer, int8 weights ------------------------------
        if (lane == 0) {
            constexpr int kAhead = 12;  // k-blocks of weights requested into L2 ahead of their TMA load
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int row_w = (t / p.tiles_x) * kTileN;
                const int row_w_next = ((t + (int)gridDim.x) / p.tiles_x) * kTileN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (kb + kAhead < num_kb) tma_prefetch_l2_2d(&map_w, (kb + kAhead) * kBlockK, row_w);
                    else if (t + (int)gridDim.x < total_tiles)
                        tma_prefetch_l2_2d(&map_w, (kb + kAhead - num_kb) * kBlockK, row_w_next);
                    ok = mbar_wait(empty_w8 + 8 * s, ph ^ 1u, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(full_w8 + 8 * s, kBytesW8);
                    tma_load_2d(sw8 + s * kBytesW8, &map_w, kb * kBlockK, row_w, full_w8 + 8 * s);
                    if (++s == kStagesW8) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(Widen<A>::kBf16, (uint32_t)p.tile_x);
            // Ring positions are kept incrementally (no divisions) and the barriers of the NEXT
            // k-block are probed before the MMAs of the current one are issued, so a probe's
            // latency overlaps the issue; this thread's loop is the critical path of the kernel.
            uint32_t s_a = 0, ph_a = 0, s_x = 0, ph_x = 0, it = 0;
            bool ok = true, pre = false;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++it) {
                const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
                ok = mbar_wait(tmem_empty + 8 * acc, acc_ph ^ 1u, abort_flag);  // epilogue drained this accumulator
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kMaxTileX;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!pre) {
                        const bool r0 = mbar_try(full_a + 8 * s_a, ph_a), r1 = mbar_try(full_x + 8 * s_x, ph_x);
                        ok = (r0 || mbar_wait(full_a + 8 * s_a, ph_a, abort_flag)) &&
                             (r1 || mbar_wait(full_x + 8 * s_x, ph_x, abort_flag));
                        if (!ok) break;
                    }
                    tc_fence_after();
                    uint32_t ns_a = s_a + 1, nph_a = ph_a, ns_x = s_x + 1, nph_x = ph_x;
                    if (ns_a == kStagesA) { ns_a = 0; nph_a ^= 1u; }
                    if (ns_x == kStagesX) { ns_x = 0; nph_x ^= 1u; }
                    const bool n0 = mbar_try(full_a + 8 * ns_a, nph_a), n1 = mbar_try(full_x + 8 * ns_x, nph_x);
                    const uint64_t adesc = make_kmajor_sw128_desc(sa + s_a * kBytesA);
                    const uint64_t bdesc = make_kmajor_sw128_desc(sx + s_x * kBytesX);
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        // +32 bytes per 16-element k step: +2 in the (>>4) start-address field
                        umma_f16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                                 (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_a + 8 * s_a);  // both operand slots are free once these MMAs retire
                    umma_commit(empty_x + 8 * s_x);
                    pre = n0 && n1;
                    s_a = ns_a; ph_a = nph_a; s_x = ns_x; ph_x = nph_x;
                }
                if (!ok) break;
                umma_commit(tmem_full + 8 * acc);  // accumulator complete -> epilogue
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ------------------------------ epilogue ------------------------------
        const int quarter = warp & 3;  // a warp may only touch TMEM lanes 32*(warp%4) .. +31
        const A* xo = static_cast<const A*>(p.xo);
        const A* wo = static_cast<const A*>(p.wo);
        A* y = static_cast<A*>(p.y);
        uint32_t it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++it) {
            const int tx = t % p.tiles_x, tn = t / p.tiles_x;
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            const int64_t n = (int64_t)tn * kTileN + quarter * 32 + lane;
            const bool n_ok = n < p.N;
            const float scale = n_ok ? load_scalar(p.scales, p.scales_dtype, n) : 0.0f;
            const float bias = (n_ok && p.bias) ? load_scalar(p.bias, p.bias_dtype, n) : 0.0f;
            {
                int okw = 1;
                if (lane == 0) okw = mbar_wait(tmem_full + 8 * acc, acc_ph, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
            }
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
                    float v = __uint_as_float(r[c]) * scale;
                    if (p.KO > 0 && n_ok) {
                        // side product over the outlier columns: the activation row is the same address
                        // in every lane (broadcast load), the weight row is this lane's own
                        const A* xrow = xo + m * p.ldxo;
                        const A* wrow = wo + n * p.KO;
                        for (int j = 0; j < (int)p.KO; ++j)
                            v = fmaf(Widen<A>::to_float(__ldg(xrow + j)), Widen<A>::to_float(__ldg(wrow + j)), v);
                    }
                    v += bias;
                    if (n_ok) y[m * p.ldy + n] = Widen<A>::from_float(v);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty + 8 * acc);
        }
    } else if (warp < kW8Warp) {
        // ------------------------------ converters ------------------------------
        const int cid = (warp - (2 + kEpiWarps)) * 32 + lane;  // 0 .. 255
        uint32_t s_w = 0, ph_w = 0, s_a = 0, ph_a = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
            for (int kb = 0; kb < num_kb; ++kb) {
                {
                    // lane 0 probes both barriers back to back, the warp shares the verdict
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
                const uint32_t src = sw8 + s_w * kBytesW8, dst = sa + s_a * kBytesA;
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
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(full_a + 8 * s_a);
                    mbar_arrive(empty_w8 + 8 * s_w);
                }
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

// Activation rows per tile: the multiple of 16 (<= 256) that wastes the fewest SM-slots over the
// persistent schedule of ceil(M / tile) * ceil(N / 128) tiles on `sms` CTAs.
static int pick_tile_x(int64_t M, int64_t N, int sms) {
    const int64_t tiles_n = (N + kTileN - 1) / kTileN;
    int best = 256;
    double best_cost = 1e30;
    for (int tx = 256; tx >= 32; tx -= 16) {
        const int64_t tiles = ((M + tx - 1) / tx) * tiles_n;
        const int64_t waves = (tiles + sms - 1) / sms;
        // time ~ waves * (tile_x + fixed per-tile overhead expressed in rows)
        const double cost = (double)waves * (tx + 512);  // measured: a k-block costs nearly the same for every tile height
        if (cost < best_cost - 1e-9) { best_cost = cost; best = tx; }
    }
    return best;
}

cudaError_t launch_w8a16_tc(const W8A16Args& a, cudaStream_t s) {
    const int sms = sm_count();
    TcParams p;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.scales = a.scales; p.scales_dtype = a.scales_dtype;
    p.bias = a.bias; p.bias_dtype = a.bias_dtype;
    p.xo = a.xo; p.wo = a.wo; p.KO = a.KO; p.ldxo = a.ldxo;
    p.y = a.y; p.ldy = a.ldy;
    p.tile_x = pick_tile_x(a.M, a.N, sms);
    p.tiles_x = (int)((a.M + p.tile_x - 1) / p.tile_x);
    p.tiles_n = (int)((a.N + kTileN - 1) / kTileN);
    p.error_flag = error_word();
    if (!p.error_flag) return cudaErrorUnknown;

    CUtensorMap map_x, map_w;
    const CUtensorMapDataType xdt = a.act_dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!make_map_2d(&map_x, xdt, a.x, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.ldx * 2, kBlockK, (uint32_t)p.tile_x,
                     CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorNotSupported;
    if (!make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.K, kBlockK,
                     kTileN, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorNotSupported;

    const int64_t tiles = (int64_t)p.tiles_x * p.tiles_n;
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    // the opt-in shared-memory size is a per-device function attribute
    static bool attr_done[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int which = a.act_dtype == kBF16 ? 0 : 1;
    if (dev >= 0 && dev < 64 && !attr_done[dev][which]) {
        cudaError_t e = which == 0
            ? cudaFuncSetAttribute(w8a16_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes)
            : cudaFuncSetAttribute(w8a16_tc_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev][which] = true;
    }
    if (which == 0) w8a16_tc_kernel<__nv_bfloat16><<<grid, kThreads, kSmemBytes, s>>>(map_x, map_w, p);
    else w8a16_tc_kernel<__half><<<grid, kThreads, kSmemBytes, s>>>(map_x, map_w, p);
    return cudaPeekAtLastError();
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
