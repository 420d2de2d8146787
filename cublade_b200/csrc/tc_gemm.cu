// Dense GEMM  C[M, N] = A[M, K] . B[K, N]  for fp16 / bf16 (fp32 accumulate) and int8 / uint8 (int32
// accumulate) on tcgen05 / TMEM, fed by TMA.
//
// Replaces the reference's multi-precision WMMA kernel (cublade/kernels/cuda/wmma.cu:29-182: 16x16x16
// wmma fragments, cp.async double buffering; entry point wmma_gemm at :184-262, binding
// cublade/bindings/cuda/wmma.py:16-47).  Same contract: row-major A [M, K] and B [K, N] of one dtype, C
// row-major in the accumulator type (fp32, or int32 for the 8-bit inputs; fp16 output for fp16 inputs is
// the fp32 accumulator rounded once at the end).
//
// Structure: the skeleton of the W8A8 kernel (w8a8_tc.cu).  tcgen05 wants both operands K-major here, so
// B is first transposed into Bt [N, K] (a tiled shared-memory transpose into the caller's workspace);
// then Bt tiles are UMMA operand A (M = 128 rows of Bt = columns of C = tensor-memory lanes) and A tiles
// are operand B (N <= 256 rows of A = accumulator columns): for a fixed row m of C the 32 lanes of an
// epilogue warp store 32 consecutive n, one full 128-byte line for fp32 / int32.
// One operand ring of 4 x 48 KiB stages (128 bytes of k per row and stage), two accumulators in tensor
// memory.  No TMA multicast, no clusters; every mbarrier wait is bounded (error flag, clean return).
#include "tc_common.cuh"

#include <mutex>

namespace cb {

unsigned int* w8a16_tc_error_word();

namespace {

using namespace tc;

constexpr int kTileN = 128;       // columns of C per tile = UMMA M
constexpr int kMaxTileX = 256;    // rows of C per tile = UMMA N
constexpr int kRowBytes = 128;    // bytes of k per row and stage (one swizzle row)
constexpr int kStages = 4;
constexpr int kEpiWarps = 8;  // two per tensor-memory lane quarter, each draining every other 32-column chunk
constexpr int kThreads = (3 + kEpiWarps) * 32;
constexpr int kWWarp = 2 + kEpiWarps;
constexpr int kTmemCols = 512;
constexpr uint32_t kBytesX = kMaxTileX * kRowBytes;
constexpr uint32_t kBytesW = kTileN * kRowBytes;

struct Smem {
    static constexpr uint32_t x = 0;
    static constexpr uint32_t w = x + kStages * kBytesX;
    static constexpr uint32_t bars = w + kStages * kBytesW;
    static constexpr uint32_t n_bars = 2 * kStages + 4;
    static constexpr uint32_t tmem_slot = bars + n_bars * 8;
    static constexpr uint32_t abort_flag = tmem_slot + 4;
    static constexpr uint32_t total = abort_flag + 4;
};
constexpr uint32_t kSmemBytes = Smem::total + 1024;

enum InKind : int { kInF16 = 0, kInBF16 = 1, kInS8 = 2, kInU8 = 3 };
enum OutKind : int { kOutF32 = 0, kOutF16 = 1, kOutS32 = 2, kOutBF16 = 3 };

struct Params {
    int64_t M, N, K;
    void* c;
    int64_t ldc;
    int in_kind, out_kind;
    int leaky_relu;  // 1: float accumulators pass through x >= 0 ? x : 0.01 x before they are stored
    int tile_x, tiles_x, tiles_n;
    int elems_per_stage;  // k elements per stage = 128 / sizeof(element)
    unsigned int* error_flag;
};

__device__ __forceinline__ uint32_t idesc_for(int in_kind, uint32_t n) {
    if (in_kind == kInF16 || in_kind == kInBF16) return make_idesc(in_kind == kInBF16, n);
    const uint32_t fmt = in_kind == kInS8 ? 1u : 0u;  // kind::i8: 0 = unsigned, 1 = signed 8-bit
    return (2u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((uint32_t)(kUmmaM >> 4) << 24);
}

__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
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
    const int num_kb = (int)((p.K + p.elems_per_stage - 1) / p.elems_per_stage);
    const int total_tiles = p.tiles_x * p.tiles_n;
    const uint32_t x_bytes = (uint32_t)p.tile_x * kRowBytes;

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
                    ok = mbar_wait(empty + 8 * s, ph ^ 1u, abort_flag);
                    if (!ok) break;
                    if (is_x) {
                        mbar_expect_tx(full + 8 * s, x_bytes);
                        tma_load_2d(sx + s * kBytesX, &map_x, kb * p.elems_per_stage, row, full + 8 * s);
                    } else {
                        mbar_expect_tx(full + 8 * s, kBytesW);
                        tma_load_2d(sw + s * kBytesW, &map_w, kb * p.elems_per_stage, row, full + 8 * s);
                    }
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const uint32_t idesc = idesc_for(p.in_kind, (uint32_t)p.tile_x);
            const bool integer = p.in_kind >= kInS8;
            uint32_t s = 0, ph = 0, it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++it) {
                const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
                ok = mbar_wait(tmem_empty + 8 * acc, acc_ph ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kMaxTileX;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(full + 8 * s, ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t adesc = make_kmajor_sw128_desc(sw + s * kBytesW);
                    const uint64_t bdesc = make_kmajor_sw128_desc(sx + s * kBytesX);
#pragma unroll
                    for (int k = 0; k < kRowBytes / 32; ++k) {
                        // one instruction consumes 32 bytes of k per row (16 16-bit or 32 8-bit elements)
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        if (integer) umma_i8(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, accumulate);
                        else umma_f16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, accumulate);
                    }
                    umma_commit(empty + 8 * s);
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                umma_commit(tmem_full + 8 * acc);
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ------------------------------ epilogue ------------------------------
        const int quarter = warp & 3;
        uint32_t it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++it) {
            const int tx = t % p.tiles_x, tn = t / p.tiles_x;
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            const int64_t n = (int64_t)tn * kTileN + quarter * 32 + lane;
            const bool n_ok = n < p.N;
            {
                int okw = 1;
                if (lane == 0) okw = mbar_wait(tmem_full + 8 * acc, acc_ph, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
            }
            if (!ok) break;
            tc_fence_after();
            // This warp takes every other chunk of 32 rows of C; the tcgen05.ld of its next chunk is in flight while
            // the current one is stored (a load takes a few thousand cycles while the MMAs of the next tile run).
            const int64_t m_base = (int64_t)tx * p.tile_x;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kMaxTileX;
            const int nchunks = (p.tile_x + 31) / 32, parts = kEpiWarps / 4;
            auto store_chunk = [&](const uint32_t (&r)[32], int ch) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int64_t m = m_base + ch * 32 + c;
                    if (m >= p.M || ch * 32 + c >= p.tile_x) break;  // uniform across the warp
                    if (!n_ok) continue;
                    // fp32 and int32 accumulators are stored as they are (the same 32 bits)
                    uint32_t bits = r[c];
                    if (p.leaky_relu) {
                        const float f = __uint_as_float(bits);
                        bits = __float_as_uint(f >= 0.0f ? f : 0.01f * f);
                    }
                    if (p.out_kind == kOutF16) static_cast<__half*>(p.c)[m * p.ldc + n] = __float2half_rn(__uint_as_float(bits));
                    else if (p.out_kind == kOutBF16) static_cast<__nv_bfloat16*>(p.c)[m * p.ldc + n] = __float2bfloat16_rn(__uint_as_float(bits));
                    else static_cast<uint32_t*>(p.c)[m * p.ldc + n] = bits;
                }
            };
            uint32_t ra[32], rb[32];
            int ch = (warp - 2) >> 2;
            if (ch < nchunks) tmem_ld32(taddr + (uint32_t)(ch * 32), ra);
            while (ch < nchunks) {
                tmem_ld_wait();
                int nx = ch + parts;
                if (nx < nchunks) tmem_ld32(taddr + (uint32_t)(nx * 32), rb);
                store_chunk(ra, ch);
                ch = nx;
                if (ch >= nchunks) break;
                tmem_ld_wait();
                nx = ch + parts;
                if (nx < nchunks) tmem_ld32(taddr + (uint32_t)(nx * 32), ra);
                store_chunk(rb, ch);
                ch = nx;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty + 8 * acc);
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag) {
        atomicExch(p.error_flag, 1u);
        __nanosleep(200000);
    }
}

// Bt[n, k] = B[k, n]; 32 x 32 tiles through shared memory (padded against bank conflicts)
template <typename E>
__global__ void __launch_bounds__(256) transpose_kernel(const E* __restrict__ b, int64_t K, int64_t N, E* __restrict__ bt) {
    __shared__ E tile[32][33];
    const int64_t k0 = (int64_t)blockIdx.y * 32, n0 = (int64_t)blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        const int64_t k = k0 + ty + j, n = n0 + tx;
        if (k < K && n < N) tile[ty + j][tx] = b[k * N + n];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        const int64_t n = n0 + ty + j, k = k0 + tx;
        if (n < N && k < K) bt[n * K + k] = tile[tx][ty + j];
    }
}

// any shape / alignment: one thread per element of C, B read in place
template <typename E, typename Acc>
__device__ __forceinline__ Acc widen_in(E v);
template <> __device__ __forceinline__ float widen_in<__half, float>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float widen_in<__nv_bfloat16, float>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ int widen_in<int8_t, int>(int8_t v) { return (int)v; }
template <> __device__ __forceinline__ int widen_in<uint8_t, int>(uint8_t v) { return (int)v; }

template <typename E, typename Acc>
__global__ void __launch_bounds__(256) gemm_simple_kernel(const E* __restrict__ a, const E* __restrict__ b, int64_t M,
                                                          int64_t N, int64_t K, void* __restrict__ c, int64_t ldc,
                                                          int out_kind, int leaky_relu) {
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= M * N) return;
    const int64_t m = idx / N, n = idx - m * N;
    Acc acc = 0;
    for (int64_t k = 0; k < K; ++k) acc += widen_in<E, Acc>(a[m * K + k]) * widen_in<E, Acc>(b[k * N + n]);
    if (leaky_relu && acc < (Acc)0) acc = (Acc)(0.01f * (float)acc);  // float accumulators only (the entry point checks)
    if (out_kind == kOutF16) static_cast<__half*>(c)[m * ldc + n] = __float2half_rn((float)acc);
    else if (out_kind == kOutBF16) static_cast<__nv_bfloat16*>(c)[m * ldc + n] = __float2bfloat16_rn((float)acc);
    else static_cast<Acc*>(c)[m * ldc + n] = acc;
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

bool make_map(CUtensorMap* map, CUtensorMapDataType dt, int elem, const void* ptr, uint64_t inner, uint64_t outer,
              uint32_t box_outer) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * (uint64_t)elem};
    cuuint32_t box[2] = {(cuuint32_t)(kRowBytes / elem), box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

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

}  // namespace

size_t tc_gemm_workspace_bytes(int64_t N, int64_t K, int in_kind) {
    const size_t elem = in_kind <= kInBF16 ? 2 : 1;
    return ((size_t)N * (size_t)K * elem + 255) & ~(size_t)255;  // the transposed copy of B
}

cudaError_t launch_tc_gemm(const void* a, const void* b, int64_t M, int64_t N, int64_t K, int in_kind, void* c,
                           int64_t ldc, int out_kind, void* workspace, size_t workspace_bytes, cudaStream_t s, int leaky_relu) {
    const int elem = in_kind <= kInBF16 ? 2 : 1;
    auto al16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    const bool tc_ok = (K * elem) % 16 == 0 && K * elem >= 16 && al16(a) && workspace && al16(workspace) &&
                       workspace_bytes >= tc_gemm_workspace_bytes(N, K, in_kind) && encode_fn() != nullptr;
    if (!tc_ok) {
        const unsigned grid = (unsigned)((M * N + 255) / 256);
        switch (in_kind) {
            case kInF16: gemm_simple_kernel<__half, float><<<grid, 256, 0, s>>>(static_cast<const __half*>(a), static_cast<const __half*>(b), M, N, K, c, ldc, out_kind, leaky_relu); break;
            case kInBF16: gemm_simple_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), M, N, K, c, ldc, out_kind, leaky_relu); break;
            case kInS8: gemm_simple_kernel<int8_t, int><<<grid, 256, 0, s>>>(static_cast<const int8_t*>(a), static_cast<const int8_t*>(b), M, N, K, c, ldc, out_kind, leaky_relu); break;
            default: gemm_simple_kernel<uint8_t, int><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(b), M, N, K, c, ldc, out_kind, leaky_relu); break;
        }
        return cudaPeekAtLastError();
    }
    // 1. Bt = B^T into the workspace
    const dim3 tgrid((unsigned)((N + 31) / 32), (unsigned)((K + 31) / 32));
    if (elem == 2) transpose_kernel<uint16_t><<<tgrid, 256, 0, s>>>(static_cast<const uint16_t*>(b), K, N, static_cast<uint16_t*>(workspace));
    else transpose_kernel<uint8_t><<<tgrid, 256, 0, s>>>(static_cast<const uint8_t*>(b), K, N, static_cast<uint8_t*>(workspace));
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return e;
    // 2. the GEMM
    const int sms = sm_count();
    Params p;
    p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc; p.in_kind = in_kind; p.out_kind = out_kind; p.leaky_relu = leaky_relu;
    p.tile_x = pick_tile_x(M, N, sms);
    p.tiles_x = (int)((M + p.tile_x - 1) / p.tile_x);
    p.tiles_n = (int)((N + kTileN - 1) / kTileN);
    p.elems_per_stage = kRowBytes / elem;
    p.error_flag = w8a16_tc_error_word();
    if (!p.error_flag) return cudaErrorUnknown;
    const CUtensorMapDataType dt = in_kind == kInF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                   : in_kind == kInBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, dt, elem, a, (uint64_t)K, (uint64_t)M, (uint32_t)p.tile_x)) return cudaErrorNotSupported;
    if (!make_map(&map_w, dt, elem, workspace, (uint64_t)K, (uint64_t)N, kTileN)) return cudaErrorNotSupported;
    const int64_t tiles = (int64_t)p.tiles_x * p.tiles_n;
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        e = cudaFuncSetAttribute(tc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    tc_gemm_kernel<<<grid, kThreads, kSmemBytes, s>>>(map_x, map_w, p);
    return cudaPeekAtLastError();
}

}  // namespace cb
