// Memory-bound quantize / dequantize kernels for sm_100a.
//
// Replaces, kernel for kernel, the reference's SIMT kernels in
// cublade/kernels/cuda/quantization/{quantize_per_tensor_fp8,dequantize_per_tensor_fp8,
// quantize_int8,dequantize_int8}.cu, with these structural differences:
//   * per-channel / per-group quantization is ONE pass: a team of threads
//     (4..32 lanes of a warp, or a whole CTA) keeps its row / group in
//     registers between the amax reduction and the cast, so x is read from
//     HBM once (3 B per element instead of 5);
//   * per-tensor quantization stays two-phase (amax, then cast) because the
//     amax is global, but both phases are persistent grid-stride kernels with
//     four 128-bit loads in flight per thread and one integer atomicMax per
//     CTA (valid on the bit pattern of a non-negative float);
//   * dequantization is one flat kernel for all three granularities: the
//     scale index is pack_index / packs_per_segment.
// All products are single fp32 multiplies and all divisions IEEE (pack.cuh).

#include "launch.h"
#include "pack.cuh"

namespace cb {

constexpr int kBlock = 256;

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// CTA-wide max; result valid in every thread.  `red` holds kBlock/32 floats.
__device__ __forceinline__ float block_max(float v, float* red) {
    v = team_max<32>(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.0f;
    r = team_max<8>(r);  // blockDim.x <= 256 -> at most 8 warps
    r = __shfl_sync(0xffffffffu, r, 0);
    __syncthreads();
    return r;
}

// ===========================================================================
// Per-tensor phase 1: amax.   (reference: quantize_per_tensor_fp8.cu:38-86,
// quantize_int8.cu:47-101)
// A CTA iteration covers one contiguous chunk of kBlock*4 packs (16 KiB).
// ===========================================================================
template <typename T, bool PARTIALS>
__global__ void __launch_bounds__(kBlock) amax_tensor_kernel(const T* __restrict__ x, int64_t n,
                                                             float* __restrict__ amax) {
    constexpr int E = DTypeTraits<T>::kLanes;
    constexpr int kChunkPacks = kBlock * 4;
    // Launched with a programmatic edge: this CTA may be resident before the kernel ahead of it in the stream (which
    // may have produced x) has finished, so it waits for that kernel first; the cast kernel behind it may then be
    // set up in turn and takes this CTA's place as soon as it leaves.
    pdl_wait();
    pdl_trigger();
    const int64_t npk = n / E;
    const int64_t nchunks = (npk + kChunkPacks - 1) / kChunkPacks;
    const uint4* xp = reinterpret_cast<const uint4*>(x);
    AbsMax<T> am;
    for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const int64_t p0 = c * kChunkPacks + threadIdx.x;
        if (p0 + 3 * kBlock < npk) {
            uint4 v0 = ld_keep16(xp + p0);
            uint4 v1 = ld_keep16(xp + p0 + kBlock);
            uint4 v2 = ld_keep16(xp + p0 + 2 * kBlock);
            uint4 v3 = ld_keep16(xp + p0 + 3 * kBlock);
            am.update(v0);
            am.update(v1);
            am.update(v2);
            am.update(v3);
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int64_t p = p0 + k * kBlock;
                if (p < npk) am.update(ld_keep16(xp + p));
            }
        }
    }
    // ragged tail (< one pack), CTA 0
    if (blockIdx.x == 0) {
        const int64_t t = npk * E + threadIdx.x;
        if (t < n) am.update1(DTypeTraits<T>::to_float(x[t]));
    }
    __shared__ float red[kBlock / 32];
    float m = block_max(am.finish(), red);
    if (threadIdx.x == 0) {
        // PARTIALS: one slot per CTA, no atomics and nothing to pre-zero (the cast kernel folds the
        // slots); otherwise an integer atomicMax on the bit pattern of a non-negative float.
        if constexpr (PARTIALS) amax[blockIdx.x] = m;
        else atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(m));
    }
}

// any alignment
template <typename T, bool PARTIALS>
__global__ void __launch_bounds__(kBlock) amax_tensor_scalar_kernel(const T* __restrict__ x, int64_t n,
                                                                    float* __restrict__ amax) {
    pdl_wait();
    pdl_trigger();
    float m = 0.0f;
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (int64_t)gridDim.x * kBlock)
        m = fmaxf(m, fabsf(DTypeTraits<T>::to_float(x[i])));
    __shared__ float red[kBlock / 32];
    m = block_max(m, red);
    if (threadIdx.x == 0) {
        if constexpr (PARTIALS) amax[blockIdx.x] = m;
        else atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(m));
    }
}

// amax for the cast kernels: amax[0] when nparts == 0, else the max over nparts per-CTA partials
__device__ __forceinline__ float fold_amax(const float* __restrict__ amax, int nparts, float* red) {
    if (nparts <= 0) return __ldg(amax);
    float m = 0.0f;
    for (int i = threadIdx.x; i < nparts; i += blockDim.x) m = fmaxf(m, __ldg(amax + i));
    return block_max(m, red);
}

// ===========================================================================
// Per-tensor phase 2: cast.  (reference: quantize_per_tensor_fp8.cu:88-132,
// quantize_int8.cu:103-166)
// ===========================================================================
template <typename T, typename Code>
__global__ void __launch_bounds__(kBlock) cast_tensor_kernel(const T* __restrict__ x, int64_t n,
                                                             const float* __restrict__ amax, int nparts, float eps,
                                                             uint8_t* __restrict__ q, float* __restrict__ scale_out) {
    constexpr int E = DTypeTraits<T>::kLanes;
    constexpr int kChunkPacks = kBlock * 4;
    __shared__ float red_amax[kBlock / 32];
    const int64_t npk = n / E;
    const int64_t nchunks = (npk + kChunkPacks - 1) / kChunkPacks;
    const uint4* xp = reinterpret_cast<const uint4*>(x);
    // The first chunk's loads are issued BEFORE the wait on the amax kernel: x is an input nobody writes,
    // so under a programmatic launch edge they overlap that kernel's tail; the amax itself is read after.
    uint4 v[4];
    bool ok[4];
    int64_t c = blockIdx.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int64_t p = c * kChunkPacks + threadIdx.x + k * kBlock;
        ok[k] = c < nchunks && p < npk;
        if (ok[k]) v[k] = ld_stream16(xp + p);
    }
    pdl_wait();
    pdl_trigger();  // a dequantize kernel behind this one may start its prologue
    const InvScale is = inv_and_scale<Code>(fold_amax(amax, nparts, red_amax), eps);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = is.scale;
    while (c < nchunks) {
        const int64_t p0 = c * kChunkPacks + threadIdx.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (!ok[k]) continue;
            const int64_t p = p0 + k * kBlock;
            const uint2 codes = pack_encode<T, Code>(v[k], is.inv);
            if constexpr (E == 8) st_stream8(q + p * 8, codes);
            else st_stream4(q + p * 4, codes.x);
        }
        c += gridDim.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t p = c * kChunkPacks + threadIdx.x + k * kBlock;
            ok[k] = c < nchunks && p < npk;
            if (ok[k]) v[k] = ld_stream16(xp + p);
        }
    }
    if (blockIdx.x == 0) {
        const int64_t t = npk * E + threadIdx.x;
        if (t < n) q[t] = Code::encode1(__fmul_rn(DTypeTraits<T>::to_float(x[t]), is.inv));
    }
}

template <typename T, typename Code>
__global__ void __launch_bounds__(kBlock) cast_tensor_scalar_kernel(const T* __restrict__ x, int64_t n,
                                                                    const float* __restrict__ amax, int nparts,
                                                                    float eps, uint8_t* __restrict__ q,
                                                                    float* __restrict__ scale_out) {
    __shared__ float red_amax[kBlock / 32];
    pdl_wait();
    pdl_trigger();
    const InvScale is = inv_and_scale<Code>(fold_amax(amax, nparts, red_amax), eps);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = is.scale;
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (int64_t)gridDim.x * kBlock)
        q[i] = Code::encode1(__fmul_rn(DTypeTraits<T>::to_float(x[i]), is.inv));
}

// ===========================================================================
// Per-segment one-pass quantize (channels = rows of [C,F]; groups = rows of
// [num_groups, G]).  A TEAM of threads owns one segment; thread t holds packs
// t, t+TEAM, ... (PACKS of them) in registers across the amax reduction.
// Needs L % lanes == 0 and 16-byte aligned x, L*PACKS... checked by the launcher.
// (reference: quantize_int8.cu:173-297 per-channel, :307-371 per-group)
// ===========================================================================
template <typename T, typename Code, int TEAM, int PACKS, int BLOCK>
__global__ void __launch_bounds__(BLOCK) quant_segments_kernel(const T* __restrict__ x, int64_t nseg, int npk,
                                                                float eps, uint8_t* __restrict__ q,
                                                                float* __restrict__ scale_out) {
    constexpr int E = DTypeTraits<T>::kLanes;
    constexpr int kTeamsPerCta = BLOCK / TEAM;
    pdl_trigger();  // a dequantize kernel queued behind this one may be set up while the last CTAs run
    const int t = threadIdx.x % TEAM;
    const int64_t seg = (int64_t)blockIdx.x * kTeamsPerCta + threadIdx.x / TEAM;
    const bool live = seg < nseg;
    const uint4* xp = reinterpret_cast<const uint4*>(x) + seg * (int64_t)npk;

    uint4 v[PACKS];
#pragma unroll
    for (int k = 0; k < PACKS; ++k) {
        const int p = t + k * TEAM;
        if (live && p < npk) v[k] = ld_stream16(xp + p);
        else v[k] = make_uint4(0u, 0u, 0u, 0u);
    }
    AbsMax<T> am;
#pragma unroll
    for (int k = 0; k < PACKS; ++k) am.update(v[k]);
    float m = am.finish();

    if constexpr (TEAM <= 32) {
        m = team_max<TEAM>(m);
    } else {
        __shared__ float red[kBlock / 32];
        m = block_max(m, red);
    }
    const InvScale is = inv_and_scale<Code>(m, eps);
    if (live && t == 0) scale_out[seg] = is.scale;

    uint8_t* qp = q + seg * (int64_t)npk * E;
#pragma unroll
    for (int k = 0; k < PACKS; ++k) {
        const int p = t + k * TEAM;
        if (live && p < npk) {
            const uint2 codes = pack_encode<T, Code>(v[k], is.inv);
            if constexpr (E == 8) st_stream8(qp + (int64_t)p * 8, codes);
            else st_stream4(qp + (int64_t)p * 4, codes.x);
        }
    }
}

// Rows too long for registers: one CTA per row, the row is read twice but the
// second read follows the first immediately and is served by L2.
template <typename T, typename Code>
__global__ void __launch_bounds__(kBlock) quant_long_rows_kernel(const T* __restrict__ x, int64_t npk, float eps,
                                                                 uint8_t* __restrict__ q,
                                                                 float* __restrict__ scale_out) {
    constexpr int E = DTypeTraits<T>::kLanes;
    const int64_t seg = blockIdx.x;
    const uint4* xp = reinterpret_cast<const uint4*>(x) + seg * npk;
    AbsMax<T> am;
    for (int64_t p = threadIdx.x; p < npk; p += kBlock) am.update(ld_keep16(xp + p));
    __shared__ float red[kBlock / 32];
    const float m = block_max(am.finish(), red);
    const InvScale is = inv_and_scale<Code>(m, eps);
    if (threadIdx.x == 0) scale_out[seg] = is.scale;
    uint8_t* qp = q + seg * npk * E;
    for (int64_t p = threadIdx.x; p < npk; p += kBlock) {
        const uint2 codes = pack_encode<T, Code>(ld_stream16(xp + p), is.inv);
        if constexpr (E == 8) st_stream8(qp + p * 8, codes);
        else st_stream4(qp + p * 4, codes.x);
    }
}

// Any L, any alignment: one CTA of 128 threads per segment, scalar accesses.
template <typename T, typename Code>
__global__ void __launch_bounds__(128) quant_segments_scalar_kernel(const T* __restrict__ x, int64_t L, float eps,
                                                                    uint8_t* __restrict__ q,
                                                                    float* __restrict__ scale_out) {
    const int64_t seg = blockIdx.x;
    const T* xs = x + seg * L;
    float m = 0.0f;
    for (int64_t i = threadIdx.x; i < L; i += 128) m = fmaxf(m, fabsf(DTypeTraits<T>::to_float(xs[i])));
    __shared__ float red[kBlock / 32];
    m = block_max(m, red);
    const InvScale is = inv_and_scale<Code>(m, eps);
    if (threadIdx.x == 0) scale_out[seg] = is.scale;
    uint8_t* qs = q + seg * L;
    for (int64_t i = threadIdx.x; i < L; i += 128)
        qs[i] = Code::encode1(__fmul_rn(DTypeTraits<T>::to_float(xs[i]), is.inv));
}

// ===========================================================================
// Dequantize: y = T_rn(float(code) * scale[segment]).  One flat kernel.
// (reference: dequantize_per_tensor_fp8.cu:23-66, dequantize_int8.cu:29-134)
// SEG: 0 = one scale; 1 = packs per segment is a power of two (shift);
//      2 = general (64-bit divide).
// A CTA iteration covers kBlock*4 packs of 8 codes = 8 KiB in, 16 KiB out.
// ===========================================================================
template <typename OutT, typename Code, int SEG>
__global__ void __launch_bounds__(kBlock) dequant_kernel(const uint8_t* __restrict__ q,
                                                         const float* __restrict__ scale, int64_t n,
                                                         int64_t pps /* packs per segment, or shift */,
                                                         OutT* __restrict__ y) {
    constexpr int kChunkPacks = kBlock * 4;
    pdl_wait();  // codes and scales may come from the kernel just before this one
    pdl_trigger();
    const int64_t npk = n / 8;
    const int64_t nchunks = (npk + kChunkPacks - 1) / kChunkPacks;
    const uint2* qp = reinterpret_cast<const uint2*>(q);
    uint4* yp = reinterpret_cast<uint4*>(y);
    float s0 = 0.0f;
    if constexpr (SEG == 0) s0 = __ldg(scale);
    for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const int64_t p0 = c * kChunkPacks + threadIdx.x;
        uint2 v[4];
        float s[4];
        bool ok[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t p = p0 + k * kBlock;
            ok[k] = p < npk;
            if (ok[k]) {
                v[k] = ld_stream8(qp + p);
                if constexpr (SEG == 0) s[k] = s0;
                else if constexpr (SEG == 1) s[k] = __ldg(scale + (p >> pps));
                else s[k] = __ldg(scale + (p / pps));
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (!ok[k]) continue;
            st_stream16(yp + p0 + k * kBlock, codes_decode8<OutT, Code>(v[k], s[k]));
        }
    }
    if constexpr (SEG == 0) {
        if (blockIdx.x == 0) {
            const int64_t t = npk * 8 + threadIdx.x;
            if (t < n) y[t] = DTypeTraits<OutT>::from_float(__fmul_rn(Code::decode1(q[t]), s0));
        }
    }
}

// Same, 16 codes per thread per step: one 128-bit load of codes, one 256-bit store of 16-bit values
// (a full 32-byte sector per thread per store instruction).  Needs n and seg_len to be multiples
// of 16 apart from a scalar tail, q 16-byte and y 32-byte aligned.
template <typename OutT, typename Code, int SEG>
__global__ void __launch_bounds__(kBlock) dequant16_kernel(const uint8_t* __restrict__ q,
                                                           const float* __restrict__ scale, int64_t n,
                                                           int64_t pps /* 16-packs per segment, or shift */,
                                                           int64_t seg_len, OutT* __restrict__ y) {
    constexpr int kChunkPacks = kBlock * 4;
    pdl_wait();  // codes and scales may come from the kernel just before this one
    pdl_trigger();
    const int64_t npk = n / 16;
    const int64_t nchunks = (npk + kChunkPacks - 1) / kChunkPacks;
    const uint4* qp = reinterpret_cast<const uint4*>(q);
    float s0 = 0.0f;
    if constexpr (SEG == 0) s0 = __ldg(scale);
    for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const int64_t p0 = c * kChunkPacks + threadIdx.x;
        uint4 v[4];
        float s[4];
        bool ok[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t p = p0 + k * kBlock;
            ok[k] = p < npk;
            if (ok[k]) {
                v[k] = ld_stream16(qp + p);
                if constexpr (SEG == 0) s[k] = s0;
                else if constexpr (SEG == 1) s[k] = __ldg(scale + (p >> pps));
                else s[k] = __ldg(scale + (p / pps));
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (!ok[k]) continue;
            const uint4 lo = codes_decode8<OutT, Code>(make_uint2(v[k].x, v[k].y), s[k]);
            const uint4 hi = codes_decode8<OutT, Code>(make_uint2(v[k].z, v[k].w), s[k]);
            st_stream32(y + (p0 + k * kBlock) * 16, lo, hi);
        }
    }
    if (blockIdx.x == 0) {  // fewer than 16 trailing codes
        const int64_t t = npk * 16 + threadIdx.x;
        if (t < n) {
            const float st = __ldg(scale + (seg_len > 0 ? t / seg_len : 0));
            y[t] = DTypeTraits<OutT>::from_float(__fmul_rn(Code::decode1(q[t]), st));
        }
    }
}

template <typename OutT, typename Code>
__global__ void __launch_bounds__(kBlock) dequant_scalar_kernel(const uint8_t* __restrict__ q,
                                                                const float* __restrict__ scale, int64_t n,
                                                                int64_t seg_len, OutT* __restrict__ y) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (int64_t)gridDim.x * kBlock) {
        const float s = __ldg(scale + (seg_len > 0 ? i / seg_len : 0));
        y[i] = DTypeTraits<OutT>::from_float(__fmul_rn(Code::decode1(q[i]), s));
    }
}

// ===========================================================================
// Launchers
// ===========================================================================
static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// CTAs for a grid-stride loop over work_items chunks: at most ctas_per_sm resident CTAs per SM, and of the
// grids with that many loop iterations the smallest, so every CTA gets the same number of chunks (+-1)
// instead of a full wave followed by a partly filled one.
static inline int persistent_grid(int64_t work_items, int ctas_per_sm) {
    const int64_t cap = (int64_t)sm_count() * ctas_per_sm;
    if (work_items <= cap) return (int)(work_items < 1 ? 1 : work_items);
    const int64_t iters = (work_items + cap - 1) / cap;
    return (int)((work_items + iters - 1) / iters);
}

// grid of the amax kernel for n elements (= number of partial slots it writes in PARTIALS mode)
template <typename T>
static int amax_grid(const void* x, int64_t n) {
    constexpr int E = DTypeTraits<T>::kLanes;
    if (aligned(x, 16)) return persistent_grid((n / E + kBlock * 4 - 1) / (kBlock * 4), 8);
    return persistent_grid((n + kBlock - 1) / kBlock, 8);
}

template <typename T, bool PARTIALS>
static cudaError_t amax_tensor_t(const void* x, int64_t n, float* amax, int* nparts, cudaStream_t s) {
    if (nparts) *nparts = 0;
    if (n <= 0) return cudaSuccess;
    const int grid = amax_grid<T>(x, n);
    if (nparts) *nparts = grid;
    if (aligned(x, 16))
        return launch_dependent(amax_tensor_kernel<T, PARTIALS>, (unsigned)grid, kBlock, 0, s, static_cast<const T*>(x), n,
                                amax);
    return launch_dependent(amax_tensor_scalar_kernel<T, PARTIALS>, (unsigned)grid, kBlock, 0, s, static_cast<const T*>(x),
                            n, amax);
}

cudaError_t launch_amax_tensor(const void* x, int dtype, int64_t n, float* amax, cudaStream_t s) {
    switch (dtype) {
        case kF16: return amax_tensor_t<__half, false>(x, n, amax, nullptr, s);
        case kBF16: return amax_tensor_t<__nv_bfloat16, false>(x, n, amax, nullptr, s);
        case kF32: return amax_tensor_t<float, false>(x, n, amax, nullptr, s);
    }
    return cudaErrorInvalidValue;
}

int per_tensor_scratch_floats() { return sm_count() * 8; }

cudaError_t launch_amax_partials(const void* x, int dtype, int64_t n, float* partials, int* nparts, cudaStream_t s) {
    switch (dtype) {
        case kF16: return amax_tensor_t<__half, true>(x, n, partials, nparts, s);
        case kBF16: return amax_tensor_t<__nv_bfloat16, true>(x, n, partials, nparts, s);
        case kF32: return amax_tensor_t<float, true>(x, n, partials, nparts, s);
    }
    return cudaErrorInvalidValue;
}

template <typename T, typename Code>
static cudaError_t cast_tensor_t(const void* x, int64_t n, const float* amax, int nparts, float eps, void* q,
                                 float* scale_out, cudaStream_t s) {
    constexpr int E = DTypeTraits<T>::kLanes;
    // n == 0 still writes the scale (amax 0 -> eps), as the reference's launch of an empty grid would not;
    // the host layer never calls with n == 0, keep one CTA so scale_out is defined.
    if (aligned(x, 16) && aligned(q, 8)) {
        const int64_t nchunks = (n / E + kBlock * 4 - 1) / (kBlock * 4);
        return launch_dependent(cast_tensor_kernel<T, Code>, (unsigned)persistent_grid(nchunks, 8), kBlock, 0, s,
                                static_cast<const T*>(x), n, amax, nparts, eps, static_cast<uint8_t*>(q), scale_out);
    }
    return launch_dependent(cast_tensor_scalar_kernel<T, Code>, (unsigned)persistent_grid((n + kBlock - 1) / kBlock, 8),
                            kBlock, 0, s, static_cast<const T*>(x), n, amax, nparts, eps, static_cast<uint8_t*>(q),
                            scale_out);
}

cudaError_t launch_cast_tensor(const void* x, int dtype, int64_t n, const float* amax, int nparts, float eps, int code,
                               void* q, float* scale_out, cudaStream_t s) {
    if (code == kCodeE4M3) {
        switch (dtype) {
            case kF16: return cast_tensor_t<__half, E4M3Code>(x, n, amax, nparts, eps, q, scale_out, s);
            case kBF16: return cast_tensor_t<__nv_bfloat16, E4M3Code>(x, n, amax, nparts, eps, q, scale_out, s);
            case kF32: return cast_tensor_t<float, E4M3Code>(x, n, amax, nparts, eps, q, scale_out, s);
        }
    } else if (code == kCodeInt8) {
        switch (dtype) {
            case kF16: return cast_tensor_t<__half, Int8CodeClamped>(x, n, amax, nparts, eps, q, scale_out, s);
            case kBF16: return cast_tensor_t<__nv_bfloat16, Int8CodeClamped>(x, n, amax, nparts, eps, q, scale_out, s);
            case kF32: return cast_tensor_t<float, Int8CodeClamped>(x, n, amax, nparts, eps, q, scale_out, s);
        }
    }
    return cudaErrorInvalidValue;
}

template <typename T, typename Code, int TEAM, int PACKS>
static void seg_launch(const void* x, int64_t nseg, int npk, float eps, void* q, float* scale_out, cudaStream_t s) {
    // sub-warp teams share a 256-thread CTA; a CTA-wide team is its own CTA
    constexpr int BLOCK = TEAM > 32 ? TEAM : kBlock;
    constexpr int kTeamsPerCta = BLOCK / TEAM;
    const int64_t grid = (nseg + kTeamsPerCta - 1) / kTeamsPerCta;
    quant_segments_kernel<T, Code, TEAM, PACKS, BLOCK><<<(unsigned)grid, BLOCK, 0, s>>>(
        static_cast<const T*>(x), nseg, npk, eps, static_cast<uint8_t*>(q), scale_out);
}

template <typename T, typename Code, int TEAM>
static void seg_pick_packs(int packs, const void* x, int64_t nseg, int npk, float eps, void* q, float* sc,
                           cudaStream_t s) {
    if (packs <= 1) seg_launch<T, Code, TEAM, 1>(x, nseg, npk, eps, q, sc, s);
    else if (packs <= 2) seg_launch<T, Code, TEAM, 2>(x, nseg, npk, eps, q, sc, s);
    else if (packs <= 4) seg_launch<T, Code, TEAM, 4>(x, nseg, npk, eps, q, sc, s);
    else {
        if constexpr (TEAM > 32) seg_launch<T, Code, TEAM, 8>(x, nseg, npk, eps, q, sc, s);
    }
}

template <typename T, typename Code>
static cudaError_t quant_segments_t(const void* x, int64_t nseg, int64_t L, float eps, void* q, float* scale_out,
                                    cudaStream_t s) {
    constexpr int E = DTypeTraits<T>::kLanes;
    if (nseg <= 0 || L <= 0) return cudaSuccess;
    if (nseg > 0x7fffffffLL) return cudaErrorInvalidValue;
    const bool vec_ok = (L % E == 0) && aligned(x, 16) && aligned(q, E == 8 ? 8 : 4);
    if (!vec_ok) {
        quant_segments_scalar_kernel<T, Code><<<(unsigned)nseg, 128, 0, s>>>(
            static_cast<const T*>(x), L, eps, static_cast<uint8_t*>(q), scale_out);
        return cudaPeekAtLastError();
    }
    const int64_t npk64 = L / E;
    if (npk64 > kBlock * 8) {
        quant_long_rows_kernel<T, Code><<<(unsigned)nseg, kBlock, 0, s>>>(
            static_cast<const T*>(x), npk64, eps, static_cast<uint8_t*>(q), scale_out);
        return cudaPeekAtLastError();
    }
    const int npk = (int)npk64;
    // smallest team whose threads need at most 4 packs each (8 for a whole CTA)
    if (npk <= 4 * 4) seg_pick_packs<T, Code, 4>((npk + 3) / 4, x, nseg, npk, eps, q, scale_out, s);
    else if (npk <= 8 * 4) seg_pick_packs<T, Code, 8>((npk + 7) / 8, x, nseg, npk, eps, q, scale_out, s);
    else if (npk <= 16 * 4) seg_pick_packs<T, Code, 16>((npk + 15) / 16, x, nseg, npk, eps, q, scale_out, s);
    else if (npk <= 32 * 4) seg_pick_packs<T, Code, 32>((npk + 31) / 32, x, nseg, npk, eps, q, scale_out, s);
    else seg_pick_packs<T, Code, kBlock>((npk + kBlock - 1) / kBlock, x, nseg, npk, eps, q, scale_out, s);
    return cudaPeekAtLastError();
}

cudaError_t launch_quant_segments(const void* x, int dtype, int64_t nseg, int64_t L, float eps, int code, void* q,
                                  float* scale_out, cudaStream_t s) {
    if (code == kCodeInt8) {
        switch (dtype) {
            case kF16: return quant_segments_t<__half, Int8Code>(x, nseg, L, eps, q, scale_out, s);
            case kBF16: return quant_segments_t<__nv_bfloat16, Int8Code>(x, nseg, L, eps, q, scale_out, s);
            case kF32: return quant_segments_t<float, Int8Code>(x, nseg, L, eps, q, scale_out, s);
        }
    } else if (code == kCodeE4M3) {
        switch (dtype) {
            case kF16: return quant_segments_t<__half, E4M3Code>(x, nseg, L, eps, q, scale_out, s);
            case kBF16: return quant_segments_t<__nv_bfloat16, E4M3Code>(x, nseg, L, eps, q, scale_out, s);
            case kF32: return quant_segments_t<float, E4M3Code>(x, nseg, L, eps, q, scale_out, s);
        }
    }
    return cudaErrorInvalidValue;
}

template <typename OutT, typename Code>
static cudaError_t dequant_t(const void* q, const float* scale, int64_t n, int64_t seg_len, void* y, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    const bool vec_ok = aligned(q, 8) && aligned(y, 16) && (seg_len == 0 || seg_len % 8 == 0);
    const uint8_t* qp = static_cast<const uint8_t*>(q);
    OutT* yp = static_cast<OutT*>(y);
    if (!vec_ok) {
        launch_dependent(dequant_scalar_kernel<OutT, Code>, (unsigned)persistent_grid((n + kBlock - 1) / kBlock, 8), kBlock, 0, s, 
            qp, scale, n, seg_len, yp);
        return cudaPeekAtLastError();
    }
    if (aligned(q, 16) && aligned(y, 32) && (seg_len == 0 || seg_len % 16 == 0)) {
        const int64_t nchunks16 = (n / 16 + kBlock * 4 - 1) / (kBlock * 4);
        const int grid16 = persistent_grid(nchunks16, 8);
        if (seg_len == 0) {
            launch_dependent(dequant16_kernel<OutT, Code, 0>, (unsigned)grid16, kBlock, 0, s, qp, scale, n, 0, 0, yp);
        } else {
            const int64_t pps = seg_len / 16;
            if ((pps & (pps - 1)) == 0) {
                int shift = 0;
                while ((int64_t(1) << shift) < pps) ++shift;
                launch_dependent(dequant16_kernel<OutT, Code, 1>, (unsigned)grid16, kBlock, 0, s, qp, scale, n, shift, seg_len, yp);
            } else {
                launch_dependent(dequant16_kernel<OutT, Code, 2>, (unsigned)grid16, kBlock, 0, s, qp, scale, n, pps, seg_len, yp);
            }
        }
        return cudaPeekAtLastError();
    }
    const int64_t nchunks = (n / 8 + kBlock * 4 - 1) / (kBlock * 4);
    const int grid = persistent_grid(nchunks, 8);
    if (seg_len == 0) {
        launch_dependent(dequant_kernel<OutT, Code, 0>, (unsigned)grid, kBlock, 0, s, qp, scale, n, 0, yp);
    } else {
        const int64_t pps = seg_len / 8;
        if ((pps & (pps - 1)) == 0) {
            int shift = 0;
            while ((int64_t(1) << shift) < pps) ++shift;
            launch_dependent(dequant_kernel<OutT, Code, 1>, (unsigned)grid, kBlock, 0, s, qp, scale, n, shift, yp);
        } else {
            launch_dependent(dequant_kernel<OutT, Code, 2>, (unsigned)grid, kBlock, 0, s, qp, scale, n, pps, yp);
        }
    }
    return cudaPeekAtLastError();
}

cudaError_t launch_dequant(const void* q, int code, const float* scale, int64_t n, int64_t seg_len, int out_dtype,
                           void* y, cudaStream_t s) {
    if (code == kCodeInt8) {
        if (out_dtype == kF16) return dequant_t<__half, Int8Code>(q, scale, n, seg_len, y, s);
        if (out_dtype == kBF16) return dequant_t<__nv_bfloat16, Int8Code>(q, scale, n, seg_len, y, s);
    } else if (code == kCodeE4M3) {
        if (out_dtype == kF16) return dequant_t<__half, E4M3Code>(q, scale, n, seg_len, y, s);
        if (out_dtype == kBF16) return dequant_t<__nv_bfloat16, E4M3Code>(q, scale, n, seg_len, y, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cb
