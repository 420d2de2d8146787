// INT8 per-channel quantize / dequantize along ANY axis of a contiguous tensor, without a transpose.
//
// The reference advertises an axis-configurable per-channel mode (README.md:16) but its code accepts
// only axis 0 (cublade/quantization/quantizers.py:117-120) and its group mode moves other axes to the
// back with an ATen copy (quantizers.py:122-132).  Here the tensor is viewed as [outer, C, inner]
// (C = the channel axis, inner = product of the axes behind it) and indexed in place.  The arithmetic
// per channel is that of the axis-0 quantizer (cublade/kernels/cuda/quantization/quantize_int8.cu:
// 245-296): amax over the channel, inv = 127 / max(amax, eps), q = clamp(rint(x * inv)), scale = 1 / inv,
// so the result equals "movedim(axis, 0), quantize per channel, move back" bit for bit.
//
// A channel's elements are scattered over `outer` runs, so the amax is global per channel and the
// op is two-phase like the per-tensor quantizer: (1) per-channel amax by integer atomicMax on the bit
// pattern of a non-negative float, (2) a C-thread kernel turning amax into inv and scale, (3) the cast.
// x is read twice: 5 bytes per element, or 3 when the tensor fits in the 126 MB L2.
//
// Two vector layouts cover the common shapes:
//   kRuns  : inner % lanes == 0 -- every 16-byte pack lies inside one channel run; channel of pack p is
//            (p / (inner / lanes)) % C.  (Weights quantized along axis 1 of [O, I, kh, kw], ...)
//   kLast  : inner == 1, C % lanes == 0 -- the channel axis is the last one ([tokens, hidden] per
//            feature); a thread owns one pack of 8 (4) adjacent channels and walks down the rows.
// Everything else takes a scalar kernel.
#include "launch.h"
#include "pack.cuh"

namespace cb {

namespace {

constexpr int kBlock = 256;

__device__ __forceinline__ void atomic_max_abs(float* slot, float m) {
    // m >= 0: the order of non-negative floats is the order of their bit patterns
    if (m > 0.0f) atomicMax(reinterpret_cast<unsigned int*>(slot), __float_as_uint(m));
}

// channel of pack p when a channel run is ppr packs long: (p / ppr) % C.  64-bit division is an
// instruction sequence of its own; tensors below 2^31 packs (every real one) take the 32-bit route.
__device__ __forceinline__ int64_t channel_of_pack(int64_t p, int64_t ppr, int64_t C, bool small) {
    if (small) return (int64_t)(((uint32_t)p / (uint32_t)ppr) % (uint32_t)C);
    return (p / ppr) % C;
}

template <typename T>
__device__ __forceinline__ float pack_absmax(const uint4& raw) {
    AbsMax<T> am;
    am.update(raw);
    return am.finish();
}

// ---------------------------------------------------------------------------------------------
// kRuns layout
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kBlock) amax_runs_kernel(const T* __restrict__ x, int64_t npk, int64_t ppr, int64_t C,
                                                           float* __restrict__ amax) {
    const uint4* xp = reinterpret_cast<const uint4*>(x);
    constexpr int kChunkPacks = kBlock * 4;
    const int64_t nchunks = (npk + kChunkPacks - 1) / kChunkPacks;
    const bool small = npk < 0x7fffffffLL && C < 0x7fffffffLL;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ float red[kBlock / 32];
    for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const int64_t first = c * kChunkPacks;
        const int64_t last = first + kChunkPacks - 1 < npk ? first + kChunkPacks - 1 : npk - 1;
        const int64_t p0 = first + threadIdx.x;
        uint4 v[4];
        bool ok[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            ok[k] = p0 + k * kBlock < npk;
            v[k] = ok[k] ? ld_keep16(xp + p0 + k * kBlock) : make_uint4(0u, 0u, 0u, 0u);
        }
        const int64_t run_first = small ? (int64_t)((uint32_t)first / (uint32_t)ppr) : first / ppr;
        const int64_t run_last = small ? (int64_t)((uint32_t)last / (uint32_t)ppr) : last / ppr;
        if (run_first == run_last) {
            // the whole 16 KiB chunk lies in one channel run: one atomic for the CTA
            AbsMax<T> am;
#pragma unroll
            for (int k = 0; k < 4; ++k) am.update(v[k]);
            float m = team_max<32>(am.finish());
            if (lane == 0) red[warp] = m;
            __syncthreads();
            if (warp == 0) {
                m = team_max<8>(lane < kBlock / 32 ? red[lane] : 0.0f);
                if (lane == 0) atomic_max_abs(amax + (small ? (int64_t)((uint32_t)run_first % (uint32_t)C) : run_first % C), m);
            }
            __syncthreads();
        } else {
            // runs shorter than a chunk: lanes of a warp that share a channel elect one of them
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int64_t p = p0 + k * kBlock;
                const int ch = ok[k] ? (int)channel_of_pack(p, ppr, C, small) : -1;
                const unsigned bits = __float_as_uint(pack_absmax<T>(v[k]));
                if (small) {
                    const unsigned peers = __match_any_sync(0xffffffffu, ch);
                    const unsigned top = __reduce_max_sync(peers, bits);
                    if (ch >= 0 && lane == __ffs(peers) - 1 && top != 0u)
                        atomicMax(reinterpret_cast<unsigned int*>(amax) + ch, top);
                } else if (ok[k]) {
                    atomic_max_abs(amax + channel_of_pack(p, ppr, C, false), __uint_as_float(bits));
                }
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kBlock) cast_runs_kernel(const T* __restrict__ x, int64_t npk, int64_t ppr, int64_t C,
                                                           const float* __restrict__ inv, uint8_t* __restrict__ q) {
    constexpr int E = DTypeTraits<T>::kLanes;
    const uint4* xp = reinterpret_cast<const uint4*>(x);
    constexpr int kChunkPacks = kBlock * 4;
    const int64_t nchunks = (npk + kChunkPacks - 1) / kChunkPacks;
    const bool small = npk < 0x7fffffffLL && C < 0x7fffffffLL;
    for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const int64_t p0 = c * kChunkPacks + threadIdx.x;
        uint4 v[4];
        float iv[4];
        bool ok[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t p = p0 + k * kBlock;
            ok[k] = p < npk;
            if (ok[k]) {
                v[k] = ld_stream16(xp + p);
                iv[k] = __ldg(inv + channel_of_pack(p, ppr, C, small));
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (!ok[k]) continue;
            const int64_t p = p0 + k * kBlock;
            const uint2 codes = pack_encode<T, Int8CodeClamped>(v[k], iv[k]);
            if constexpr (E == 8) st_stream8(q + p * 8, codes);
            else st_stream4(q + p * 4, codes.x);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// kLast layout: x is [rows, C]; thread = one pack of adjacent channels, blockIdx.y = a slab of rows
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kBlock) amax_last_kernel(const T* __restrict__ x, int64_t rows, int64_t cpk,
                                                           int64_t rows_per_slab, float* __restrict__ amax) {
    constexpr int E = DTypeTraits<T>::kLanes;
    const int64_t cp = (int64_t)blockIdx.x * kBlock + threadIdx.x;  // column pack
    if (cp >= cpk) return;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_slab;
    const int64_t r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
    const uint4* xp = reinterpret_cast<const uint4*>(x) + cp;
    float m[E];
#pragma unroll
    for (int e = 0; e < E; ++e) m[e] = 0.0f;
    int64_t r = r0;
    for (; r + 8 <= r1; r += 8) {  // eight rows in flight
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = ld_keep16(xp + (r + k) * cpk);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float f[E];
            pack_to_floats<T>(v[k], f);
#pragma unroll
            for (int e = 0; e < E; ++e) m[e] = fmaxf(m[e], fabsf(f[e]));
        }
    }
    for (; r < r1; ++r) {
        float f[E];
        pack_to_floats<T>(ld_keep16(xp + r * cpk), f);
#pragma unroll
        for (int e = 0; e < E; ++e) m[e] = fmaxf(m[e], fabsf(f[e]));
    }
#pragma unroll
    for (int e = 0; e < E; ++e) atomic_max_abs(amax + cp * E + e, m[e]);
}

template <typename T>
__global__ void __launch_bounds__(kBlock) cast_last_kernel(const T* __restrict__ x, int64_t rows, int64_t cpk,
                                                           int64_t rows_per_slab, const float* __restrict__ inv,
                                                           uint8_t* __restrict__ q) {
    constexpr int E = DTypeTraits<T>::kLanes;
    const int64_t cp = (int64_t)blockIdx.x * kBlock + threadIdx.x;
    if (cp >= cpk) return;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_slab;
    const int64_t r1 = r0 + rows_per_slab < rows ? r0 + rows_per_slab : rows;
    const uint4* xp = reinterpret_cast<const uint4*>(x) + cp;
    float iv[E];
#pragma unroll
    for (int e = 0; e < E; ++e) iv[e] = __ldg(inv + cp * E + e);
    auto emit = [&](int64_t r, const uint4& raw) {
        float f[E];
        pack_to_floats<T>(raw, f);
#pragma unroll
        for (int e = 0; e < E; ++e) f[e] = __fmul_rn(f[e], iv[e]);
        const uint32_t lo = Int8CodeClamped::encode4(f[0], f[1], f[2], f[3]);
        if constexpr (E == 8) {
            const uint32_t hi = Int8CodeClamped::encode4(f[4], f[5], f[6], f[7]);
            st_stream8(q + (r * cpk + cp) * 8, make_uint2(lo, hi));
        } else {
            st_stream4(q + (r * cpk + cp) * 4, lo);
        }
    };
    int64_t r = r0;
    for (; r + 8 <= r1; r += 8) {
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = ld_stream16(xp + (r + k) * cpk);
#pragma unroll
        for (int k = 0; k < 8; ++k) emit(r + k, v[k]);
    }
    for (; r < r1; ++r) emit(r, ld_stream16(xp + r * cpk));
}

// ---------------------------------------------------------------------------------------------
// any shape, any alignment
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kBlock) amax_axis_scalar_kernel(const T* __restrict__ x, int64_t n, int64_t inner,
                                                                  int64_t C, float* __restrict__ amax) {
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (int64_t)gridDim.x * kBlock)
        atomic_max_abs(amax + (i / inner) % C, fabsf(DTypeTraits<T>::to_float(x[i])));
}

template <typename T>
__global__ void __launch_bounds__(kBlock) cast_axis_scalar_kernel(const T* __restrict__ x, int64_t n, int64_t inner,
                                                                  int64_t C, const float* __restrict__ inv,
                                                                  uint8_t* __restrict__ q) {
    for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (int64_t)gridDim.x * kBlock)
        q[i] = Int8CodeClamped::encode1(__fmul_rn(DTypeTraits<T>::to_float(x[i]), __ldg(inv + (i / inner) % C)));
}

// amax[c] -> inv[c] (kept in the scratch, overwriting amax) and scale[c]
__global__ void __launch_bounds__(kBlock) finish_axis_scales_kernel(float* __restrict__ amax_to_inv, int64_t C, float eps,
                                                                    float* __restrict__ scale_out) {
    const int64_t c = (int64_t)blockIdx.x * kBlock + threadIdx.x;
    if (c >= C) return;
    const InvScale is = inv_and_scale<Int8Code>(amax_to_inv[c], eps);
    amax_to_inv[c] = is.inv;
    scale_out[c] = is.scale;
}

// ---------------------------------------------------------------------------------------------
// dequantize: y[o, c, i] = T(float(q[o, c, i]) * scale[c])
// ---------------------------------------------------------------------------------------------
// LAYOUT 0: every 8-code pack inside one run (inner % 8 == 0); 1: last axis, C % 8 == 0; 2: scalar
template <typename OutT, int LAYOUT>
__global__ void __launch_bounds__(kBlock) dequant_axis_kernel(const uint8_t* __restrict__ q,
                                                              const float* __restrict__ scale, int64_t n, int64_t inner,
                                                              int64_t C, OutT* __restrict__ y) {
    if constexpr (LAYOUT == 2) {
        for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (int64_t)gridDim.x * kBlock)
            y[i] = DTypeTraits<OutT>::from_float(__fmul_rn(Int8Code::decode1(q[i]), __ldg(scale + (i / inner) % C)));
    } else {
        const int64_t npk = n / 8;
        const int64_t ppr = LAYOUT == 0 ? inner / 8 : 0, cpk = LAYOUT == 1 ? C / 8 : 0;
        const uint2* qp = reinterpret_cast<const uint2*>(q);
        uint4* yp = reinterpret_cast<uint4*>(y);
        const bool small = npk < 0x7fffffffLL && C < 0x7fffffffLL;
        for (int64_t p = (int64_t)blockIdx.x * kBlock + threadIdx.x; p < npk; p += (int64_t)gridDim.x * kBlock) {
            const uint2 codes = ld_stream8(qp + p);
            if constexpr (LAYOUT == 0) {
                st_stream16(yp + p, codes_decode8<OutT, Int8Code>(codes, __ldg(scale + channel_of_pack(p, ppr, C, small))));
            } else {
                const int64_t cp = small ? (int64_t)((uint32_t)p % (uint32_t)cpk) : p % cpk;
                const float4* sp = reinterpret_cast<const float4*>(scale) + cp * 2;
                const float4 s0 = __ldg(sp), s1 = __ldg(sp + 1);
                float a[4], b[4];
                Int8Code::decode4(codes.x, a);
                Int8Code::decode4(codes.y, b);
                uint4 out;
                out.x = DTypeTraits<OutT>::float2_to_word(__fmul_rn(a[0], s0.x), __fmul_rn(a[1], s0.y));
                out.y = DTypeTraits<OutT>::float2_to_word(__fmul_rn(a[2], s0.z), __fmul_rn(a[3], s0.w));
                out.z = DTypeTraits<OutT>::float2_to_word(__fmul_rn(b[0], s1.x), __fmul_rn(b[1], s1.y));
                out.w = DTypeTraits<OutT>::float2_to_word(__fmul_rn(b[2], s1.z), __fmul_rn(b[3], s1.w));
                st_stream16(yp + p, out);
            }
        }
    }
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

inline int persistent_grid(int64_t work_items, int ctas_per_sm) {
    const int64_t cap = (int64_t)sm_count() * ctas_per_sm;
    const int64_t g = work_items < cap ? work_items : cap;
    return (int)(g < 1 ? 1 : g);
}

template <typename T>
cudaError_t quant_axis_t(const void* xv, int64_t outer, int64_t C, int64_t inner, float eps, void* qv, float* scale_out,
                         float* scratch, cudaStream_t s) {
    constexpr int E = DTypeTraits<T>::kLanes;
    const T* x = static_cast<const T*>(xv);
    uint8_t* q = static_cast<uint8_t*>(qv);
    const int64_t n = outer * C * inner;
    cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)C * sizeof(float), s);
    if (e != cudaSuccess) return e;
    const bool al = aligned_to(x, 16) && aligned_to(q, E == 8 ? 8 : 4);
    const unsigned cgrid = (unsigned)((C + kBlock - 1) / kBlock);
    if (n > 0 && al && inner % E == 0) {
        const int64_t npk = n / E, ppr = inner / E;
        const int grid = persistent_grid((npk + kBlock * 4 - 1) / (kBlock * 4), 8);
        amax_runs_kernel<T><<<grid, kBlock, 0, s>>>(x, npk, ppr, C, scratch);
        finish_axis_scales_kernel<<<cgrid, kBlock, 0, s>>>(scratch, C, eps, scale_out);
        cast_runs_kernel<T><<<grid, kBlock, 0, s>>>(x, npk, ppr, C, scratch, q);
    } else if (n > 0 && al && inner == 1 && C % E == 0) {
        const int64_t cpk = C / E, rows = outer;
        const unsigned gx = (unsigned)((cpk + kBlock - 1) / kBlock);
        // enough row slabs to fill the GPU four CTAs deep (8 x 16 bytes in flight per thread), at least 32 rows
        // each: every slab ends with one atomicMax per channel, so fewer, taller slabs mean less contention
        int64_t slabs = ((int64_t)sm_count() * 4 + gx - 1) / gx;
        if (slabs > (rows + 31) / 32) slabs = (rows + 31) / 32;
        if (slabs < 1) slabs = 1;
        if (slabs > 65535) slabs = 65535;
        const int64_t rows_per_slab = (rows + slabs - 1) / slabs;
        const dim3 grid(gx, (unsigned)((rows + rows_per_slab - 1) / rows_per_slab));
        amax_last_kernel<T><<<grid, kBlock, 0, s>>>(x, rows, cpk, rows_per_slab, scratch);
        finish_axis_scales_kernel<<<cgrid, kBlock, 0, s>>>(scratch, C, eps, scale_out);
        cast_last_kernel<T><<<grid, kBlock, 0, s>>>(x, rows, cpk, rows_per_slab, scratch, q);
    } else {
        const int grid = persistent_grid((n + kBlock - 1) / kBlock, 8);
        if (n > 0) amax_axis_scalar_kernel<T><<<grid, kBlock, 0, s>>>(x, n, inner, C, scratch);
        finish_axis_scales_kernel<<<cgrid, kBlock, 0, s>>>(scratch, C, eps, scale_out);
        if (n > 0) cast_axis_scalar_kernel<T><<<grid, kBlock, 0, s>>>(x, n, inner, C, scratch, q);
    }
    return cudaPeekAtLastError();
}

template <typename OutT>
cudaError_t dequant_axis_t(const void* qv, const float* scale, int64_t outer, int64_t C, int64_t inner, void* yv,
                           cudaStream_t s) {
    const uint8_t* q = static_cast<const uint8_t*>(qv);
    OutT* y = static_cast<OutT*>(yv);
    const int64_t n = outer * C * inner;
    if (n <= 0) return cudaSuccess;
    const bool al = aligned_to(q, 8) && aligned_to(y, 16);
    if (al && inner % 8 == 0) {
        dequant_axis_kernel<OutT, 0><<<persistent_grid((n / 8 + kBlock - 1) / kBlock, 16), kBlock, 0, s>>>(q, scale, n, inner,
                                                                                                         C, y);
    } else if (al && inner == 1 && C % 8 == 0 && aligned_to(scale, 16)) {
        dequant_axis_kernel<OutT, 1><<<persistent_grid((n / 8 + kBlock - 1) / kBlock, 16), kBlock, 0, s>>>(q, scale, n, inner,
                                                                                                         C, y);
    } else {
        dequant_axis_kernel<OutT, 2><<<persistent_grid((n + kBlock - 1) / kBlock, 16), kBlock, 0, s>>>(q, scale, n, inner, C,
                                                                                                     y);
    }
    return cudaPeekAtLastError();
}

}  // namespace

cudaError_t launch_quant_axis(const void* x, int dtype, int64_t outer, int64_t C, int64_t inner, float eps, void* q,
                              float* scale_out, float* scratch, cudaStream_t s) {
    switch (dtype) {
        case kF16: return quant_axis_t<__half>(x, outer, C, inner, eps, q, scale_out, scratch, s);
        case kBF16: return quant_axis_t<__nv_bfloat16>(x, outer, C, inner, eps, q, scale_out, scratch, s);
        case kF32: return quant_axis_t<float>(x, outer, C, inner, eps, q, scale_out, scratch, s);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_dequant_axis(const void* q, const float* scale, int64_t outer, int64_t C, int64_t inner, int out_dtype,
                                void* y, cudaStream_t s) {
    if (out_dtype == kF16) return dequant_axis_t<__half>(q, scale, outer, C, inner, y, s);
    if (out_dtype == kBF16) return dequant_axis_t<__nv_bfloat16>(q, scale, outer, C, inner, y, s);
    return cudaErrorInvalidValue;
}

}  // namespace cb
