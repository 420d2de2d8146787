// INT8 per-group quantize / dequantize with the groups running along a NON-LAST axis of a contiguous
// [outer, C, inner] tensor, where the data lies -- no transposed copy before or after.
//
// The reference serves this case by moving the axis last with a materialised copy, quantizing rows of
// group_size contiguous elements, and moving the codes back with a second copy
// (cublade/quantization/quantizers.py:122-132, dequantizers.py:58-72): 2 + 2 + (2 + 1) + 1 + 1 = 9 bytes
// per element of HBM traffic instead of 3.  The arithmetic per group is the reference's
// (quantize_int8.cu:345-371, dequantize_int8.cu:118-134): amax over the group, inv = 127 / max(amax, eps),
// code = rint(x * inv), scale = 1 / inv.  Scales come out in the reference's order, i.e. flat over the
// moved layout [outer, inner, C / G]: scale[(o * inner + i) * (C / G) + c / G].
//
// Layout of the work: a group is G elements `inner` apart, so a thread takes the same 16-byte pack
// (8 or 4 neighbours along `inner`) of rows of a group: its lanes belong to 8 (4) DIFFERENT groups,
// adjacent threads read adjacent packs (coalesced), and every lane keeps its own running maximum,
// reciprocal and scale.  The second read of the packs comes from L2.
#include "launch.h"
#include "pack.cuh"

namespace cb {

namespace {

constexpr int kBlock = 256;

// per-lane running max |x| over packs: 16-bit types keep four packed pairs (one packed max per word)
template <typename T>
struct LaneAbsMax;

template <>
struct LaneAbsMax<float> {
    float m[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    __device__ __forceinline__ void update(const uint4& r) {
        m[0] = fmaxf(m[0], fabsf(__uint_as_float(r.x)));
        m[1] = fmaxf(m[1], fabsf(__uint_as_float(r.y)));
        m[2] = fmaxf(m[2], fabsf(__uint_as_float(r.z)));
        m[3] = fmaxf(m[3], fabsf(__uint_as_float(r.w)));
    }
    __device__ __forceinline__ void finish(float (&out)[4]) const {
#pragma unroll
        for (int k = 0; k < 4; ++k) out[k] = m[k];
    }
};

template <typename T, typename T2>
struct LaneAbsMax16 {
    uint32_t m[4] = {0u, 0u, 0u, 0u};  // packed pairs of non-negative 16-bit floats
    __device__ __forceinline__ void word(int k, uint32_t w) {
        w &= 0x7fff7fffu;
        const T2 r = __hmax2(*reinterpret_cast<const T2*>(&m[k]), *reinterpret_cast<const T2*>(&w));  // drops NaN
        m[k] = *reinterpret_cast<const uint32_t*>(&r);
    }
    __device__ __forceinline__ void update(const uint4& r) { word(0, r.x); word(1, r.y); word(2, r.z); word(3, r.w); }
    __device__ __forceinline__ void finish(float (&out)[8]) const {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 p = DTypeTraits<T>::word_to_float2(m[k]);
            out[2 * k] = p.x;
            out[2 * k + 1] = p.y;
        }
    }
};
template <>
struct LaneAbsMax<__half> : LaneAbsMax16<__half, __half2> {};
template <>
struct LaneAbsMax<__nv_bfloat16> : LaneAbsMax16<__nv_bfloat16, __nv_bfloat162> {};

// x viewed as packs: [outer, C, ppr] packs, ppr = inner / E.  One work item = (o, group cg, pack ip); a CTA of
// kWarps warps takes 32 consecutive items -- lane = item, so a warp's loads of one row are 32 adjacent packs -- and
// warp w takes rows w, w + kWarps, ... of the groups (four loads in flight per thread).  The per-lane maxima of the
// warps meet in shared memory; every thread then derives its items' reciprocals and encodes its own rows -- kept in
// registers for groups of up to 128 rows, read a second time (from L2) for longer ones.
constexpr int kWarps = kBlock / 32;

// R > 0: the thread's rows (at most R = ceil(G / kWarps) of them) stay in registers between the maximum and the encode,
// so x is read once; R == 0: any G, the rows are read a second time (from L2).
template <typename T, int R>
__global__ void __launch_bounds__(kBlock) quant_group_axis_kernel(const T* __restrict__ x, int64_t items, int64_t C,
                                                                  int64_t ppr, int G, float eps,
                                                                  uint8_t* __restrict__ q,
                                                                  float* __restrict__ scale_out) {
    constexpr int E = DTypeTraits<T>::kLanes;
    constexpr int RR = R > 0 ? R : 1;
    pdl_trigger();
    __shared__ float red[kWarps][E][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t ngr = C / G, inner = ppr * E;
    const uint4* xp = reinterpret_cast<const uint4*>(x);
    const int64_t w = (int64_t)blockIdx.x * 32 + lane;
    const bool live = w < items;
    const int64_t ip = live ? w % ppr : 0, og = live ? w / ppr : 0, cg = og % ngr, o = og / ngr;
    const int64_t pack0 = (o * C + cg * G) * ppr + ip;  // pack of row j of the group: pack0 + j * ppr
    LaneAbsMax<T> am;
    uint4 held[RR];
    if (live) {
        if constexpr (R > 0) {
#pragma unroll
            for (int k = 0; k < R; ++k) {
                const int j = warp + k * kWarps;
                held[k] = j < G ? ld_stream16(xp + pack0 + (int64_t)j * ppr) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int k = 0; k < R; ++k) am.update(held[k]);
        } else {
            int j = warp;
            for (; j + 3 * kWarps < G; j += 4 * kWarps) {
                const uint4 v0 = ld_keep16(xp + pack0 + (int64_t)(j + 0 * kWarps) * ppr);
                const uint4 v1 = ld_keep16(xp + pack0 + (int64_t)(j + 1 * kWarps) * ppr);
                const uint4 v2 = ld_keep16(xp + pack0 + (int64_t)(j + 2 * kWarps) * ppr);
                const uint4 v3 = ld_keep16(xp + pack0 + (int64_t)(j + 3 * kWarps) * ppr);
                am.update(v0); am.update(v1); am.update(v2); am.update(v3);
            }
            for (; j < G; j += kWarps) am.update(ld_keep16(xp + pack0 + (int64_t)j * ppr));
        }
    }
    float amax[E], inv[E];
    am.finish(amax);
#pragma unroll
    for (int l = 0; l < E; ++l) red[warp][l][lane] = amax[l];
    __syncthreads();
#pragma unroll
    for (int l = 0; l < E; ++l) {
        float m = red[0][l][lane];
#pragma unroll
        for (int k = 1; k < kWarps; ++k) m = fmaxf(m, red[k][l][lane]);
        const InvScale is = inv_and_scale<Int8Code>(m, eps);
        inv[l] = is.inv;
        // lane l of item (o, cg, ip) is position i = ip * E + l of the inner axis
        if (live && warp == (l % kWarps)) scale_out[(o * inner + ip * E + l) * ngr + cg] = is.scale;
    }
    if (!live) return;
    auto encode_store = [&](const uint4& raw, int64_t p) {
        float f[E];
        pack_to_floats<T>(raw, f);
#pragma unroll
        for (int l = 0; l < E; ++l) f[l] = __fmul_rn(f[l], inv[l]);
        const uint32_t lo = Int8Code::encode4(f[0], f[1], f[2], f[3]);
        if constexpr (E == 8) st_stream8(q + p * 8, make_uint2(lo, Int8Code::encode4(f[4], f[5], f[6], f[7])));
        else st_stream4(q + p * 4, lo);
    };
    if constexpr (R > 0) {
#pragma unroll
        for (int k = 0; k < R; ++k) {
            const int j = warp + k * kWarps;
            if (j < G) encode_store(held[k], pack0 + (int64_t)j * ppr);
        }
    } else {
        for (int j = warp; j < G; j += kWarps) {
            const int64_t p = pack0 + (int64_t)j * ppr;
            encode_store(ld_stream16(xp + p), p);
        }
    }
}

// any inner / alignment: one thread per (o, group, i)
template <typename T>
__global__ void __launch_bounds__(kBlock) quant_group_axis_scalar_kernel(const T* __restrict__ x, int64_t items,
                                                                         int64_t C, int64_t inner, int G, float eps,
                                                                         uint8_t* __restrict__ q,
                                                                         float* __restrict__ scale_out) {
    pdl_trigger();
    const int64_t ngr = C / G;
    for (int64_t w = (int64_t)blockIdx.x * kBlock + threadIdx.x; w < items; w += (int64_t)gridDim.x * kBlock) {
        const int64_t i = w % inner, og = w / inner, cg = og % ngr, o = og / ngr;
        const int64_t e0 = (o * C + cg * G) * inner + i;
        float m = 0.0f;
        for (int j = 0; j < G; ++j) m = fmaxf(m, fabsf(DTypeTraits<T>::to_float(x[e0 + (int64_t)j * inner])));
        const InvScale is = inv_and_scale<Int8Code>(m, eps);
        scale_out[(o * inner + i) * ngr + cg] = is.scale;
        for (int j = 0; j < G; ++j) {
            const int64_t e = e0 + (int64_t)j * inner;
            q[e] = Int8Code::encode1(__fmul_rn(DTypeTraits<T>::to_float(x[e]), is.inv));
        }
    }
}

// y[o, c, i] = float(q[o, c, i]) * scale[(o * inner + i) * (C / G) + c / G].
// Vector form: the work item of the quantizer -- (o, group, pack of 8 positions along inner), lane = item, warp w
// takes rows w, w + kWarps, ... -- so the eight scales of an item (C / G floats apart) are fetched once per thread
// and reused for all its rows.
template <typename OutT>
__global__ void __launch_bounds__(kBlock) dequant_group_axis_kernel(const uint8_t* __restrict__ q,
                                                                    const float* __restrict__ scale, int64_t items,
                                                                    int64_t C, int64_t ppr, int G,
                                                                    OutT* __restrict__ y) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t w = (int64_t)blockIdx.x * 32 + lane;
    if (w >= items || warp >= G) return;
    const int64_t ngr = C / G, inner = ppr * 8;
    const int64_t ip = w % ppr, og = w / ppr, cg = og % ngr, o = og / ngr;
    const int64_t pack0 = (o * C + cg * G) * ppr + ip;
    const float* sp = scale + (o * inner + ip * 8) * ngr + cg;
    float s[8];
#pragma unroll
    for (int l = 0; l < 8; ++l) s[l] = __ldg(sp + (int64_t)l * ngr);
    const uint2* qp = reinterpret_cast<const uint2*>(q);
    uint4* yp = reinterpret_cast<uint4*>(y);
    auto decode = [&](const uint2& codes) {
        float a[4], b[4];
        Int8Code::decode4(codes.x, a);
        Int8Code::decode4(codes.y, b);
        uint4 out;
        out.x = DTypeTraits<OutT>::float2_to_word(__fmul_rn(a[0], s[0]), __fmul_rn(a[1], s[1]));
        out.y = DTypeTraits<OutT>::float2_to_word(__fmul_rn(a[2], s[2]), __fmul_rn(a[3], s[3]));
        out.z = DTypeTraits<OutT>::float2_to_word(__fmul_rn(b[0], s[4]), __fmul_rn(b[1], s[5]));
        out.w = DTypeTraits<OutT>::float2_to_word(__fmul_rn(b[2], s[6]), __fmul_rn(b[3], s[7]));
        return out;
    };
    int j = warp;
    for (; j + 3 * kWarps < G; j += 4 * kWarps) {
        const int64_t p0 = pack0 + (int64_t)(j + 0 * kWarps) * ppr, p1 = pack0 + (int64_t)(j + 1 * kWarps) * ppr;
        const int64_t p2 = pack0 + (int64_t)(j + 2 * kWarps) * ppr, p3 = pack0 + (int64_t)(j + 3 * kWarps) * ppr;
        const uint2 c0 = ld_stream8(qp + p0), c1 = ld_stream8(qp + p1), c2 = ld_stream8(qp + p2), c3 = ld_stream8(qp + p3);
        st_stream16(yp + p0, decode(c0));
        st_stream16(yp + p1, decode(c1));
        st_stream16(yp + p2, decode(c2));
        st_stream16(yp + p3, decode(c3));
    }
    for (; j < G; j += kWarps) {
        const int64_t p = pack0 + (int64_t)j * ppr;
        st_stream16(yp + p, decode(ld_stream8(qp + p)));
    }
}

template <typename OutT>
__global__ void __launch_bounds__(kBlock) dequant_group_axis_scalar_kernel(const uint8_t* __restrict__ q,
                                                                           const float* __restrict__ scale, int64_t n,
                                                                           int64_t C, int64_t inner, int G,
                                                                           OutT* __restrict__ y) {
    pdl_wait();
    pdl_trigger();
    const int64_t ngr = C / G;
    for (int64_t e = (int64_t)blockIdx.x * kBlock + threadIdx.x; e < n; e += (int64_t)gridDim.x * kBlock) {
        const int64_t i = e % inner, oc = e / inner, c = oc % C, o = oc / C;
        const float s = __ldg(scale + (o * inner + i) * ngr + c / G);
        y[e] = DTypeTraits<OutT>::from_float(__fmul_rn(Int8Code::decode1(q[e]), s));
    }
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

inline unsigned grid_for(int64_t items, int ctas_per_sm) {
    const int64_t cap = (int64_t)sm_count() * ctas_per_sm;
    int64_t g = (items + kBlock - 1) / kBlock;
    if (g > cap) g = cap;
    return (unsigned)(g < 1 ? 1 : g);
}

template <typename T>
cudaError_t quant_t(const void* xv, int64_t outer, int64_t C, int64_t inner, int G, float eps, void* qv,
                    float* scale_out, cudaStream_t s) {
    constexpr int E = DTypeTraits<T>::kLanes;
    const T* x = static_cast<const T*>(xv);
    uint8_t* q = static_cast<uint8_t*>(qv);
    if (outer * C * inner <= 0) return cudaSuccess;
    if (inner % E == 0 && aligned_to(x, 16) && aligned_to(q, E == 8 ? 8 : 4)) {
        const int64_t ppr = inner / E, items = outer * (C / G) * ppr;
        const int64_t ctas = (items + 31) / 32;
        if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
        const int rows_per_thread = (G + kWarps - 1) / kWarps;
        if (rows_per_thread <= 4) quant_group_axis_kernel<T, 4><<<(unsigned)ctas, kBlock, 0, s>>>(x, items, C, ppr, G, eps, q, scale_out);
        else if (rows_per_thread <= 16) quant_group_axis_kernel<T, 16><<<(unsigned)ctas, kBlock, 0, s>>>(x, items, C, ppr, G, eps, q, scale_out);
        else quant_group_axis_kernel<T, 0><<<(unsigned)ctas, kBlock, 0, s>>>(x, items, C, ppr, G, eps, q, scale_out);
    } else {
        const int64_t items = outer * (C / G) * inner;
        quant_group_axis_scalar_kernel<T><<<grid_for(items, 8), kBlock, 0, s>>>(x, items, C, inner, G, eps, q, scale_out);
    }
    return cudaPeekAtLastError();
}

template <typename OutT>
cudaError_t dequant_t(const void* qv, const float* scale, int64_t outer, int64_t C, int64_t inner, int G, void* yv,
                      cudaStream_t s) {
    const uint8_t* q = static_cast<const uint8_t*>(qv);
    OutT* y = static_cast<OutT*>(yv);
    const int64_t n = outer * C * inner;
    if (n <= 0) return cudaSuccess;
    if (inner % 8 == 0 && aligned_to(q, 8) && aligned_to(y, 16)) {
        const int64_t ppr = inner / 8, items = outer * (C / G) * ppr, ctas = (items + 31) / 32;
        if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
        return launch_dependent(dequant_group_axis_kernel<OutT>, (unsigned)ctas, kBlock, 0, s, q, scale, items, C, ppr, G,
                                y);
    }
    return launch_dependent(dequant_group_axis_scalar_kernel<OutT>, grid_for(n, 8), kBlock, 0, s, q, scale, n, C, inner,
                            G, y);
}

}  // namespace

cudaError_t launch_quant_group_axis(const void* x, int dtype, int64_t outer, int64_t C, int64_t inner, int G, float eps,
                                    void* q, float* scale_out, cudaStream_t s) {
    switch (dtype) {
        case kF16: return quant_t<__half>(x, outer, C, inner, G, eps, q, scale_out, s);
        case kBF16: return quant_t<__nv_bfloat16>(x, outer, C, inner, G, eps, q, scale_out, s);
        case kF32: return quant_t<float>(x, outer, C, inner, G, eps, q, scale_out, s);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_dequant_group_axis(const void* q, const float* scale, int64_t outer, int64_t C, int64_t inner, int G,
                                      int out_dtype, void* y, cudaStream_t s) {
    if (out_dtype == kF16) return dequant_t<__half>(q, scale, outer, C, inner, G, y, s);
    if (out_dtype == kBF16) return dequant_t<__nv_bfloat16>(q, scale, outer, C, inner, G, y, s);
    return cudaErrorInvalidValue;
}

}  // namespace cb
