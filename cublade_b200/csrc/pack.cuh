// Pack vocabulary shared by every quantize / dequantize kernel in this library.
//
// One *pack* is 16 bytes of input: 8 half / bf16 lanes or 4 fp32 lanes, moved
// with a single 128-bit memory instruction.  `DTypeTraits<T>` holds the per
// dtype conversions, `Pack16<T>` aliases the 16 bytes as raw bits or lanes,
// and the free functions below turn a pack into quantized codes (or codes
// back into a pack).  It plays the role of the reference's
// cublade/kernels/cuda/quantization/fp8_pack.cuh:20-88 and int8_pack.cuh:23-100
// (DTypeTraits / Pack16 / Pack16Int8 / PackInT / LanesPerInt4 /
// round_half_even_clamp_int8), re-cut for kernels that keep several packs in
// flight per thread.
//
// Arithmetic contract (the bit-exactness gate):
//   * every product is a single fp32 multiply (no FMA contraction, no
//     fast-math, no flush-to-zero) -- build without --use_fast_math;
//   * reciprocal scales use IEEE round-to-nearest division (__fdiv_rn), which
//     equals the reference's "divide in fp64, narrow to fp32" route because a
//     quotient of two fp32 numbers needs at most 2*24+2 bits to be rounded
//     once correctly;
//   * INT8 codes: cvt.rni.s32.f32 then clamp to [-127, 127];
//   * FP8 codes:  cvt.rn.satfinite.e4m3x2.f32 on the fp32 product.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace cb {

constexpr float kInt8Qmax = 127.0f;
constexpr float kE4M3Qmax = 448.0f;

// ---------------------------------------------------------------------------
// DTypeTraits<T>: lanes per 16-byte pack and scalar conversions.
// ---------------------------------------------------------------------------
template <typename T>
struct DTypeTraits;

template <>
struct DTypeTraits<__half> {
    static constexpr int kLanes = 8;
    __device__ __forceinline__ static float to_float(__half v) { return __half2float(v); }
    __device__ __forceinline__ static __half from_float(float v) { return __float2half_rn(v); }
    // two lanes packed in one 32-bit word -> two fp32
    __device__ __forceinline__ static float2 word_to_float2(uint32_t w) {
        return __half22float2(*reinterpret_cast<const __half2*>(&w));
    }
    __device__ __forceinline__ static uint32_t float2_to_word(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

template <>
struct DTypeTraits<__nv_bfloat16> {
    static constexpr int kLanes = 8;
    __device__ __forceinline__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
    // bf16 is the top half of an fp32: widening is two integer ops, exact.
    __device__ __forceinline__ static float2 word_to_float2(uint32_t w) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
    __device__ __forceinline__ static uint32_t float2_to_word(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

template <>
struct DTypeTraits<float> {
    static constexpr int kLanes = 4;
    __device__ __forceinline__ static float to_float(float v) { return v; }
    __device__ __forceinline__ static float from_float(float v) { return v; }
};

// ---------------------------------------------------------------------------
// Pack16<T>: 16 bytes viewed as raw bits, 32-bit words, or lanes of T.
// ---------------------------------------------------------------------------
template <typename T>
union Pack16 {
    uint4 raw;
    uint32_t w[4];
    T lane[DTypeTraits<T>::kLanes];
};

// 16 quantized codes (int8 or e4m3) in one 128-bit word; 8 codes in 64 bits.
union Codes16 {
    uint4 raw;
    uint2 half8[2];
    uint8_t c[16];
};

// Unpack a pack into fp32 lanes (exact for every supported T).
template <typename T>
__device__ __forceinline__ void pack_to_floats(const uint4& raw, float (&f)[DTypeTraits<T>::kLanes]) {
    if constexpr (DTypeTraits<T>::kLanes == 4) {
        f[0] = __uint_as_float(raw.x);
        f[1] = __uint_as_float(raw.y);
        f[2] = __uint_as_float(raw.z);
        f[3] = __uint_as_float(raw.w);
    } else {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 p = DTypeTraits<T>::word_to_float2(w[k]);
            f[2 * k] = p.x;
            f[2 * k + 1] = p.y;
        }
    }
}

// Running max |lane|, NaN lanes dropped (both fmaxf and __hmax2 return the non-NaN operand).
// 16-bit types keep a packed pair of running maxima and compare two lanes per instruction:
// clearing the sign bits is one AND, the max is one packed min/max instruction.
template <typename T>
struct AbsMax;

template <>
struct AbsMax<float> {
    float m = 0.0f;
    __device__ __forceinline__ void update(const uint4& raw) {
        m = fmaxf(m, fmaxf(fmaxf(fabsf(__uint_as_float(raw.x)), fabsf(__uint_as_float(raw.y))),
                           fmaxf(fabsf(__uint_as_float(raw.z)), fabsf(__uint_as_float(raw.w)))));
    }
    __device__ __forceinline__ void update1(float v) { m = fmaxf(m, fabsf(v)); }
    __device__ __forceinline__ float finish() const { return m; }
};

template <>
struct AbsMax<__nv_bfloat16> {
    __nv_bfloat162 m2 = __nv_bfloat162(__ushort_as_bfloat16(0), __ushort_as_bfloat16(0));
    float m1 = 0.0f;
    __device__ __forceinline__ void word(uint32_t w) {
        w &= 0x7fff7fffu;
        m2 = __hmax2(m2, *reinterpret_cast<const __nv_bfloat162*>(&w));
    }
    __device__ __forceinline__ void update(const uint4& raw) { word(raw.x); word(raw.y); word(raw.z); word(raw.w); }
    __device__ __forceinline__ void update1(float v) { m1 = fmaxf(m1, fabsf(v)); }
    __device__ __forceinline__ float finish() const {
        return fmaxf(m1, fmaxf(__bfloat162float(__low2bfloat16(m2)), __bfloat162float(__high2bfloat16(m2))));
    }
};

template <>
struct AbsMax<__half> {
    __half2 m2 = __half2(__ushort_as_half(0), __ushort_as_half(0));
    float m1 = 0.0f;
    __device__ __forceinline__ void word(uint32_t w) {
        w &= 0x7fff7fffu;
        m2 = __hmax2(m2, *reinterpret_cast<const __half2*>(&w));
    }
    __device__ __forceinline__ void update(const uint4& raw) { word(raw.x); word(raw.y); word(raw.z); word(raw.w); }
    __device__ __forceinline__ void update1(float v) { m1 = fmaxf(m1, fabsf(v)); }
    __device__ __forceinline__ float finish() const {
        return fmaxf(m1, fmaxf(__half2float(__low2half(m2)), __half2float(__high2half(m2))));
    }
};

// Warp-shuffle max over WIDTH adjacent lanes (WIDTH a power of two <= 32).
template <int WIDTH>
__device__ __forceinline__ float team_max(float v) {
#pragma unroll
    for (int off = WIDTH / 2; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// ---------------------------------------------------------------------------
// Scalar code conversions.
// ---------------------------------------------------------------------------
// round-half-even then clamp to the symmetric range; NaN -> 0 (cvt.rni of NaN).
__device__ __forceinline__ int round_half_even_clamp_int8(float v) {
    int r = __float2int_rn(v);
    r = max(r, -127);
    r = min(r, 127);
    return r;
}

__device__ __forceinline__ uint8_t float_to_e4m3(float v) {
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float e4m3_to_float(uint8_t c) {
    __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&hr));
}

// ---------------------------------------------------------------------------
// Whole-pack conversions.  Code kinds.
// ---------------------------------------------------------------------------
// d = (c << 16) | (sat_s8(a) << 8) | sat_s8(b)
__device__ __forceinline__ uint32_t cvt_pack_s8(int a, int b, uint32_t c) {
    uint32_t d;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// CLAMP_LOW: also clamp at -127.  When the multiplier is 127 / max(amax, eps) with amax the true
// maximum of the data, |x * inv| <= 127 * (1 + 2^-24)^2 < 127.5, so the rounded value is already
// inside [-127, 127] (NaN converts to 0) and the saturating pack alone reproduces the reference's
// clamp; a caller-supplied amax (split-phase entry point) needs the explicit lower clamp.
template <bool CLAMP_LOW>
struct Int8CodeT {
    static constexpr float kQmax = kInt8Qmax;
    __device__ __forceinline__ static uint32_t encode4(float a, float b, float c, float d) {
        int ia = __float2int_rn(a), ib = __float2int_rn(b), ic = __float2int_rn(c), id = __float2int_rn(d);
        if constexpr (CLAMP_LOW) {
            ia = max(ia, -127); ib = max(ib, -127); ic = max(ic, -127); id = max(id, -127);
        }
        return cvt_pack_s8(ib, ia, cvt_pack_s8(id, ic, 0u));
    }
    __device__ __forceinline__ static uint8_t encode1(float a) { return (uint8_t)round_half_even_clamp_int8(a); }
    // four codes in one word -> four fp32, exactly: the byte (biased by 128) is dropped into the
    // mantissa of 2^23 and the bias subtracted, one permute and one add per lane.
    __device__ __forceinline__ static void decode4(uint32_t w, float (&f)[4]) {
        const uint32_t u = w ^ 0x80808080u;
        f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
        f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
        f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
        f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
    }
    __device__ __forceinline__ static float decode1(uint8_t c) { return (float)(int)(int8_t)c; }
};
using Int8Code = Int8CodeT<false>;
using Int8CodeClamped = Int8CodeT<true>;

struct E4M3Code {
    static constexpr float kQmax = kE4M3Qmax;
    __device__ __forceinline__ static uint32_t encode4(float a, float b, float c, float d) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
        return lo | (hi << 16);
    }
    __device__ __forceinline__ static uint8_t encode1(float a) { return float_to_e4m3(a); }
    __device__ __forceinline__ static void decode4(uint32_t w, float (&f)[4]) {
        __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xffffu), __NV_E4M3);
        __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
        float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
        float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
    }
    __device__ __forceinline__ static float decode1(uint8_t c) { return e4m3_to_float(c); }
};

// Quantize one pack: lanes * inv -> codes.  16-bit inputs give 8 codes (uint2),
// fp32 inputs give 4 codes (one word, returned in .x).
template <typename T, typename Code>
__device__ __forceinline__ uint2 pack_encode(const uint4& raw, float inv) {
    constexpr int L = DTypeTraits<T>::kLanes;
    float f[L];
    pack_to_floats<T>(raw, f);
#pragma unroll
    for (int k = 0; k < L; ++k) f[k] = __fmul_rn(f[k], inv);
    uint2 out;
    out.x = Code::encode4(f[0], f[1], f[2], f[3]);
    if constexpr (L == 8) out.y = Code::encode4(f[4], f[5], f[6], f[7]);
    else out.y = 0u;
    return out;
}

// Dequantize 8 codes (uint2) into one 16-byte pack of OutT (half / bf16).
template <typename OutT, typename Code>
__device__ __forceinline__ uint4 codes_decode8(const uint2& codes, float s) {
    float a[4], b[4];
    Code::decode4(codes.x, a);
    Code::decode4(codes.y, b);
    uint4 out;
    out.x = DTypeTraits<OutT>::float2_to_word(__fmul_rn(a[0], s), __fmul_rn(a[1], s));
    out.y = DTypeTraits<OutT>::float2_to_word(__fmul_rn(a[2], s), __fmul_rn(a[3], s));
    out.z = DTypeTraits<OutT>::float2_to_word(__fmul_rn(b[0], s), __fmul_rn(b[1], s));
    out.w = DTypeTraits<OutT>::float2_to_word(__fmul_rn(b[2], s), __fmul_rn(b[3], s));
    return out;
}

// The two numbers every quantizer derives from an amax:
//   inv   = qmax / max(amax, eps)   (what the codes are multiplied by)
//   scale = 1 / inv                 (what dequantize multiplies by; NOT amax/qmax)
// Reference: quantize_per_tensor_fp8.cu:99-102, quantize_int8.cu:120-126.
struct InvScale {
    float inv;
    float scale;
};
template <typename Code>
__device__ __forceinline__ InvScale inv_and_scale(float amax, float eps) {
    InvScale r;
    r.inv = __fdiv_rn(Code::kQmax, fmaxf(amax, eps));
    r.scale = __fdiv_rn(1.0f, r.inv);
    return r;
}

// 256-bit global store (sm_100): one full 32-byte sector per thread per instruction.
__device__ __forceinline__ void st_stream32(void* p, const uint4& lo, const uint4& hi) {
    asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(lo.x), "r"(lo.y), "r"(lo.z),
                 "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                 : "memory");
}

// Streaming 128-bit / 64-bit / 32-bit global accesses.
__device__ __forceinline__ uint4 ld_stream16(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint4 ld_keep16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ld_stream8(const void* p) { return __ldcs(reinterpret_cast<const uint2*>(p)); }
__device__ __forceinline__ void st_stream16(void* p, uint4 v) { __stcs(reinterpret_cast<uint4*>(p), v); }
__device__ __forceinline__ void st_stream8(void* p, uint2 v) { __stcs(reinterpret_cast<uint2*>(p), v); }
__device__ __forceinline__ void st_stream4(void* p, uint32_t v) { __stcs(reinterpret_cast<uint32_t*>(p), v); }

}  // namespace cb
