// Fused RMSNorm -> per-row (per-token) quantize, one pass over x.
//
// The reference names this op as the purpose of its DTypeTraits / Pack16 headers
// ("upcoming RMSNorm-fused-quant work", README.md:20) but does not contain it; unfused, the
// chain costs 7 bytes per element (RMSNorm 2 in + 2 out, per-row quantize 2 in + 1 out).  Here
// a team of threads keeps the row in registers from the first load to the last store, so the
// chain costs 3 bytes per element (2 in, 1 out) -- the same structure as quant_segments_kernel
// (quant.cu) with a normalisation between the load and the amax.
//
// Arithmetic, per row of H elements of type T (fp16 / bf16), all intermediates fp32:
//   ss    = sum_i x_i^2                      (tree order of this kernel; see note)
//   r     = 1 / sqrt(ss / H + rms_eps)       (IEEE division, IEEE reciprocal square root)
//   n_i   = T(x_i * r)                       (rounded to T like an unfused RMSNorm's output)
//   y_i   = T(float(n_i) * float(g_i))       (skipped when there is no weight vector g)
//   amax  = max_i |y_i|;  inv = qmax / max(amax, q_eps);  q_i = code(float(y_i) * inv);  scale = 1 / inv
// so, given r, codes and scale are bit-identical to "RMSNorm, then per-channel quantize of its
// output" (quantize_int8.cu:173-297 for the second half).  Note: ss is a floating-point sum, its
// last bits depend on the order of additions, and r inherits that.
#include "launch.h"
#include "pack.cuh"

namespace cb {

namespace {

constexpr int kBlock = 256;

template <int WIDTH>
__device__ __forceinline__ float team_sum(float v) {
#pragma unroll
    for (int off = WIDTH / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// CTA-wide sum / max over 256 threads; `red` holds 8 floats; result valid in every thread
template <bool IS_MAX>
__device__ __forceinline__ float block_reduce(float v, float* red) {
    v = IS_MAX ? team_max<32>(v) : team_sum<32>(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = lane < kBlock / 32 ? red[lane] : 0.0f;
    r = IS_MAX ? team_max<8>(r) : team_sum<8>(r);
    r = __shfl_sync(0xffffffffu, r, 0);
    __syncthreads();
    return r;
}

// the same for N values at once (one pair of barriers for all of them); `red` holds N x 8 floats
template <bool IS_MAX, int N>
__device__ __forceinline__ void block_reduce_n(float (&v)[N], float (*red)[kBlock / 32]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        v[i] = IS_MAX ? team_max<32>(v[i]) : team_sum<32>(v[i]);
        if (lane == 0) red[i][warp] = v[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < N; ++i) {
        float r = lane < kBlock / 32 ? red[i][lane] : 0.0f;
        r = IS_MAX ? team_max<8>(r) : team_sum<8>(r);
        v[i] = __shfl_sync(0xffffffffu, r, 0);
    }
    __syncthreads();
}

__device__ __forceinline__ float inv_rms(float ss, int64_t H, float rms_eps) {
    return __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)H), rms_eps));
}

// one pack of x (8 lanes of T) -> sum of squares
template <typename T>
__device__ __forceinline__ float pack_sumsq(const uint4& raw) {
    float f[8];
    pack_to_floats<T>(raw, f);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s = __fmaf_rn(f[k], f[k], s);
    return s;
}

// two lanes times two lanes in T: the product of two 16-bit floats is exact in fp32 (at most 22 significant
// bits), so the packed multiply's single rounding equals "widen, multiply in fp32, round to T"
__device__ __forceinline__ uint32_t mul2(__half, uint32_t a, uint32_t b) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t mul2(__nv_bfloat16, uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// normalise one pack in place: y = T(T(x * r) * g)
template <typename T, bool HAS_G>
__device__ __forceinline__ uint4 pack_normalise(const uint4& raw, float r, const uint4& graw) {
    float f[8];
    pack_to_floats<T>(raw, f);
    const uint32_t g[4] = {graw.x, graw.y, graw.z, graw.w};
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        w[k] = DTypeTraits<T>::float2_to_word(__fmul_rn(f[2 * k], r), __fmul_rn(f[2 * k + 1], r));
        if constexpr (HAS_G) w[k] = mul2(T(), w[k], g[k]);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// A TEAM of threads (32 lanes of a warp, or a whole 256-thread CTA) owns ROWS rows at a time; thread t holds
// packs t, t + TEAM, ... (PACKS of them) of each row in registers.  Needs H % 8 == 0 and 16-byte aligned rows.
// ROWS = 2 halves the number of CTA barriers per row (the two rows' sums and maxima travel through the
// same reductions) and loads the gain once for both.
template <typename T, typename Code, int TEAM, int PACKS, int ROWS, bool HAS_G>
__global__ void __launch_bounds__(kBlock, ROWS * PACKS <= 2 ? 6 : (ROWS * PACKS <= 4 ? 5 : 2)) rmsnorm_quant_rows_kernel(const T* __restrict__ x, int64_t rows, int npk,
                                                                    const T* __restrict__ gamma, float rms_eps,
                                                                    float q_eps, uint8_t* __restrict__ q,
                                                                    float* __restrict__ scale_out,
                                                                    T* __restrict__ y_out, float* __restrict__ rstd_out) {
    constexpr int kTeamsPerCta = kBlock / TEAM;
    const int t = threadIdx.x % TEAM;
    const int64_t row0 = ((int64_t)blockIdx.x * kTeamsPerCta + threadIdx.x / TEAM) * ROWS;
    const uint4* gp = reinterpret_cast<const uint4*>(gamma);
    __shared__ float red[ROWS][kBlock / 32];

    uint4 v[ROWS][PACKS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const uint4* xp = reinterpret_cast<const uint4*>(x) + (row0 + r) * (int64_t)npk;
#pragma unroll
        for (int k = 0; k < PACKS; ++k) {
            const int p = t + k * TEAM;
            v[r][k] = (row0 + r < rows && p < npk) ? ld_stream16(xp + p) : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    float ss[ROWS], r_inv[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        ss[r] = 0.0f;
#pragma unroll
        for (int k = 0; k < PACKS; ++k) ss[r] += pack_sumsq<T>(v[r][k]);
    }
    if constexpr (TEAM <= 32) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) ss[r] = team_sum<TEAM>(ss[r]);
    } else {
        block_reduce_n<false, ROWS>(ss, red);
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        r_inv[r] = inv_rms(ss[r], (int64_t)npk * 8, rms_eps);
        if (rstd_out && row0 + r < rows && t == 0) rstd_out[row0 + r] = r_inv[r];
    }

    float m[ROWS];
    AbsMax<T> am[ROWS];
#pragma unroll
    for (int k = 0; k < PACKS; ++k) {
        const int p = t + k * TEAM;
        uint4 g = make_uint4(0u, 0u, 0u, 0u);
        if constexpr (HAS_G) {
            if (p < npk) g = ld_keep16(gp + p);  // the gain: 2 * H bytes shared by every row, served by L1 / L2
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            v[r][k] = pack_normalise<T, HAS_G>(v[r][k], r_inv[r], g);  // packs beyond the row stay zero
            am[r].update(v[r][k]);
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) m[r] = am[r].finish();
    if constexpr (TEAM <= 32) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) m[r] = team_max<TEAM>(m[r]);
    } else {
        block_reduce_n<true, ROWS>(m, red);
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int64_t row = row0 + r;
        if (row >= rows) continue;
        const InvScale is = inv_and_scale<Code>(m[r], q_eps);
        if (t == 0) scale_out[row] = is.scale;
        uint8_t* qp = q + row * (int64_t)npk * 8;
        uint4* yp = y_out ? reinterpret_cast<uint4*>(y_out) + row * (int64_t)npk : nullptr;
#pragma unroll
        for (int k = 0; k < PACKS; ++k) {
            const int p = t + k * TEAM;
            if (p < npk) {
                st_stream8(qp + (int64_t)p * 8, pack_encode<T, Code>(v[r][k], is.inv));
                if (yp) st_stream16(yp + p, v[r][k]);
            }
        }
    }
}

// Any H, any alignment: one CTA per row, scalar accesses, the row is read three times (the second
// and third time from L1 / L2).
template <typename T, typename Code>
__global__ void __launch_bounds__(kBlock) rmsnorm_quant_scalar_kernel(const T* __restrict__ x, int64_t H,
                                                                      const T* __restrict__ gamma, float rms_eps,
                                                                      float q_eps, uint8_t* __restrict__ q,
                                                                      float* __restrict__ scale_out,
                                                                      T* __restrict__ y_out, float* __restrict__ rstd_out) {
    const int64_t row = blockIdx.x;
    const T* xs = x + row * H;
    __shared__ float red[kBlock / 32];
    float ss = 0.0f;
    for (int64_t i = threadIdx.x; i < H; i += kBlock) {
        const float f = DTypeTraits<T>::to_float(xs[i]);
        ss = __fmaf_rn(f, f, ss);
    }
    ss = block_reduce<false>(ss, red);
    const float r = inv_rms(ss, H, rms_eps);
    if (rstd_out && threadIdx.x == 0) rstd_out[row] = r;
    auto normalised = [&](int64_t i) {
        T n = DTypeTraits<T>::from_float(__fmul_rn(DTypeTraits<T>::to_float(xs[i]), r));
        if (gamma) n = DTypeTraits<T>::from_float(__fmul_rn(DTypeTraits<T>::to_float(n), DTypeTraits<T>::to_float(gamma[i])));
        return n;
    };
    float m = 0.0f;
    for (int64_t i = threadIdx.x; i < H; i += kBlock) m = fmaxf(m, fabsf(DTypeTraits<T>::to_float(normalised(i))));
    m = block_reduce<true>(m, red);
    const InvScale is = inv_and_scale<Code>(m, q_eps);
    if (threadIdx.x == 0) scale_out[row] = is.scale;
    for (int64_t i = threadIdx.x; i < H; i += kBlock) {
        const T n = normalised(i);
        q[row * H + i] = Code::encode1(__fmul_rn(DTypeTraits<T>::to_float(n), is.inv));
        if (y_out) y_out[row * H + i] = n;
    }
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

template <typename T, typename Code, int TEAM, int PACKS>
void launch_rows(const T* x, int64_t rows, int npk, const T* gamma, float rms_eps, float q_eps, uint8_t* q,
                 float* scale_out, T* y_out, float* rstd_out, cudaStream_t s) {
    // measured on B200 (16384 x 8192 bf16): two rows per team (half the barriers per row) is no faster than
    // one and costs registers; what matters is occupancy -- 96 registers held the kernel to 2 CTAs per SM
    constexpr int ROWS = 1;
    constexpr int kRowsPerCta = kBlock / TEAM * ROWS;
    const unsigned grid = (unsigned)((rows + kRowsPerCta - 1) / kRowsPerCta);
    if (gamma) rmsnorm_quant_rows_kernel<T, Code, TEAM, PACKS, ROWS, true><<<grid, kBlock, 0, s>>>(
        x, rows, npk, gamma, rms_eps, q_eps, q, scale_out, y_out, rstd_out);
    else rmsnorm_quant_rows_kernel<T, Code, TEAM, PACKS, ROWS, false><<<grid, kBlock, 0, s>>>(
        x, rows, npk, gamma, rms_eps, q_eps, q, scale_out, y_out, rstd_out);
}

template <typename T, typename Code>
cudaError_t rmsnorm_quant_t(const void* xv, int64_t rows, int64_t H, const void* gv, float rms_eps, float q_eps,
                            void* qv, float* scale_out, void* yv, float* rstd_out, cudaStream_t s) {
    if (rows <= 0 || H <= 0) return cudaSuccess;
    if (rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    const T* x = static_cast<const T*>(xv);
    const T* gamma = static_cast<const T*>(gv);
    uint8_t* q = static_cast<uint8_t*>(qv);
    T* y = static_cast<T*>(yv);
    const bool vec_ok = H % 8 == 0 && H <= (int64_t)kBlock * 8 * 8 && aligned_to(x, 16) && aligned_to(q, 8) &&
                        (!gamma || aligned_to(gamma, 16)) && (!y || aligned_to(y, 16));
    if (!vec_ok) {
        rmsnorm_quant_scalar_kernel<T, Code><<<(unsigned)rows, kBlock, 0, s>>>(x, H, gamma, rms_eps, q_eps, q, scale_out, y,
                                                                               rstd_out);
        return cudaPeekAtLastError();
    }
    const int npk = (int)(H / 8);
    // a warp per row up to 1024 elements, a CTA per row up to 16 384
    if (npk <= 32) launch_rows<T, Code, 32, 1>(x, rows, npk, gamma, rms_eps, q_eps, q, scale_out, y, rstd_out, s);
    else if (npk <= 64) launch_rows<T, Code, 32, 2>(x, rows, npk, gamma, rms_eps, q_eps, q, scale_out, y, rstd_out, s);
    else if (npk <= 128) launch_rows<T, Code, 32, 4>(x, rows, npk, gamma, rms_eps, q_eps, q, scale_out, y, rstd_out, s);
    else if (npk <= 256) launch_rows<T, Code, kBlock, 1>(x, rows, npk, gamma, rms_eps, q_eps, q, scale_out, y, rstd_out, s);
    else if (npk <= 512) launch_rows<T, Code, kBlock, 2>(x, rows, npk, gamma, rms_eps, q_eps, q, scale_out, y, rstd_out, s);
    else if (npk <= 1024) launch_rows<T, Code, kBlock, 4>(x, rows, npk, gamma, rms_eps, q_eps, q, scale_out, y, rstd_out, s);
    else launch_rows<T, Code, kBlock, 8>(x, rows, npk, gamma, rms_eps, q_eps, q, scale_out, y, rstd_out, s);
    return cudaPeekAtLastError();
}

}  // namespace

cudaError_t launch_rmsnorm_quant(const void* x, int dtype, int64_t rows, int64_t H, const void* gamma, float rms_eps,
                                 float q_eps, int code, void* q, float* scale_out, void* y_out, float* rstd_out,
                                 cudaStream_t s) {
    if (code == kCodeInt8) {
        if (dtype == kF16) return rmsnorm_quant_t<__half, Int8Code>(x, rows, H, gamma, rms_eps, q_eps, q, scale_out, y_out, rstd_out, s);
        if (dtype == kBF16)
            return rmsnorm_quant_t<__nv_bfloat16, Int8Code>(x, rows, H, gamma, rms_eps, q_eps, q, scale_out, y_out, rstd_out, s);
    } else if (code == kCodeE4M3) {
        if (dtype == kF16) return rmsnorm_quant_t<__half, E4M3Code>(x, rows, H, gamma, rms_eps, q_eps, q, scale_out, y_out, rstd_out, s);
        if (dtype == kBF16)
            return rmsnorm_quant_t<__nv_bfloat16, E4M3Code>(x, rows, H, gamma, rms_eps, q_eps, q, scale_out, y_out, rstd_out, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cb
