// W8A16 linear, weight-streaming kernel for skinny activations (decode shapes).
//
//   y[m, n] = (sum_k x[m, k] * wq[n, k]) * scale[n] + sum_j xo[m, j] * wo[n, j] + bias[n]
//
// For M <= 64 the op is bound by streaming the N*K int8 weights from HBM once,
// so the kernel is built around that stream: each warp owns 16 weight rows and
// a slice of K, pulls its int8 rows straight from global memory into registers
// with 128-bit loads (no shared-memory staging, no transpose, no bf16 copy of
// the weights -- the reference materialises both, cublade/quantization/linear.py:123-126
// and cublade/bindings/triton/matmul.py:20-21), widens them to 16-bit floats in
// registers and feeds warp-level mma.m16n8k16 with the weights as the 16-row
// operand and up to 64 activation rows as the 8-column operand(s).
//
// The k index inside one 16-wide mma step is a free permutation as long as
// both operands use the same one, so a thread's 16 contiguous weight bytes
// (k = 16t .. 16t+15 of a 64-wide block, t = lane % 4) serve four mma steps
// and the matching activations are its own 32 contiguous bytes of x.
//
// Four warps of a CTA split K four ways for one 16-row tile and reduce through
// shared memory; the epilogue applies the per-row scale, adds the 16-bit side
// product over the outlier columns and the bias, rounds in the reference's places, and stores.

#include "launch.h"
#include "pack.cuh"

namespace cb {

namespace {

constexpr int kWarps = 4;

template <typename A>
struct Act;
template <>
struct Act<__nv_bfloat16> {
    // four int8 codes (one word) -> two words of bf16 pairs (c0,c1) (c2,c3)
    __device__ __forceinline__ static void widen4(uint32_t c, uint32_t& lo, uint32_t& hi) {
        // bf16 magic in packed arithmetic, exact: with b the code's byte, P = 0x4300 | b per 16-bit lane;
        // A = P with bit 7 cleared = 128 + (b & 127), C = P with only bit 7 kept = 128 or 256 (both exact bf16),
        // and A - C = b for b < 128, b - 256 otherwise: the signed code, an integer of magnitude <= 128 that
        // bf16 holds exactly, so the packed subtraction rounds nothing.  Two permutes, four logic ops and two
        // packed subtractions per four codes (the fp32 route took eleven instructions).
        const uint32_t p01 = __byte_perm(c, 0x43434343u, 0x4140), p23 = __byte_perm(c, 0x43434343u, 0x4342);
        const uint32_t a01 = p01 & 0xFF7FFF7Fu, c01 = p01 & 0xFF80FF80u;
        const uint32_t a23 = p23 & 0xFF7FFF7Fu, c23 = p23 & 0xFF80FF80u;
        const __nv_bfloat162 d01 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&a01), *reinterpret_cast<const __nv_bfloat162*>(&c01));
        const __nv_bfloat162 d23 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&a23), *reinterpret_cast<const __nv_bfloat162*>(&c23));
        lo = *reinterpret_cast<const uint32_t*>(&d01);
        hi = *reinterpret_cast<const uint32_t*>(&d23);
    }
    __device__ __forceinline__ static void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ __forceinline__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Act<__half> {
    __device__ __forceinline__ static void widen4(uint32_t c, uint32_t& lo, uint32_t& hi) {
        // fp16 magic: 0x6400 | (code ^ 0x80) = 1024 + code + 128; subtract 1152 (exact in fp16).
        const uint32_t u = c ^ 0x80808080u;
        const uint32_t p0 = __byte_perm(u, 0x64006400u, 0x7150);  // bytes: u0, 0x64, u1, 0x64
        const uint32_t p1 = __byte_perm(u, 0x64006400u, 0x7352);
        const __half2 k = __half2half2(__ushort_as_half((unsigned short)0x6480));  // 1152.0
        __half2 a = __hsub2(*reinterpret_cast<const __half2*>(&p0), k);
        __half2 b = __hsub2(*reinterpret_cast<const __half2*>(&p1), k);
        lo = *reinterpret_cast<uint32_t*>(&a);
        hi = *reinterpret_cast<uint32_t*>(&b);
    }
    __device__ __forceinline__ static void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ __forceinline__ static float to_float(__half v) { return __half2float(v); }
    __device__ __forceinline__ static __half from_float(float v) { return __float2half_rn(v); }
};

// v rounded to the activation type and widened back: the epilogues below round where the reference's
// forward materialises a 16-bit tensor (after the GEMM, after the scales, after adding the outlier
// product, after the bias; cublade/quantization/linear.py:97-135), so results agree with it bit for
// bit up to the order of the fp32 accumulation.
template <typename A>
__device__ __forceinline__ float ref_round(float v) { return Act<A>::to_float(Act<A>::from_float(v)); }

__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
    if (dtype == kF32) return static_cast<const float*>(p)[i];
    if (dtype == kBF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    return __half2float(static_cast<const __half*>(p)[i]);
}

struct StreamParams {
    const void* x;
    int64_t M, K, ldx;
    const int8_t* wq;
    int64_t N;
    const void* scales;
    int scales_dtype;
    const void* bias;
    int bias_dtype;
    const void* xo;
    const void* wo;
    int64_t KO, ldxo;
    void* y;
    int64_t ldy;
    int64_t m0;  // first activation row of this pass
    int weights_ready;  // 1: the first stage of weights may be fetched before waiting for the kernel ahead
};

// One 16-byte (VEC==16) / 8 / 4 / 1-byte-granular load of weight codes for row `r`, k in [k, k+VEC').
// Returns the bytes as words; out-of-range parts are zero.
template <int VEC>
__device__ __forceinline__ void load_codes(const int8_t* __restrict__ row, int64_t k, int64_t K, bool row_ok,
                                           uint32_t (&w)[VEC >= 4 ? VEC / 4 : 1]) {
    constexpr int NW = VEC >= 4 ? VEC / 4 : 1;
#pragma unroll
    for (int i = 0; i < NW; ++i) w[i] = 0u;
    if (!row_ok) return;
    if constexpr (VEC == 16) {
        if (k + 16 <= K) {
            const uint4 v = __ldcs(reinterpret_cast<const uint4*>(row + k));
            w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
        }
    } else if constexpr (VEC == 8) {
        if (k + 8 <= K) {
            const uint2 v = __ldcs(reinterpret_cast<const uint2*>(row + k));
            w[0] = v.x; w[1] = v.y;
        }
    } else if constexpr (VEC == 4) {
        if (k + 4 <= K) w[0] = __ldcs(reinterpret_cast<const uint32_t*>(row + k));
    } else {
#pragma unroll
        for (int b = 0; b < 4; ++b)
            if (k + b < K) w[0] |= (uint32_t)(uint8_t)row[k + b] << (8 * b);
    }
}

// Activations for the same k range: VEC' elements of 2 bytes -> words of pairs.
template <typename A, int VEC>
__device__ __forceinline__ void load_acts(const A* __restrict__ row, int64_t k, int64_t K, bool row_ok,
                                          uint32_t (&w)[VEC >= 4 ? VEC / 2 : 2]) {
    constexpr int NW = VEC >= 4 ? VEC / 2 : 2;
#pragma unroll
    for (int i = 0; i < NW; ++i) w[i] = 0u;
    if (!row_ok) return;
    if constexpr (VEC == 16) {
        if (k + 16 <= K) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(row + k));
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(row + k + 8));
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
            w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        }
    } else if constexpr (VEC == 8) {
        if (k + 8 <= K) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(row + k));
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
        }
    } else if constexpr (VEC == 4) {
        if (k + 4 <= K) {
            const uint2 a = __ldg(reinterpret_cast<const uint2*>(row + k));
            w[0] = a.x; w[1] = a.y;
        }
    } else {
        const unsigned short* r16 = reinterpret_cast<const unsigned short*>(row);
#pragma unroll
        for (int b = 0; b < 4; ++b)
            if (k + b < K) w[b / 2] |= (uint32_t)r16[k + b] << (16 * (b & 1));
    }
}

// VEC: bytes of weight codes a thread loads at once (16, 8, 4) or 1 for the
// byte-wise path that accepts any K / alignment.  MT: activation 8-row tiles.
template <typename A, int VEC, int MT>
__global__ void __launch_bounds__(kWarps * 32) w8a16_stream_kernel(const StreamParams p) {
    constexpr int KSTEP = VEC >= 4 ? VEC * 4 : 16;   // k covered by a warp per load round
    constexpr int NSTEP = VEC >= 4 ? VEC / 4 : 1;    // mma k16-steps per load round
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t n0 = (int64_t)blockIdx.x * 16;
    const A* x = static_cast<const A*>(p.x);

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    const bool r0_ok = n0 + g < p.N, r1_ok = n0 + g + 8 < p.N;
    const int8_t* w0 = p.wq + (n0 + g) * p.K;
    const int8_t* w1 = p.wq + (n0 + g + 8) * p.K;
    const int kper = VEC >= 4 ? VEC : 4;

    // This warp's K slice: rounds of KSTEP, dealt to the four warps in groups of U rounds.  The
    // loop is software-pipelined over two register stages: the loads of the next group (weights,
    // and the activations too when they fit in registers) are issued before the current group is
    // widened and multiplied, so HBM latency overlaps the arithmetic inside each warp.
    constexpr int U = 2;
    constexpr int CW = VEC >= 4 ? VEC / 4 : 1;
    constexpr int XW = VEC >= 4 ? VEC / 2 : 2;
    constexpr bool kPrefetchX = MT <= 2;
    struct Stage {
        uint32_t c0[U][CW], c1[U][CW];
        uint32_t xa[kPrefetchX ? U : 1][kPrefetchX ? MT : 1][XW];
    };
    const int64_t nrounds = (p.K + KSTEP - 1) / KSTEP;
    auto load_stage = [&](Stage& st, int64_t r) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool valid = (r + u) < nrounds;
            const int64_t k = (r + u) * KSTEP + (int64_t)t * kper;
            load_codes<VEC>(w0, k, p.K, r0_ok && valid, st.c0[u]);
            load_codes<VEC>(w1, k, p.K, r1_ok && valid, st.c1[u]);
            if constexpr (kPrefetchX) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int64_t m = p.m0 + mt * 8 + g;
                    load_acts<A, VEC>(x + m * p.ldx, k, p.K, valid && m < p.M, st.xa[u][mt]);
                }
            }
        }
    };
    auto compute_stage = [&](Stage& st, int64_t r) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if ((r + u) >= nrounds) continue;
            uint32_t xl[kPrefetchX ? 1 : MT][XW];
            if constexpr (!kPrefetchX) {
                const int64_t k = (r + u) * KSTEP + (int64_t)t * kper;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int64_t m = p.m0 + mt * 8 + g;
                    load_acts<A, VEC>(x + m * p.ldx, k, p.K, m < p.M, xl[mt]);
                }
            }
#pragma unroll
            for (int s = 0; s < NSTEP; ++s) {
                uint32_t a[4];
                Act<A>::widen4(st.c0[u][s], a[0], a[2]);
                Act<A>::widen4(st.c1[u][s], a[1], a[3]);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    if constexpr (kPrefetchX) Act<A>::mma(acc[mt], a, st.xa[u][mt][2 * s], st.xa[u][mt][2 * s + 1]);
                    else Act<A>::mma(acc[mt], a, xl[mt][2 * s], xl[mt][2 * s + 1]);
                }
            }
        }
    };
    {
        Stage st0, st1;
        int64_t r = (int64_t)warp * U;
        const int64_t step = (int64_t)kWarps * U;
        // this variant's stages hold activations as well, so it waits for the kernel ahead before its first load
        pdl_wait();
        pdl_trigger();
        load_stage(st0, r);
        while (r < nrounds) {
            load_stage(st1, r + step);
            compute_stage(st0, r);
            r += step;
            if (r >= nrounds) break;
            load_stage(st0, r + step);
            compute_stage(st1, r);
            r += step;
        }
    }

    // cross-warp reduction of the K split
    __shared__ float red[kWarps - 1][MT * 4][32];
    if (warp > 0) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) red[warp - 1][mt * 4 + j][lane] = acc[mt][j];
    }
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int w = 0; w < kWarps - 1; ++w)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[mt][j] += red[w][mt * 4 + j][lane];

    // GEMM output and its product with the per-row scale (rows g and g+8 of this tile), each rounded
    // to the activation type as in the reference
    const float s0 = r0_ok ? ref_round<A>(load_as_float(p.scales, p.scales_dtype, n0 + g)) : 0.0f;
    const float s1 = r1_ok ? ref_round<A>(load_as_float(p.scales, p.scales_dtype, n0 + g + 8)) : 0.0f;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        acc[mt][0] = ref_round<A>(ref_round<A>(acc[mt][0]) * s0); acc[mt][1] = ref_round<A>(ref_round<A>(acc[mt][1]) * s0);
        acc[mt][2] = ref_round<A>(ref_round<A>(acc[mt][2]) * s1); acc[mt][3] = ref_round<A>(ref_round<A>(acc[mt][3]) * s1);
    }

    // 16-bit side product over the outlier columns (few: this warp alone), rounded, then added
    if (p.KO > 0) {
        const A* xo = static_cast<const A*>(p.xo);
        const A* wo = static_cast<const A*>(p.wo);
        float side[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) side[mt][j] = 0.0f;
        const int64_t osteps = (p.KO + 15) / 16;
        for (int64_t st = 0; st < osteps; ++st) {
            const int64_t k = st * 16 + t * 4;
            uint32_t a0[2], a1[2];
            load_acts<A, 1>(wo + (n0 + g) * p.KO, k, p.KO, r0_ok, a0);
            load_acts<A, 1>(wo + (n0 + g + 8) * p.KO, k, p.KO, r1_ok, a1);
            const uint32_t a[4] = {a0[0], a1[0], a0[1], a1[1]};
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int64_t m = p.m0 + mt * 8 + g;
                uint32_t b[2];
                load_acts<A, 1>(xo + m * p.ldxo, k, p.KO, m < p.M, b);
                Act<A>::mma(side[mt], a, b[0], b[1]);
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[mt][j] = ref_round<A>(acc[mt][j] + ref_round<A>(side[mt][j]));
    }

    // D fragment: acc[mt][0..1] -> (row g, m = 2t, 2t+1), acc[mt][2..3] -> (row g+8, same m)
    A* y = static_cast<A*>(p.y);
    const bool has_bias = p.bias != nullptr;
    const float b0 = (has_bias && r0_ok) ? ref_round<A>(load_as_float(p.bias, p.bias_dtype, n0 + g)) : 0.0f;
    const float b1 = (has_bias && r1_ok) ? ref_round<A>(load_as_float(p.bias, p.bias_dtype, n0 + g + 8)) : 0.0f;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int64_t m = p.m0 + mt * 8 + 2 * t + j;
            if (m >= p.M) continue;
            if (r0_ok) y[m * p.ldy + n0 + g] = Act<A>::from_float(has_bias ? acc[mt][j] + b0 : acc[mt][j]);
            if (r1_ok) y[m * p.ldy + n0 + g + 8] = Act<A>::from_float(has_bias ? acc[mt][2 + j] + b1 : acc[mt][2 + j]);
        }
    }
}

// Fast path of the same kernel for the common aligned case: K a multiple of 64, N a multiple of 16,
// 16-byte aligned rows.  No bounds checks or 64-bit index arithmetic inside the k loop: pointers
// are set up once and advanced by constants, rows beyond M are handled by a loop-invariant
// predicate.  Everything else (operand orientation, k permutation, two-stage software pipeline,
// 4-way split of K, epilogue) is as in w8a16_stream_kernel.
template <typename A, int MT>
__global__ void __launch_bounds__(kWarps * 32, 7) w8a16_stream_fast_kernel(const StreamParams p) {
    // Seven CTAs per SM (<= 72 registers per thread) so that the N / 16 tiles of the usual layer
    // shapes are all resident at once: with fewer, a short second wave of CTAs doubles the run time.
    // Only the weight stream is staged in registers (two stages of two 64-k rounds); the
    // activations are read where they are used, they are served by L1.
    // rounds (64 k each) per pipeline stage; one with two activation tiles, whose second accumulator set would
    // otherwise spill under the 72-register cap (measured: M=16 17.0 -> 15.7 us)
    constexpr int U = MT == 1 ? 2 : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t n0 = (int64_t)blockIdx.x * 16;

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    // 16-byte units: a round of a weight row is 4 units (thread t takes unit t), of an activation
    // row 8 units (thread t takes units 2t, 2t+1)
    const uint4* w0 = reinterpret_cast<const uint4*>(p.wq + (n0 + g) * p.K) + t;
    const uint4* w1 = reinterpret_cast<const uint4*>(p.wq + (n0 + g + 8) * p.K) + t;
    const uint4* xr[MT];
    bool m_ok[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int64_t m = p.m0 + mt * 8 + g;
        m_ok[mt] = m < p.M;
        xr[mt] = reinterpret_cast<const uint4*>(static_cast<const A*>(p.x) + (m_ok[mt] ? m : 0) * p.ldx) + 2 * t;
    }
    const int nrounds = (int)(p.K / 64);

    struct Stage {
        uint4 c0[U], c1[U];
    };
    auto load_stage = [&](Stage& st, int r) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (r + u < nrounds) {
                st.c0[u] = __ldcs(w0 + (r + u) * 4);
                st.c1[u] = __ldcs(w1 + (r + u) * 4);
            }
        }
    };
    auto compute_stage = [&](const Stage& st, int r) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (r + u >= nrounds) continue;
            uint4 xa[MT][2];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                if (m_ok[mt]) {
                    xa[mt][0] = __ldg(xr[mt] + (r + u) * 8);
                    xa[mt][1] = __ldg(xr[mt] + (r + u) * 8 + 1);
                } else {
                    xa[mt][0] = make_uint4(0u, 0u, 0u, 0u);
                    xa[mt][1] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            const uint32_t cw0[4] = {st.c0[u].x, st.c0[u].y, st.c0[u].z, st.c0[u].w};
            const uint32_t cw1[4] = {st.c1[u].x, st.c1[u].y, st.c1[u].z, st.c1[u].w};
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                uint32_t a[4];
                Act<A>::widen4(cw0[s], a[0], a[2]);
                Act<A>::widen4(cw1[s], a[1], a[3]);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint4& xq = xa[mt][s >> 1];
                    const uint32_t b0 = (s & 1) ? xq.z : xq.x, b1 = (s & 1) ? xq.w : xq.y;
                    Act<A>::mma(acc[mt], a, b0, b1);
                }
            }
        }
    };
    {
        Stage st0, st1;
        int r = warp * U;
        constexpr int step = kWarps * U;
        // Programmatic launch edge: the first stage of weights is requested before the wait for the kernel ahead
        // (which may still be producing the activations), so the stream ramps up under that kernel's tail.
        if (p.weights_ready) {
            pdl_trigger();
            load_stage(st0, r);
            pdl_wait();
        } else {
            pdl_wait();
            pdl_trigger();
            load_stage(st0, r);
        }
        while (r < nrounds) {
            load_stage(st1, r + step);
            compute_stage(st0, r);
            r += step;
            if (r >= nrounds) break;
            load_stage(st0, r + step);
            compute_stage(st1, r);
            r += step;
        }
    }

    __shared__ float red[kWarps - 1][MT * 4][32];
    if (warp > 0) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) red[warp - 1][mt * 4 + j][lane] = acc[mt][j];
    }
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int w = 0; w < kWarps - 1; ++w)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[mt][j] += red[w][mt * 4 + j][lane];

    // the reference's rounding order: GEMM output, product with the scale, sum with the outlier product,
    // sum with the bias -- each rounded to the activation type
    const float s0 = ref_round<A>(load_as_float(p.scales, p.scales_dtype, n0 + g));
    const float s1 = ref_round<A>(load_as_float(p.scales, p.scales_dtype, n0 + g + 8));
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        acc[mt][0] = ref_round<A>(ref_round<A>(acc[mt][0]) * s0); acc[mt][1] = ref_round<A>(ref_round<A>(acc[mt][1]) * s0);
        acc[mt][2] = ref_round<A>(ref_round<A>(acc[mt][2]) * s1); acc[mt][3] = ref_round<A>(ref_round<A>(acc[mt][3]) * s1);
    }
    if (p.KO > 0) {
        const A* xo = static_cast<const A*>(p.xo);
        const A* wo = static_cast<const A*>(p.wo);
        float side[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) side[mt][j] = 0.0f;
        const int64_t osteps = (p.KO + 15) / 16;
        for (int64_t st = 0; st < osteps; ++st) {
            const int64_t k = st * 16 + t * 4;
            uint32_t a0[2], a1[2];
            load_acts<A, 1>(wo + (n0 + g) * p.KO, k, p.KO, true, a0);
            load_acts<A, 1>(wo + (n0 + g + 8) * p.KO, k, p.KO, true, a1);
            const uint32_t a[4] = {a0[0], a1[0], a0[1], a1[1]};
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int64_t m = p.m0 + mt * 8 + g;
                uint32_t b[2];
                load_acts<A, 1>(xo + m * p.ldxo, k, p.KO, m < p.M, b);
                Act<A>::mma(side[mt], a, b[0], b[1]);
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[mt][j] = ref_round<A>(acc[mt][j] + ref_round<A>(side[mt][j]));
    }
    A* y = static_cast<A*>(p.y);
    const bool has_bias = p.bias != nullptr;
    const float b0 = has_bias ? ref_round<A>(load_as_float(p.bias, p.bias_dtype, n0 + g)) : 0.0f;
    const float b1 = has_bias ? ref_round<A>(load_as_float(p.bias, p.bias_dtype, n0 + g + 8)) : 0.0f;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int64_t m = p.m0 + mt * 8 + 2 * t + j;
            if (m >= p.M) continue;
            y[m * p.ldy + n0 + g] = Act<A>::from_float(has_bias ? acc[mt][j] + b0 : acc[mt][j]);
            y[m * p.ldy + n0 + g + 8] = Act<A>::from_float(has_bias ? acc[mt][2 + j] + b1 : acc[mt][2 + j]);
        }
    }
}

template <typename Elem>
__global__ void gather_cols_kernel(const Elem* __restrict__ src, int64_t M, int64_t ld_src,
                                   const int64_t* __restrict__ cols, int64_t ncols, int64_t ncols_padded,
                                   Elem* __restrict__ dst, int64_t ld_dst) {
    pdl_wait();  // src may come from the kernel ahead
    pdl_trigger();
    const int64_t total = M * ncols_padded;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / ncols_padded, j = i - m * ncols_padded;
        dst[m * ld_dst + j] = j < ncols ? src[m * ld_src + __ldg(cols + j)] : Elem(0);
    }
}

inline bool al(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

template <typename A, int VEC>
cudaError_t stream_pick_mt(StreamParams p, cudaStream_t s) {
    const unsigned grid = (unsigned)((p.N + 15) / 16);
    int64_t m0 = 0;
    int extra = -1;  // launches beyond the one the C entry point accounts for
    while (m0 < p.M) {
        ++extra;
        const int64_t left = p.M - m0;
        p.m0 = m0;
        if (left > 32) {
            launch_dependent(w8a16_stream_kernel<A, VEC, 8>, grid, kWarps * 32, 0, s, p);
            m0 += 64;
        } else if (left > 16) {
            launch_dependent(w8a16_stream_kernel<A, VEC, 4>, grid, kWarps * 32, 0, s, p);
            m0 += 32;
        } else if (left > 8) {
            launch_dependent(w8a16_stream_kernel<A, VEC, 2>, grid, kWarps * 32, 0, s, p);
            m0 += 16;
        } else {
            launch_dependent(w8a16_stream_kernel<A, VEC, 1>, grid, kWarps * 32, 0, s, p);
            m0 += 8;
        }
    }
    if (extra > 0) count_launches(extra);
    return cudaPeekAtLastError();
}

template <typename A>
cudaError_t stream_fast(StreamParams p, cudaStream_t s) {
    const unsigned grid = (unsigned)(p.N / 16);
    int64_t m0 = 0;
    int extra = -1;  // launches beyond the one the C entry point accounts for
    while (m0 < p.M) {
        ++extra;
        const int64_t left = p.M - m0;
        p.m0 = m0;
        if (left > 8) {
            launch_dependent(w8a16_stream_fast_kernel<A, 2>, grid, kWarps * 32, 0, s, p);
            m0 += 16;
        } else {
            launch_dependent(w8a16_stream_fast_kernel<A, 1>, grid, kWarps * 32, 0, s, p);
            m0 += 8;
        }
    }
    if (extra > 0) count_launches(extra);
    return cudaPeekAtLastError();
}

template <typename A>
cudaError_t stream_pick_vec(const StreamParams& p, cudaStream_t s) {
    const bool base16 = al(p.wq, 16) && al(p.x, 16);
    if (base16 && p.M <= 16 && p.K % 64 == 0 && p.N % 16 == 0 && p.ldx % 8 == 0) return stream_fast<A>(p, s);
    if (base16 && p.K % 16 == 0 && p.ldx % 8 == 0) return stream_pick_mt<A, 16>(p, s);
    if (al(p.wq, 8) && al(p.x, 16) && p.K % 8 == 0 && p.ldx % 8 == 0) return stream_pick_mt<A, 8>(p, s);
    if (al(p.wq, 4) && al(p.x, 8) && p.K % 4 == 0 && p.ldx % 4 == 0) return stream_pick_mt<A, 4>(p, s);
    return stream_pick_mt<A, 1>(p, s);
}

}  // namespace

cudaError_t launch_w8a16_stream(const W8A16Args& a, cudaStream_t s) {
    StreamParams p;
    p.x = a.x; p.M = a.M; p.K = a.K; p.ldx = a.ldx;
    p.wq = a.wq; p.N = a.N;
    p.scales = a.scales; p.scales_dtype = a.scales_dtype;
    p.bias = a.bias; p.bias_dtype = a.bias_dtype;
    p.xo = a.xo; p.wo = a.wo; p.KO = a.KO; p.ldxo = a.ldxo;
    p.y = a.y; p.ldy = a.ldy; p.m0 = 0; p.weights_ready = a.weights_ready ? 1 : 0;
    if (a.act_dtype == kBF16) return stream_pick_vec<__nv_bfloat16>(p, s);
    if (a.act_dtype == kF16) return stream_pick_vec<__half>(p, s);
    return cudaErrorInvalidValue;
}

cudaError_t launch_gather_cols(const void* src, int64_t M, int64_t ld_src, const int64_t* cols, int64_t ncols,
                               int64_t ncols_padded, void* dst, int64_t ld_dst, int elem_size, cudaStream_t s) {
    const int64_t total = M * ncols_padded;
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
    if (blocks < 1) blocks = 1;
    if (elem_size == 2)
        launch_dependent(gather_cols_kernel<uint16_t>, (unsigned)blocks, 256, 0, s, static_cast<const uint16_t*>(src), M, ld_src,
                                                                        cols, ncols, ncols_padded, static_cast<uint16_t*>(dst),
                                                                        ld_dst);
    else
        launch_dependent(gather_cols_kernel<uint32_t>, (unsigned)blocks, 256, 0, s, static_cast<const uint32_t*>(src), M, ld_src,
                                                                        cols, ncols, ncols_padded, static_cast<uint32_t*>(dst),
                                                                        ld_dst);
    return cudaPeekAtLastError();
}

}  // namespace cb
