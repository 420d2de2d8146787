// W4A16 linear: 4-bit weights (one scale per output feature), 16-bit activations, fp32 accumulation.
//
//   y[m, n] = T( (sum_k x[m, k] * code[n, k]) * scale[n] + bias[n] ),   code in [-7, 7]
//
// The reference reserves the layer type ("w4a16" in the registry comment of
// cublade/quantization/quantizers.py:169-171) without a kernel, a storage format or a layer.  The
// quantizer follows the reference's symmetric INT8 arithmetic (cublade/kernels/cuda/quantization/
// quantize_int8.cu:245-296) with qmax = 7:  a = max(amax, eps); inv = float(7 / double(a));
// scale = float(1 / double(inv)); code = clamp(rint(x * inv), -7, 7).
//
// Storage: row n of the packed matrix is K / 2 bytes; its 32-bit word i holds the codes k = 8i .. 8i + 7 as
// two's-complement nibbles, byte j carrying code 8i + j in its low and code 8i + 4 + j in its high nibble.
// With that order one AND gives four codes of consecutive k as the four bytes of a word, which is the
// form the packed-bf16 widening of the W8A16 kernels starts from: 11 instructions per 8 weights.
//
// Kernels: w4_quantize_rows_kernel (one CTA per weight row: amax, scale, codes, pack), w4_unpack_kernel
// (packed -> int8 [N, K], feeding the W8A16 tensor-core GEMM for M > 16), w4a16_stream_kernel (decode
// shapes M <= 16: the weight-streaming mma.sync kernel of w8a16_stream.cu reading half the bytes).
#include "launch.h"
#include "pack.cuh"

namespace cb {

namespace {

constexpr int kWarps = 4;

// eight nibbles of a packed word -> offset-binary bytes: lo = codes 0..3, hi = codes 4..7, each byte = code + 8
__device__ __forceinline__ void split_nibbles(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t x = w ^ 0x88888888u;  // two's complement nibble -> nibble + 8 (0 .. 15)
    lo = x & 0x0F0F0F0Fu;
    hi = (x >> 4) & 0x0F0F0F0Fu;
}

template <typename A>
struct W4Act;
template <>
struct W4Act<__nv_bfloat16> {
    // four offset-binary bytes (value + 8, 0..15) -> two words of bf16 pairs (c0,c1) (c2,c3), exact:
    // 0x4300 | b is the bf16 number 128 + b, and (128 + b) - 136 = b - 8 has magnitude <= 8.
    __device__ __forceinline__ static void widen4(uint32_t b, uint32_t& p01, uint32_t& p23) {
        const uint32_t a01 = __byte_perm(b, 0x43434343u, 0x4140), a23 = __byte_perm(b, 0x43434343u, 0x4342);
        const uint32_t k = 0x43084308u;  // 136.0 twice
        const __nv_bfloat162 d01 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&a01), *reinterpret_cast<const __nv_bfloat162*>(&k));
        const __nv_bfloat162 d23 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&a23), *reinterpret_cast<const __nv_bfloat162*>(&k));
        p01 = *reinterpret_cast<const uint32_t*>(&d01);
        p23 = *reinterpret_cast<const uint32_t*>(&d23);
    }
    __device__ __forceinline__ static void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <>
struct W4Act<__half> {
    // 0x6400 | b is the fp16 number 1024 + b; (1024 + b) - 1032 = b - 8, exact
    __device__ __forceinline__ static void widen4(uint32_t b, uint32_t& p01, uint32_t& p23) {
        const uint32_t a01 = __byte_perm(b, 0x64646464u, 0x4140), a23 = __byte_perm(b, 0x64646464u, 0x4342);
        const uint32_t k = 0x64086408u;  // 1032.0 twice
        const __half2 d01 = __hsub2(*reinterpret_cast<const __half2*>(&a01), *reinterpret_cast<const __half2*>(&k));
        const __half2 d23 = __hsub2(*reinterpret_cast<const __half2*>(&a23), *reinterpret_cast<const __half2*>(&k));
        p01 = *reinterpret_cast<const uint32_t*>(&d01);
        p23 = *reinterpret_cast<const uint32_t*>(&d23);
    }
    __device__ __forceinline__ static void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

__device__ __forceinline__ float load_float(const void* p, int dtype, int64_t i) {
    if (dtype == kF32) return static_cast<const float*>(p)[i];
    if (dtype == kBF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    return __half2float(static_cast<const __half*>(p)[i]);
}

// One CTA per weight row: amax, scale, codes, packed words.  The row is read twice (the second
// time from L2); weight quantization runs once per layer.
template <typename T>
__global__ void __launch_bounds__(256) w4_quantize_rows_kernel(const T* __restrict__ w, int64_t K, float eps,
                                                               uint32_t* __restrict__ packed, float* __restrict__ scale_out) {
    const T* row = w + (int64_t)blockIdx.x * K;
    float m = 0.0f;
    for (int64_t i = threadIdx.x; i < K; i += 256) m = fmaxf(m, fabsf(DTypeTraits<T>::to_float(row[i])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float red[8];
    __shared__ float inv_s;
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = red[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) a = fmaxf(a, red[i]);
        a = fmaxf(a, eps);
        const float inv = (float)(7.0 / (double)a);
        inv_s = inv;
        scale_out[blockIdx.x] = (float)(1.0 / (double)inv);
    }
    __syncthreads();
    const float inv = inv_s;
    uint32_t* prow = packed + (int64_t)blockIdx.x * (K / 8);
    for (int64_t i = threadIdx.x; i < K / 8; i += 256) {
        uint32_t word = 0u;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int q = __float2int_rn(__fmul_rn(DTypeTraits<T>::to_float(row[8 * i + e]), inv));
            q = max(-7, min(7, q));
            const int byte = e & 3, high = e >> 2;
            word |= (uint32_t)(q & 0xF) << (8 * byte + 4 * high);
        }
        prow[i] = word;
    }
}

// packed [N, K / 2] -> int8 [N, K]; one thread per packed word (8 codes = 8 bytes out)
__global__ void __launch_bounds__(256) w4_unpack_kernel(const uint32_t* __restrict__ packed, int64_t nwords,
                                                        uint2* __restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nwords; i += (int64_t)gridDim.x * 256) {
        uint32_t lo, hi;
        split_nibbles(__ldg(packed + i), lo, hi);
        // offset-binary bytes (code + 8) -> two's-complement int8: a per-byte subtraction of 8
        out[i] = make_uint2(__vsub4(lo, 0x08080808u), __vsub4(hi, 0x08080808u));
    }
}

struct W4Params {
    const void* x;
    int64_t M, K, ldx;
    const uint8_t* wq4;  // [N, K / 2]
    int64_t N;
    const void* scales;
    int scales_dtype;
    const void* bias;
    int bias_dtype;
    void* y;
    int64_t ldy;
    int64_t m0;  // first activation row of this pass
};

// Decode shapes.  The structure of w8a16_stream_fast_kernel (w8a16_stream.cu): a CTA owns 16 weight rows, its four
// warps split K in groups of U rounds of 128 k and reduce through shared memory; the weights are the 16-row
// operand of mma.m16n8k16, MT tiles of 8 activation rows the 8-column operand.  A thread's share of a round is
// 32 consecutive k of weight rows g and g + 8 -- one 16-byte load per row, four packed words: the low nibbles of
// word j are k 8j .. 8j + 3 (mma step 2j), the high nibbles k 8j + 4 .. 8j + 7 (step 2j + 1) -- and the same 32 k
// of each activation row.  Requires K % 128 == 0, N % 16 == 0, 16-byte aligned rows.
template <typename A, int MT>
__global__ void __launch_bounds__(kWarps * 32, 7) w4a16_stream_kernel(const W4Params p) {
    // rounds per pipeline stage: 64 bytes of weights per thread in flight; one round with two activation tiles,
    // whose second accumulator set would otherwise spill under the 72-register cap of seven CTAs per SM
    constexpr int U = MT == 1 ? 2 : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t n0 = (int64_t)blockIdx.x * 16;

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    const uint4* w0 = reinterpret_cast<const uint4*>(p.wq4 + (n0 + g) * (p.K / 2)) + t;
    const uint4* w1 = reinterpret_cast<const uint4*>(p.wq4 + (n0 + g + 8) * (p.K / 2)) + t;
    const uint4* xr[MT];
    bool m_ok[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int64_t m = p.m0 + mt * 8 + g;
        m_ok[mt] = m < p.M;
        xr[mt] = reinterpret_cast<const uint4*>(static_cast<const A*>(p.x) + (m_ok[mt] ? m : 0) * p.ldx) + 4 * t;
    }
    const int nrounds = (int)(p.K / 128);

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
            const uint32_t cw0[4] = {st.c0[u].x, st.c0[u].y, st.c0[u].z, st.c0[u].w};
            const uint32_t cw1[4] = {st.c1[u].x, st.c1[u].y, st.c1[u].z, st.c1[u].w};
#pragma unroll
            for (int half = 0; half < 2; ++half) {  // 64 k each: two packed words per row, 32 bytes of each activation row
                uint4 xa[MT][2];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    if (m_ok[mt]) {
                        xa[mt][0] = __ldg(xr[mt] + (r + u) * 16 + 2 * half);
                        xa[mt][1] = __ldg(xr[mt] + (r + u) * 16 + 2 * half + 1);
                    } else {
                        xa[mt][0] = make_uint4(0u, 0u, 0u, 0u);
                        xa[mt][1] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                uint32_t b0w[4], b1w[4];  // offset-binary bytes of mma steps 0 .. 3 of this half, rows g and g + 8
                split_nibbles(cw0[2 * half], b0w[0], b0w[1]);
                split_nibbles(cw0[2 * half + 1], b0w[2], b0w[3]);
                split_nibbles(cw1[2 * half], b1w[0], b1w[1]);
                split_nibbles(cw1[2 * half + 1], b1w[2], b1w[3]);
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    uint32_t a[4];
                    W4Act<A>::widen4(b0w[s], a[0], a[2]);
                    W4Act<A>::widen4(b1w[s], a[1], a[3]);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint4& xq = xa[mt][s >> 1];
                        const uint32_t b0 = (s & 1) ? xq.z : xq.x, b1 = (s & 1) ? xq.w : xq.y;
                        W4Act<A>::mma(acc[mt], a, b0, b1);
                    }
                }
            }
        }
    };
    {
        Stage st0, st1;
        int r = warp * U;
        constexpr int step = kWarps * U;
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

    const float s0 = load_float(p.scales, p.scales_dtype, n0 + g);
    const float s1 = load_float(p.scales, p.scales_dtype, n0 + g + 8);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        acc[mt][0] *= s0; acc[mt][1] *= s0;
        acc[mt][2] *= s1; acc[mt][3] *= s1;
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
    // D fragment: acc[mt][0..1] -> (weight row g, activation rows 2t, 2t + 1), acc[mt][2..3] -> (row g + 8, same)
    A* y = static_cast<A*>(p.y);
    const float b0 = p.bias ? load_float(p.bias, p.bias_dtype, n0 + g) : 0.0f;
    const float b1 = p.bias ? load_float(p.bias, p.bias_dtype, n0 + g + 8) : 0.0f;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int64_t m = p.m0 + mt * 8 + 2 * t + j;
            if (m >= p.M) continue;
            y[m * p.ldy + n0 + g] = DTypeTraits<A>::from_float(acc[mt][j] + b0);
            y[m * p.ldy + n0 + g + 8] = DTypeTraits<A>::from_float(acc[mt][2 + j] + b1);
        }
    }
}

}  // namespace

cudaError_t launch_w4_quantize_rows(const void* w, int dtype, int64_t N, int64_t K, float eps, void* packed,
                                    float* scale_out, cudaStream_t s) {
    if (N == 0) return cudaSuccess;
    uint32_t* out = static_cast<uint32_t*>(packed);
    const unsigned grid = (unsigned)N;
    if (dtype == kF32) w4_quantize_rows_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(w), K, eps, out, scale_out);
    else if (dtype == kBF16)
        w4_quantize_rows_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(w), K, eps, out, scale_out);
    else w4_quantize_rows_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(w), K, eps, out, scale_out);
    return cudaPeekAtLastError();
}

cudaError_t launch_w4_unpack(const void* packed, int64_t N, int64_t K, int8_t* out, cudaStream_t s) {
    const int64_t nwords = N * (K / 8);
    if (nwords == 0) return cudaSuccess;
    const int64_t want = (nwords + 255) / 256;
    const unsigned grid = (unsigned)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
    w4_unpack_kernel<<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(packed), nwords, reinterpret_cast<uint2*>(out));
    return cudaPeekAtLastError();
}

static bool w4_stream_ok(const W4A16Args& a) {
    auto al = [](const void* p, size_t n) { return (reinterpret_cast<uintptr_t>(p) % n) == 0; };
    return a.M <= 16 && a.K % 128 == 0 && a.N % 16 == 0 && (a.ldx * 2) % 16 == 0 && al(a.x, 16) && al(a.wq4, 16);
}

static size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

// Bytes of caller workspace the call may use: none on the decode route, the unpacked int8 copy of the weights
// plus the W8A16 GEMM's own workspace otherwise.
size_t w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K, bool aligned) {
    if (M < 1 || N < 1 || K < 1) return 0;
    if (aligned && M <= 16 && K % 128 == 0 && N % 16 == 0) return 0;
    return round256((size_t)N * (size_t)K) + w8a16_workspace_bytes(M, N, K);
}

cudaError_t launch_w4a16(const W4A16Args& a, cudaStream_t s, int* launches) {
    *launches = 0;
    if (w4_stream_ok(a)) {
        W4Params p;
        p.x = a.x; p.M = a.M; p.K = a.K; p.ldx = a.ldx;
        p.wq4 = static_cast<const uint8_t*>(a.wq4); p.N = a.N;
        p.scales = a.scales; p.scales_dtype = a.scales_dtype; p.bias = a.bias; p.bias_dtype = a.bias_dtype;
        p.y = a.y; p.ldy = a.ldy; p.m0 = 0;
        const unsigned grid = (unsigned)(a.N / 16);
        const bool bf16 = a.act_dtype == kBF16;
        if (a.M > 8) {
            if (bf16) w4a16_stream_kernel<__nv_bfloat16, 2><<<grid, kWarps * 32, 0, s>>>(p);
            else w4a16_stream_kernel<__half, 2><<<grid, kWarps * 32, 0, s>>>(p);
        } else {
            if (bf16) w4a16_stream_kernel<__nv_bfloat16, 1><<<grid, kWarps * 32, 0, s>>>(p);
            else w4a16_stream_kernel<__half, 1><<<grid, kWarps * 32, 0, s>>>(p);
        }
        *launches = 1;
        return cudaPeekAtLastError();
    }
    // every other shape: unpack to int8 in the caller's workspace, then the W8A16 dispatcher
    const size_t codes = round256((size_t)a.N * (size_t)a.K);
    if (!a.workspace || a.workspace_bytes < codes || (reinterpret_cast<uintptr_t>(a.workspace) & 15)) return cudaErrorInvalidValue;
    int8_t* q = static_cast<int8_t*>(a.workspace);
    cudaError_t e = launch_w4_unpack(a.wq4, a.N, a.K, q, s);
    if (e != cudaSuccess) return e;
    W8A16Args w{};
    w.x = a.x; w.M = a.M; w.K = a.K; w.ldx = a.ldx;
    w.wq = q; w.N = a.N;
    w.scales = a.scales; w.scales_dtype = a.scales_dtype; w.bias = a.bias; w.bias_dtype = a.bias_dtype;
    w.xo = nullptr; w.wo = nullptr; w.KO = 0; w.ldxo = 0;
    w.y = a.y; w.ldy = a.ldy; w.act_dtype = a.act_dtype;
    w.workspace = static_cast<char*>(a.workspace) + codes;
    w.workspace_bytes = a.workspace_bytes - codes;
    *launches = 2;
    w.weights_ready = false;  // the unpack kernel above has just written them
    return launch_w8a16(w, 0, s);
}

}  // namespace cb
