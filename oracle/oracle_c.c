/*
 * Plain-C restatement of the cuBlade quantization arithmetic.  TEST INFRASTRUCTURE.
 *
 * Independent of PyTorch: bf16 / fp16 / E4M3 conversions are done in software here, so
 * agreement between this file and oracle.py pins both against mistakes in either.
 * Only tests and the CPU-baseline leg of the benchmark load the library built from it.
 *
 * Follows (paths inside the emre570/cublade tree):
 *   FP8 quantize   cublade/kernels/cuda/quantization/quantize_per_tensor_fp8.cu:38-131
 *   FP8 dequantize cublade/kernels/cuda/quantization/dequantize_per_tensor_fp8.cu:32-65
 *   INT8 quantize  cublade/kernels/cuda/quantization/quantize_int8.cu:120-165, 245-296, 358-370
 *                  cublade/kernels/cuda/quantization/int8_pack.cuh:51-56
 *   INT8 dequant   cublade/kernels/cuda/quantization/dequantize_int8.cu:39-63, 81-108, 129-133
 *   W8A16 forward  cublade/quantization/linear.py:123-135 (value computed in double)
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -fno-fast-math -shared -fPIC oracle_c.c -o liboracle_c.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

enum { OC_F16 = 0, OC_BF16 = 1, OC_F32 = 2 };

static inline float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_to_f32(sign);
        float v = ldexpf((float)man, -24); /* subnormal: man * 2^-24 */
        return sign ? -v : v;
    }
    if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
    return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* round-to-nearest-even fp32 -> bf16 */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_to_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fffu; /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/* round-to-nearest-even fp32 -> fp16 (software, handles subnormals and overflow to inf) */
static inline uint16_t f32_to_f16(float f) {
    uint32_t u = f32_to_bits(f);
    uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7fffu);
    if (a >= 0x47800000u) { /* >= 65536: inf (values in [65520, 65536) handled by rounding below) */
        return (uint16_t)(sign | 0x7c00u);
    }
    float av = bits_to_f32(a);
    if (av < 6.103515625e-05f) { /* below min normal 2^-14: subnormal grid of 2^-24 */
        float q = nearbyintf(av * 16777216.0f);
        return (uint16_t)(sign | (uint16_t)q); /* q == 1024 encodes the min normal */
    }
    int e;
    float m = frexpf(av, &e); /* av = m * 2^e, m in [0.5, 1) */
    float mant = nearbyintf((m * 2.0f - 1.0f) * 1024.0f);
    int ee = e - 1;
    if (mant == 1024.0f) { mant = 0.0f; ee += 1; }
    if (ee > 15) return (uint16_t)(sign | 0x7c00u);
    return (uint16_t)(sign | ((uint16_t)(ee + 15) << 10) | (uint16_t)mant);
}

/* fp32 -> E4M3 (fn variant: no inf, max 448, NaN = 0x7f), round-to-nearest-even, saturate-to-finite */
static inline uint8_t f32_to_e4m3(float f) {
    uint32_t u = f32_to_bits(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint8_t)(sign | 0x7fu);
    float a = fabsf(f);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7eu);
    if (a < 0.015625f) { /* below min normal 2^-6: subnormal grid of 2^-9 */
        float q = nearbyintf(a * 512.0f);
        return (uint8_t)(sign | (uint8_t)q); /* q == 8 encodes the min normal */
    }
    int e;
    float m = frexpf(a, &e);
    float mant = nearbyintf((m * 2.0f - 1.0f) * 8.0f);
    int ee = e - 1;
    if (mant == 8.0f) { mant = 0.0f; ee += 1; }
    unsigned code = ((unsigned)(ee + 7) << 3) | (unsigned)mant;
    if (code > 0x7eu) code = 0x7eu;
    return (uint8_t)(sign | code);
}

static inline float e4m3_to_f32(uint8_t c) {
    unsigned exp = (c >> 3) & 0xfu, man = c & 7u;
    float v;
    if (exp == 15 && man == 7) return bits_to_f32(0x7fc00000u);
    if (exp == 0) v = ldexpf((float)man, -9);
    else v = ldexpf(1.0f + (float)man / 8.0f, (int)exp - 7);
    return (c & 0x80u) ? -v : v;
}

static inline float load_f32(const void* x, int dtype, int64_t i) {
    if (dtype == OC_F32) return ((const float*)x)[i];
    if (dtype == OC_BF16) return bf16_to_f32(((const uint16_t*)x)[i]);
    return f16_to_f32(((const uint16_t*)x)[i]);
}

static inline void store_16(void* y, int dtype, int64_t i, float v) {
    ((uint16_t*)y)[i] = dtype == OC_BF16 ? f32_to_bf16(v) : f32_to_f16(v);
}

/* fmaxf semantics of the kernels: NaN operands are dropped */
static float amax_abs(const void* x, int dtype, int64_t begin, int64_t end) {
    float m = 0.0f;
#pragma omp parallel for reduction(max : m) if (end - begin > 65536)
    for (int64_t i = begin; i < end; ++i) {
        float a = fabsf(load_f32(x, dtype, i));
        if (a > m) m = a; /* comparison is false for NaN: dropped */
    }
    return m;
}

int oc_fp8_quantize(const void* x, int dtype, int64_t n, float eps, uint8_t* q, float* scale) {
    float amax = amax_abs(x, dtype, 0, n);
    float a = amax > eps ? amax : eps;
    float inv = 448.0f / a;
    *scale = 1.0f / inv;
#pragma omp parallel for if (n > 65536)
    for (int64_t i = 0; i < n; ++i) q[i] = f32_to_e4m3(load_f32(x, dtype, i) * inv);
    return 0;
}

int oc_fp8_dequantize(const uint8_t* q, const float* scale, int64_t n, int out_dtype, void* y) {
    const float s = *scale;
#pragma omp parallel for if (n > 65536)
    for (int64_t i = 0; i < n; ++i) store_16(y, out_dtype, i, e4m3_to_f32(q[i]) * s);
    return 0;
}

static inline int8_t round_clamp_int8(float v) {
    if (v != v) return 0;
    float r = nearbyintf(v); /* default rounding mode: to nearest even */
    if (r > 127.0f) r = 127.0f;
    if (r < -127.0f) r = -127.0f;
    return (int8_t)r;
}

/* nseg independent segments of L elements (per tensor: nseg = 1) */
int oc_int8_quantize_segments(const void* x, int dtype, int64_t nseg, int64_t L, float eps, int8_t* q, float* scales) {
#pragma omp parallel for if (nseg > 1)
    for (int64_t s = 0; s < nseg; ++s) {
        float amax = 0.0f;
        for (int64_t i = s * L; i < (s + 1) * L; ++i) {
            float a = fabsf(load_f32(x, dtype, i));
            if (a > amax) amax = a;
        }
        float a = amax > eps ? amax : eps;
        float inv = (float)(127.0 / (double)a);
        scales[s] = (float)(1.0 / (double)inv);
        for (int64_t i = s * L; i < (s + 1) * L; ++i) q[i] = round_clamp_int8(load_f32(x, dtype, i) * inv);
    }
    return 0;
}

int oc_int8_quantize_tensor(const void* x, int dtype, int64_t n, float eps, int8_t* q, float* scale) {
    float amax = amax_abs(x, dtype, 0, n);
    float a = amax > eps ? amax : eps;
    float inv = (float)(127.0 / (double)a);
    *scale = (float)(1.0 / (double)inv);
#pragma omp parallel for if (n > 65536)
    for (int64_t i = 0; i < n; ++i) q[i] = round_clamp_int8(load_f32(x, dtype, i) * inv);
    return 0;
}

/* seg_len == 0: one scale */
int oc_int8_dequantize(const int8_t* q, const float* scales, int64_t n, int64_t seg_len, int out_dtype, void* y) {
#pragma omp parallel for if (n > 65536)
    for (int64_t i = 0; i < n; ++i) {
        float s = scales[seg_len > 0 ? i / seg_len : 0];
        store_16(y, out_dtype, i, (float)q[i] * s);
    }
    return 0;
}

/* y[m,n] = (sum_k x[m,k] q[n,k]) * scale[n] + sum_j xo[m,j] wo[n,j] + bias[n], all in double */
int oc_w8a16_forward(const void* x, int act_dtype, int64_t M, int64_t K, const int8_t* wq, int64_t N,
                     const float* scales, const float* bias, const void* xo, const void* wo, int64_t KO, double* y) {
#pragma omp parallel for collapse(2)
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            double acc = 0.0;
            for (int64_t k = 0; k < K; ++k) acc += (double)load_f32(x, act_dtype, m * K + k) * (double)wq[n * K + k];
            acc *= (double)scales[n];
            for (int64_t j = 0; j < KO; ++j)
                acc += (double)load_f32(xo, act_dtype, m * KO + j) * (double)load_f32(wo, act_dtype, n * KO + j);
            if (bias) acc += (double)bias[n];
            y[m * N + n] = acc;
        }
    return 0;
}

/* single-value probes for exhaustive conversion tests */
uint8_t oc_probe_e4m3(float v) { return f32_to_e4m3(v); }
float oc_probe_e4m3_decode(uint8_t c) { return e4m3_to_f32(c); }
uint16_t oc_probe_bf16(float v) { return f32_to_bf16(v); }
uint16_t oc_probe_f16(float v) { return f32_to_f16(v); }
float oc_probe_f16_decode(uint16_t h) { return f16_to_f32(h); }
