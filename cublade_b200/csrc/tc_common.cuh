// Inline-PTX wrappers and small helpers shared by the tcgen05 W8A16 kernels: mbarrier (bounded
// waits), TMA tile loads (never multicast), tcgen05 alloc / mma / commit / ld, UMMA shared-memory
// and instruction descriptors, exact int8 -> 16-bit widening.
#pragma once

#include "launch.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace cb {
namespace tc {

constexpr int kUmmaM = 128;    // rows of the weight operand per CTA
constexpr int kBlockK = 64;    // k per pipeline stage: 64 x 2 B = one 128-byte swizzle row

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe of a barrier phase (cluster-scope acquire: the completing arrivals may come
// from the peer CTA of a pair).
__device__ __forceinline__ bool mbar_test_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded spin on test_wait (no hardware suspend): used where arrivals come from another CTA.
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (mbar_test_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_test_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > 2000000000LL) {
            *abort_flag = 1u;
            return false;
        }
    }
}

// Bounded wait (about one second of SM clocks).  Returns false on expiry or when another role
// has already raised the abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > 2000000000LL) {
            *abort_flag = 1u;
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
// pull a tile into L2 ahead of its TMA load (no shared memory, no barrier)
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// same MMA with the A operand (128 rows x 16 k, 16-bit) read from tensor memory: lane = row, each
// 32-bit column holds two consecutive k
__device__ __forceinline__ void umma_f16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// integer MMA: A and B signed 8-bit (K = 32 per instruction), int32 accumulator
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 16 columns of 32 bits, registers -> tensor memory
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes (64 16-bit
// elements) in the 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO), descriptor
// version 1, layout type 2 (SWIZZLE_128B).  Advancing k by 16 elements adds 32 bytes to the
// start address.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);   // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;               // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                          // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
    return d;
}

// Instruction descriptor, kind::f16: fp32 accumulate, A and B of the same 16-bit format, both
// K-major, M = 128, N = tile_x.
__device__ __forceinline__ uint32_t make_idesc(bool bf16, uint32_t n) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((uint32_t)(kUmmaM >> 4) << 24);
}

// Instruction descriptor, kind::i8: int32 accumulate (format 2), A and B signed 8-bit (format 1), both
// K-major, M = 128, N = tile_x.
__device__ __forceinline__ uint32_t make_idesc_i8(uint32_t n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(kUmmaM >> 4) << 24);
}

template <typename A>
struct Widen;
template <>
struct Widen<__nv_bfloat16> {
    static constexpr bool kBf16 = true;
    // four int8 codes -> (c0,c1), (c2,c3) as bf16 pairs; exact
    __device__ __forceinline__ static void four(uint32_t c, uint32_t& lo, uint32_t& hi) {
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
    __device__ __forceinline__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
    // Packed pairs (low half = first value).  pack2 rounds two floats to the type; mul2 / add2 round the exact product /
    // sum of the pairs once -- the same value as rounding the float32 product / sum, which is exact or off by far less
    // than half a unit of the 16-bit type whenever float32 has to round it.  The _rn forms are never contracted into
    // a fused multiply-add, which would drop the rounding between the two steps.
    __device__ __forceinline__ static uint32_t pack2(float lo, float hi) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    __device__ __forceinline__ static uint32_t mul2(uint32_t a, uint32_t b) {
        const __nv_bfloat162 v = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    __device__ __forceinline__ static uint32_t add2(uint32_t a, uint32_t b) {
        const __nv_bfloat162 v = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<const uint32_t*>(&v);
    }
};
template <>
struct Widen<__half> {
    static constexpr bool kBf16 = false;
    __device__ __forceinline__ static void four(uint32_t c, uint32_t& lo, uint32_t& hi) {
        const uint32_t u = c ^ 0x80808080u;
        const uint32_t p0 = __byte_perm(u, 0x64006400u, 0x7150);
        const uint32_t p1 = __byte_perm(u, 0x64006400u, 0x7352);
        const __half2 k = __half2half2(__ushort_as_half((unsigned short)0x6480));
        __half2 a = __hsub2(*reinterpret_cast<const __half2*>(&p0), k);
        __half2 b = __hsub2(*reinterpret_cast<const __half2*>(&p1), k);
        lo = *reinterpret_cast<uint32_t*>(&a);
        hi = *reinterpret_cast<uint32_t*>(&b);
    }
    __device__ __forceinline__ static float to_float(__half v) { return __half2float(v); }
    __device__ __forceinline__ static __half from_float(float v) { return __float2half_rn(v); }
    __device__ __forceinline__ static uint32_t pack2(float lo, float hi) {
        const __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    __device__ __forceinline__ static uint32_t mul2(uint32_t a, uint32_t b) {
        const __half2 v = __hmul2_rn(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    __device__ __forceinline__ static uint32_t add2(uint32_t a, uint32_t b) {
        const __half2 v = __hadd2_rn(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<const uint32_t*>(&v);
    }
};

// v rounded to the activation type A and widened back.  The reference's forward materialises a
// 16-bit tensor after every step -- the GEMM's output, the product with the scales (themselves cast
// to the activation type), the sum with the outlier product, the sum with the bias
// (cublade/quantization/linear.py:97-135) -- so an epilogue that reproduces its results bit for bit
// (up to the order of the fp32 accumulation) rounds in the same places:
//   v = r(r(acc) * r(scale));  v = r(v + r(side));  v = r(v + r(bias))
template <typename A>
__device__ __forceinline__ float ref_round(float v) {
    return Widen<A>::to_float(Widen<A>::from_float(v));
}

__device__ __forceinline__ float load_scalar(const void* p, int dtype, int64_t i) {
    if (dtype == kF32) return static_cast<const float*>(p)[i];
    if (dtype == kBF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    return __half2float(static_cast<const __half*>(p)[i]);
}


}  // namespace tc
}  // namespace cb
