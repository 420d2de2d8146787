// Internal launch interface between the C-ABI layer (cabi.cu) and the kernel
// translation units.  Everything here takes raw device pointers and a stream;
// nothing allocates.  Return value: cudaError_t of the launch (cudaSuccess = 0).
#pragma once

#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace cb {

enum DType : int { kF16 = 0, kBF16 = 1, kF32 = 2 };
enum CodeKind : int { kCodeInt8 = 0, kCodeE4M3 = 1 };

inline int dtype_size(int dt) { return dt == kF32 ? 4 : 2; }

// number of SMs of the current device (cached per device)
int sm_count();

// ---- programmatic dependent launch ---------------------------------------------
// A kernel launched through launch_dependent() may become resident while the kernel before it in the
// stream is still running; it must call pdl_wait() before it touches anything that kernel (or any
// earlier one) wrote -- until then it may only read memory no kernel in flight writes (its inputs).
// The kernel before it calls pdl_trigger() to allow that early start.  Both are no-ops when the launch
// carries no such edge, so the same kernels also run from plain launches.  Stream capture records the
// edge, so graph replays keep the overlap.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t s,
                             Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// ---- per-tensor (two phase) ------------------------------------------------
// amax[0] = max(amax[0], max|x|); amax must hold a non-negative float (0 to start).
cudaError_t launch_amax_tensor(const void* x, int dtype, int64_t n, float* amax, cudaStream_t s);
// codes = encode(x * qmax/max(amax,eps)); scale_out[0] = 1/(qmax/max(amax,eps)).
// nparts == 0: amax is one float; nparts > 0: amax points at nparts per-CTA partial maxima to fold.
cudaError_t launch_cast_tensor(const void* x, int dtype, int64_t n, const float* amax, int nparts, float eps, int code,
                               void* q, float* scale_out, cudaStream_t s);
// Single-GPU phase 1 without atomics or pre-zeroing: partials[i] = max|x| seen by CTA i, *nparts = CTAs used
// (<= per_tensor_scratch_floats()).
int per_tensor_scratch_floats();
cudaError_t launch_amax_partials(const void* x, int dtype, int64_t n, float* partials, int* nparts, cudaStream_t s);

// ---- the amax exchange of a sharded per-tensor quantization over peer memory (peer_exchange.cu) ----
// peer_state[r]: rank r's state array (peer_exchange_state_words() 64-bit words, zeroed once before the first call,
// mapped into this process); out_amax = max over the ranks' local_amax.  Every rank calls it once per exchange.
int peer_exchange_state_words();
int peer_exchange_max_ranks();
cudaError_t launch_amax_peer_exchange(const float* local_amax, const void* const* peer_state, int rank, int world,
                                      float* out_amax, cudaStream_t s);

// ---- per-segment (rows of a [nseg, L] matrix: channels or groups), one pass --
cudaError_t launch_quant_segments(const void* x, int dtype, int64_t nseg, int64_t L, float eps, int code, void* q,
                                  float* scale_out, cudaStream_t s);

// ---- per-channel INT8 along any axis of a contiguous [outer, C, inner] tensor, in place (no transpose) ----
// scratch: C floats, overwritten.  scale_out: C floats.
cudaError_t launch_quant_axis(const void* x, int dtype, int64_t outer, int64_t C, int64_t inner, float eps, void* q,
                              float* scale_out, float* scratch, cudaStream_t s);
cudaError_t launch_dequant_axis(const void* q, const float* scale, int64_t outer, int64_t C, int64_t inner, int out_dtype,
                                void* y, cudaStream_t s);

// ---- per-group INT8 with the groups along a non-last axis of a contiguous [outer, C, inner] tensor, in place ----
// G consecutive indices of C form a group for every (outer, inner) position; C % G == 0.
// scale_out: outer * inner * (C / G) floats, index (o * inner + i) * (C / G) + c / G.
cudaError_t launch_quant_group_axis(const void* x, int dtype, int64_t outer, int64_t C, int64_t inner, int G, float eps,
                                    void* q, float* scale_out, cudaStream_t s);
cudaError_t launch_dequant_group_axis(const void* q, const float* scale, int64_t outer, int64_t C, int64_t inner, int G,
                                      int out_dtype, void* y, cudaStream_t s);

// ---- fused RMSNorm -> per-row quantize ----------------------------------------
// x [rows, H] fp16 / bf16; gamma [H] of the same type or nullptr; q [rows, H] codes; scale_out [rows];
// y_out [rows, H] (the normalised rows in x's type) or nullptr; rstd_out [rows] (1 / rms) or nullptr.
cudaError_t launch_rmsnorm_quant(const void* x, int dtype, int64_t rows, int64_t H, const void* gamma, float rms_eps,
                                 float q_eps, int code, void* q, float* scale_out, void* y_out, float* rstd_out,
                                 cudaStream_t s);

// ---- dequantize -------------------------------------------------------------
// seg_len == 0: one scale for the whole tensor; otherwise scale[i / seg_len].
cudaError_t launch_dequant(const void* q, int code, const float* scale, int64_t n, int64_t seg_len, int out_dtype,
                           void* y, cudaStream_t s);

// ---- W8A16 linear -------------------------------------------------------------
struct W8A16Args {
    const void* x;        // [M, K] bf16/f16 activations, row stride ldx elements
    int64_t M, K, ldx;
    const int8_t* wq;     // [N, K] int8 codes, row-major
    int64_t N;
    const void* scales;   // [N] per-output-channel scale
    int scales_dtype;     // kF16 / kBF16 / kF32
    const void* bias;     // [N] or nullptr
    int bias_dtype;
    // optional LLM.int8 side product: y += xo[M, KO] . wo[N, KO]^T (un-scaled)
    const void* xo;       // [M, KO] same dtype as x, row stride ldxo
    const void* wo;       // [N, KO] same dtype as x, row-major
    int64_t KO, ldxo;
    void* y;              // [M, N] same dtype as x, row stride ldy
    int64_t ldy;
    int act_dtype;        // kBF16 or kF16
    void* workspace;      // may be nullptr when workspace_bytes == 0
    size_t workspace_bytes;
    // The kernels are launched with a programmatic edge to the kernel ahead of them in the stream and fetch their
    // first weights before they wait for it: legal only when that kernel did not write wq (true for a layer's own
    // weights; false when wq was unpacked from 4-bit codes by the launch just before).
    bool weights_ready = true;
};
size_t w8a16_workspace_bytes(int64_t M, int64_t N, int64_t K);
// path: 0 = automatic, 1 = weight-streaming (skinny M) kernel, 2 = tcgen05 CTA-pair GEMM, 3 = tcgen05 single-CTA GEMM
cudaError_t launch_w8a16(const W8A16Args& a, int path, cudaStream_t s);
// ---- W8A8 linear ---------------------------------------------------------------
struct W8A8Args {
    const int8_t* xq;   // [M, K] int8 activations, row-major
    const float* xs;    // [M] per-token scales
    int64_t M, K;
    const int8_t* wq;   // [N, K] int8 weights, row-major
    int64_t N;
    const void* ws;     // [N] per-output-channel scales
    int ws_dtype;       // kF16 / kBF16 / kF32
    const void* bias;   // [N] or nullptr
    int bias_dtype;
    void* y;            // [M, N] of out_dtype, row stride ldy
    int64_t ldy;
    int out_dtype;      // kBF16 or kF16
};
cudaError_t launch_w8a8(const W8A8Args& a, cudaStream_t s);

// ---- W4A16 linear (4-bit weights, packed eight codes per 32-bit word: byte j = code j | code 4 + j << 4) ----
// w [N, K] fp16 / bf16 / fp32 -> packed [N, K / 2] + scale_out [N]; K % 8 == 0.
cudaError_t launch_w4_quantize_rows(const void* w, int dtype, int64_t N, int64_t K, float eps, void* packed,
                                    float* scale_out, cudaStream_t s);
cudaError_t launch_w4_unpack(const void* packed, int64_t N, int64_t K, int8_t* out, cudaStream_t s);
struct W4A16Args {
    const void* x;       // [M, K] bf16 / f16, row stride ldx elements
    int64_t M, K, ldx;
    const void* wq4;     // [N, K / 2] packed codes
    int64_t N;
    const void* scales;  // [N]
    int scales_dtype;
    const void* bias;    // [N] or nullptr
    int bias_dtype;
    void* y;             // [M, N] of the activation type
    int64_t ldy;
    int act_dtype;
    void* workspace;
    size_t workspace_bytes;
};
size_t w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K, bool aligned);
cudaError_t launch_w4a16(const W4A16Args& a, cudaStream_t s, int* launches);

// ---- dense GEMM C[M, N] = A[M, K] . B[K, N] (fp16 / bf16 -> fp32 accumulate, int8 / uint8 -> int32) ----------
// in_kind: 0 fp16, 1 bf16, 2 int8, 3 uint8.  out_kind: 0 fp32, 1 fp16 (fp16 inputs only), 2 int32, 3 bf16 (bf16 inputs
// only).  leaky_relu != 0 (float accumulators only): x >= 0 ? x : 0.01 x on the accumulator before it is stored.
// workspace: tc_gemm_workspace_bytes(N, K, in_kind) bytes for the transposed copy of B.
size_t tc_gemm_workspace_bytes(int64_t N, int64_t K, int in_kind);
cudaError_t launch_tc_gemm(const void* a, const void* b, int64_t M, int64_t N, int64_t K, int in_kind, void* c,
                           int64_t ldc, int out_kind, void* workspace, size_t workspace_bytes, cudaStream_t s, int leaky_relu = 0);

// reads (and leaves untouched) the per-device flag a kernel raises when one of its bounded waits
// expired; synchronises the stream.
cudaError_t w8a16_tc_read_error(unsigned int* host_value, cudaStream_t s);
// gathers columns: dst[m, j] = src[m, cols[j]] for j < ncols and 0 for ncols <= j < ncols_padded
// (activation re-pack for the outlier split; the zero columns pad K to what the tensor-core kernels load)
cudaError_t launch_gather_cols(const void* src, int64_t M, int64_t ld_src, const int64_t* cols, int64_t ncols,
                               int64_t ncols_padded, void* dst, int64_t ld_dst, int elem_size, cudaStream_t s);
// adds n to the library's launch counter (cb_launch_count)
void count_launches(int n);

}  // namespace cb
