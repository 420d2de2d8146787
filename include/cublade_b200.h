/*
 * cublade_b200 -- C ABI of the B200 (sm_100a) quantization hot path.
 *
 * One shared library, libcublade_b200.so, no torch / pybind types in any
 * signature: plain device pointers, sizes, a dtype code and a CUDA stream
 * handle (cudaStream_t passed as void*).  Every entry point
 *   - works on the CUDA device that is current on the calling thread,
 *   - enqueues on `stream` and returns without synchronising,
 *   - allocates nothing: outputs and scratch are the caller's
 *     (exception: none -- cb_*_workspace_bytes tell the caller what to bring),
 *   - returns CB_OK (0) or a cb_status error; cb_last_error() then holds text.
 *
 * Each entry point names the reference interface it stands in for, as
 * <file>:<line> inside the emre570/cublade source tree.
 */
#ifndef CUBLADE_B200_H_
#define CUBLADE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum cb_status {
    CB_OK = 0,
    CB_ERR_ARGUMENT = 1,    /* null pointer, negative size, bad enum          */
    CB_ERR_DTYPE = 2,       /* dtype not accepted by this op                  */
    CB_ERR_ALIGNMENT = 3,   /* reference-mandated alignment rule violated     */
    CB_ERR_RANGE = 4,       /* size outside the supported range               */
    CB_ERR_CUDA = 5,        /* a CUDA call or launch failed                   */
    CB_ERR_WORKSPACE = 6,   /* workspace missing or too small                 */
    CB_ERR_UNSUPPORTED = 7  /* valid request this build cannot serve          */
} cb_status;

/* element type of floating tensors */
typedef enum cb_dtype { CB_F16 = 0, CB_BF16 = 1, CB_F32 = 2 } cb_dtype;

/* library version: major*10000 + minor*100 + patch */
int32_t cb_version(void);
/* text of the last error raised on the calling thread ("" if none) */
const char* cb_last_error(void);
/* number of kernels this library has launched in the calling process */
int64_t cb_launch_count(void);

/* ------------------------------------------------------------------------
 * Per-tensor FP8 E4M3.
 * replaces quantize_per_tensor_fp8(x, eps) -> (q, scale)
 *   cublade/kernels/cuda/quantization/quantize_per_tensor_fp8.cu:162-188
 *   (binding cublade/bindings/cuda/quantize_fp8.py:15-34)
 * x: n elements of CB_F16 / CB_BF16.  q: n bytes (e4m3 codes).  scale: fp32[1].
 * amax_scratch: device scratch of cb_per_tensor_scratch_floats() floats, overwritten (one partial
 * maximum per CTA of the first pass; no atomics, nothing to pre-zero).
 * scale = 1 / (448 / max(amax, eps)); q = e4m3_rn_satfinite(float(x) * (448 / max(amax, eps))).
 * ------------------------------------------------------------------------ */
int32_t cb_per_tensor_scratch_floats(void);
int32_t cb_quantize_per_tensor_fp8(const void* x, int32_t dtype, int64_t n, float eps, void* q, float* scale,
                                   float* amax_scratch, void* stream);

/* replaces dequantize_per_tensor_fp8(q, scale, out_dtype) -> y
 *   cublade/kernels/cuda/quantization/dequantize_per_tensor_fp8.cu:84-115
 *   (binding cublade/bindings/cuda/dequantize_fp8.py:15-35)
 * y = out_dtype_rn(float(q) * scale[0]); out_dtype CB_F16 / CB_BF16. */
int32_t cb_dequantize_per_tensor_fp8(const void* q, const float* scale, int64_t n, int32_t out_dtype, void* y,
                                     void* stream);

/* ------------------------------------------------------------------------
 * INT8, symmetric, codes in [-127, 127].
 * inv = fp32(127 / max(amax, eps)); q = clamp(rint(float(x) * inv)); scale = fp32(1 / inv).
 * ------------------------------------------------------------------------ */
/* replaces quantize_per_tensor_int8(x, eps)
 *   cublade/kernels/cuda/quantization/quantize_int8.cu:470-484 (binding quantize_int8.py:18-38)
 * x: CB_F16 / CB_BF16 / CB_F32.  amax_scratch as for the FP8 call. */
int32_t cb_quantize_per_tensor_int8(const void* x, int32_t dtype, int64_t n, float eps, void* q, float* scale,
                                    float* amax_scratch, void* stream);

/* replaces quantize_per_channel_int8(x, eps): x viewed as [C, F], one scale per row
 *   cublade/kernels/cuda/quantization/quantize_int8.cu:487-509 (binding quantize_int8.py:41-62)
 * Like the reference, rejects F * sizeof(element) % 16 != 0 with CB_ERR_ALIGNMENT. scale: fp32[C]. */
int32_t cb_quantize_per_channel_int8(const void* x, int32_t dtype, int64_t C, int64_t F, float eps, void* q,
                                     float* scale, void* stream);

/* replaces quantize_per_group_int8(x_grouped, group_size, eps): x is [num_groups, group_size]
 *   cublade/kernels/cuda/quantization/quantize_int8.cu:514-536 (binding quantize_int8.py:65-87)
 * group_size in (0, 4096] else CB_ERR_RANGE.  scale: fp32[num_groups]. */
int32_t cb_quantize_per_group_int8(const void* x, int32_t dtype, int64_t num_groups, int64_t group_size, float eps,
                                   void* q, float* scale, void* stream);

/* replaces dequantize_per_tensor_int8(q, scale, out_dtype)
 *   cublade/kernels/cuda/quantization/dequantize_int8.cu:210-224 (binding dequantize_int8.py:18-38) */
int32_t cb_dequantize_per_tensor_int8(const void* q, const float* scale, int64_t n, int32_t out_dtype, void* y,
                                      void* stream);

/* replaces dequantize_per_channel_int8(q, scale, out_dtype): q is [C, F], scale fp32[C]
 *   cublade/kernels/cuda/quantization/dequantize_int8.cu:226-247 (binding dequantize_int8.py:41-58)
 * Like the reference, rejects F % 8 != 0 with CB_ERR_ALIGNMENT. */
int32_t cb_dequantize_per_channel_int8(const void* q, const float* scale, int64_t C, int64_t F, int32_t out_dtype,
                                       void* y, void* stream);

/* replaces dequantize_per_group_int8(q_grouped, scale, group_size, out_dtype)
 *   cublade/kernels/cuda/quantization/dequantize_int8.cu:249-273 (binding dequantize_int8.py:61-79) */
int32_t cb_dequantize_per_group_int8(const void* q, const float* scale, int64_t num_groups, int64_t group_size,
                                     int32_t out_dtype, void* y, void* stream);

/* ------------------------------------------------------------------------
 * Split-phase per-tensor quantization, for tensors sharded over several GPUs:
 * every rank runs cb_amax_abs on its shard, the caller max-reduces the fp32
 * value across ranks, every rank runs cb_cast_per_tensor with the global amax.
 * The two phases are the two kernels of the reference's single call
 *   cublade/kernels/cuda/quantization/quantize_per_tensor_fp8.cu:140-159
 *   cublade/kernels/cuda/quantization/quantize_int8.cu:394-410
 * cb_amax_abs: amax[0] = max(amax[0], max|x|); the caller zeroes amax first.
 * cb_cast_per_tensor: code_kind 0 = int8, 1 = e4m3.
 * ------------------------------------------------------------------------ */
int32_t cb_amax_abs(const void* x, int32_t dtype, int64_t n, float* amax, void* stream);
int32_t cb_cast_per_tensor(const void* x, int32_t dtype, int64_t n, const float* amax, float eps, int32_t code_kind,
                           void* q, float* scale, void* stream);

/* The exchange between the two phases over NVLink peer memory instead of a collective call.  No counterpart in the
 * reference (it has no multi-GPU path).  Every rank owns a state array of cb_peer_exchange_state_bytes() bytes that
 * all ranks of the node have mapped (CUDA IPC / VMM; zeroed once, followed by a barrier, before the first call) and
 * passes the mapped addresses of all ranks' arrays, its own included, as peer_state[0..world).  One launch per rank
 * and exchange: out_amax[0] = max over the ranks of local_amax[0].  The ranks' kernels wait for one another (bounded:
 * about a second, then NaN is written and the error word of cb_device_error_state is raised), so every rank must be
 * a process on a GPU of its own; world <= cb_peer_exchange_max_ranks(). */
int32_t cb_peer_exchange_state_bytes(void);
int32_t cb_peer_exchange_max_ranks(void);
int32_t cb_amax_peer_exchange(const float* local_amax, const void* const* peer_state, int32_t rank, int32_t world,
                              float* out_amax, void* stream);

/* ------------------------------------------------------------------------
 * W8A16 linear:  y[m, n] = (sum_k x[m, k] * wq[n, k]) * scales[n]
 *                          (+ sum_j xo[m, j] * wo[n, j])  (+ bias[n])
 * replaces the forward of cuBladeW8A16LinearLayer
 *   cublade/quantization/linear.py:83-137 and the Triton GEMM it calls
 *   cublade/bindings/triton/matmul.py:17-132, cublade/kernels/triton/matmul_kernel.py:9-99
 * x [M, K] and y [M, N] are CB_BF16 or CB_F16 (act_dtype), rows ldx / ldy
 * elements apart.  wq [N, K] int8 row-major.  scales [N] of scales_dtype.
 * bias [N] of bias_dtype or NULL.  xo [M, KO] / wo [N, KO] (act_dtype, KO may
 * be 0 with NULL pointers) carry the LLM.int8 outlier columns kept in 16-bit.
 * fp32 accumulation; the result is rounded to act_dtype where the reference's chain of kernels materialises a
 * tensor: r(r(acc) * r(scales)), then r(. + r(outlier product)), then r(. + r(bias)) -- linear.py:97-135 -- so it
 * equals the reference's output up to the order of the fp32 accumulation.
 * path: 0 auto, 1 weight-streaming kernel, 2 tcgen05 CTA-pair kernel, 3 tcgen05 single-CTA kernel.
 * ------------------------------------------------------------------------ */
size_t cb_w8a16_workspace_bytes(int64_t M, int64_t N, int64_t K);
int32_t cb_w8a16_linear(const void* x, int64_t M, int64_t K, int64_t ldx, const void* wq, int64_t N,
                        const void* scales, int32_t scales_dtype, const void* bias, int32_t bias_dtype,
                        const void* xo, int64_t ldxo, const void* wo, int64_t KO, void* y, int64_t ldy,
                        int32_t act_dtype, void* workspace, size_t workspace_bytes, int32_t path, void* stream);

/* Every in-kernel wait of the tensor-core path is bounded; a kernel whose wait expired raises a
 * per-device flag and returns instead of hanging.  This call synchronises `stream` and copies the
 * flag (0 = never raised) to *host_flag.  No counterpart in the reference. */
int32_t cb_device_error_state(uint32_t* host_flag, void* stream);

/* dst[m, j] = src[m, cols[j]]: re-packs activation columns for the outlier split
 * (the two fancy-index gathers of cublade/quantization/linear.py:101-102). elem_size 2 or 4. */
int32_t cb_gather_columns(const void* src, int64_t M, int64_t ld_src, const int64_t* cols, int64_t ncols, void* dst,
                          int64_t ld_dst, int32_t elem_size, void* stream);

/* The same gather with columns ncols .. ncols_padded - 1 of every dst row written as zero
 * (ncols <= ncols_padded <= ld_dst).  The tensor-core kernels behind cb_w8a16_linear load the int8
 * rows with TMA, which needs a row stride of K % 16 == 0 bytes; the LLM.int8 split leaves
 * K = in_features - n_outliers (cublade/quantization/linear.py:48-66), rarely such a multiple.  A caller
 * keeps a copy of the int8 weights with zero columns up to the next multiple of 16, re-packs the
 * activations with this call to the same width and passes the padded K: the zero columns add nothing. */
int32_t cb_gather_columns_padded(const void* src, int64_t M, int64_t ld_src, const int64_t* cols, int64_t ncols,
                                 int64_t ncols_padded, void* dst, int64_t ld_dst, int32_t elem_size, void* stream);

/* ------------------------------------------------------------------------
 * Dense GEMM  C[M, N] = A[M, K] . B[K, N], all row-major, on tcgen05 / TMEM.
 * replaces wmma_gemm(A, B, acc_dtype)
 *   cublade/kernels/cuda/wmma.cu:184-262 (kernel :29-182; binding cublade/bindings/cuda/wmma.py:16-47)
 * in_kind: 0 fp16, 1 bf16, 2 int8, 3 uint8 (A and B of the same type).
 * out_kind (type of C): 0 fp32 (fp16 / bf16 inputs), 1 fp16 (fp16 inputs; fp32 accumulation, one rounding),
 *   2 int32 (8-bit inputs, exact).  Other pairings -> CB_ERR_DTYPE, as the reference rejects them.
 * Unlike the reference M, N, K need not be multiples of 16.  workspace: cb_gemm_workspace_bytes(N, K,
 * in_kind) bytes (B is transposed into it once per call); without it, or when K * sizeof(element) is not
 * a multiple of 16, a plain CUDA-core kernel computes the product.
 * ------------------------------------------------------------------------ */
size_t cb_gemm_workspace_bytes(int64_t N, int64_t K, int32_t in_kind);
int32_t cb_gemm(const void* a, const void* b, int64_t M, int64_t N, int64_t K, int32_t in_kind, void* c, int64_t ldc,
                int32_t out_kind, void* workspace, size_t workspace_bytes, void* stream);

/* C[M, N] = activation(A[M, K] . B[K, N]) with C in the INPUT type, the contract of the reference's generic wrapper
 *   matmul(A, B, activation="", override_config=None, use_autotune=True)  cublade/bindings/triton/matmul.py:17-132
 *   (kernel cublade/kernels/triton/matmul_kernel.py:9-105: accumulate, optional leaky_relu on the accumulator,
 *   one cast to the output type)
 * in_kind 0 fp16 -> fp16, 1 bf16 -> bf16 (fp32 accumulation), 2 int8 -> int32 (activation ignored, as there).
 * activation: 0 none, 1 leaky_relu (x >= 0 ? x : 0.01 x).  The reference's tuning arguments have no meaning here.
 * Its float32 and float8_e5m2 inputs are not served (CB_ERR_DTYPE).  workspace as for cb_gemm. */
int32_t cb_matmul(const void* a, const void* b, int64_t M, int64_t N, int64_t K, int32_t in_kind, void* c, int64_t ldc,
                  int32_t activation, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * W4A16 linear: 4-bit symmetric weights (codes in [-7, 7], one scale per output feature), 16-bit activations,
 * fp32 accumulation:   y[m, n] = T( (sum_k x[m, k] * code[n, k]) * scales[n] + bias[n] )
 * The reference reserves the layer type "w4a16" (registry comment, cublade/quantization/quantizers.py:169-171)
 * and has no kernel, layer or storage format for it.
 * Packed weights wq4 [N, K / 2] bytes (K % 8 == 0): 32-bit word i of a row holds the codes k = 8i .. 8i + 7 as
 * two's-complement nibbles, byte j = code(8i + j) | code(8i + 4 + j) << 4.
 * cb_w4_quantize_rows: w [N, K] of dtype -> packed + scale_out [N] float32, the arithmetic of the reference's
 *   per-channel INT8 quantizer (cublade/kernels/cuda/quantization/quantize_int8.cu:245-296) with qmax = 7.
 * cb_w4_unpack: packed -> int8 codes [N, K].
 * cb_w4a16_linear: M <= 16 with K % 128 == 0, N % 16 == 0 and 16-byte aligned rows streams the packed weights
 *   once (no workspace); every other shape unpacks into `workspace` (cb_w4a16_workspace_bytes(M, N, K) bytes,
 *   16-byte aligned) and runs the W8A16 path.  Too small a workspace -> CB_ERR_ARGUMENT.
 * ------------------------------------------------------------------------ */
int32_t cb_w4_quantize_rows(const void* w, int32_t dtype, int64_t N, int64_t K, float eps, void* packed, float* scale_out,
                            void* stream);
int32_t cb_w4_unpack(const void* packed, int64_t N, int64_t K, void* codes_int8, void* stream);
size_t cb_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K);
int32_t cb_w4a16_linear(const void* x, int32_t act_dtype, int64_t M, int64_t K, int64_t ldx, const void* wq4, int64_t N,
                        const void* scales, int32_t scales_dtype, const void* bias, int32_t bias_dtype, void* y,
                        int64_t ldy, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * W8A8 linear on the integer tensor cores (tcgen05 kind::i8, exact int32 accumulation):
 *   y[m, n] = T( (float(sum_k xq[m, k] * wq[n, k]) * x_scales[m]) * w_scales[n] + bias[n] )
 * The layer type the reference reserves as "w8a8" (cublade/quantization/quantizers.py:169-171) and does
 * not implement.  xq [M, K] int8 row-major with x_scales fp32[M] (per token -- e.g. the outputs of
 * cb_quantize_per_channel_int8 on [M, K] or of cb_rmsnorm_quantize); wq [N, K] int8 row-major with
 * w_scales [N]; bias [N] or NULL; y [M, N] CB_BF16 / CB_F16, rows ldy apart.  Products are evaluated
 * in the order written, every operation a single IEEE fp32 operation, one rounding to T at the end.
 * K % 16 == 0 with 16-byte aligned xq / wq runs on the tensor cores, anything else on a plain kernel.
 * ------------------------------------------------------------------------ */
int32_t cb_w8a8_linear(const void* xq, const float* x_scales, int64_t M, int64_t K, const void* wq, int64_t N,
                       const void* w_scales, int32_t w_scales_dtype, const void* bias, int32_t bias_dtype, void* y,
                       int64_t ldy, int32_t out_dtype, void* stream);

/* ------------------------------------------------------------------------
 * INT8 per-channel along ANY axis, in place: x contiguous, viewed as [outer, C, inner] with C the
 * channel axis.  Same arithmetic per channel as cb_quantize_per_channel_int8, so the result equals
 * "move the axis to the front, quantize per channel, move it back" bit for bit -- without the copy.
 * The reference advertises the mode (README.md:16) but rejects every axis but 0
 *   cublade/quantization/quantizers.py:117-120, cublade/quantization/dequantizers.py:51-53
 * scale: fp32[C].  scratch: C floats of device memory, overwritten.  Two passes over x
 * (per-channel amax by atomicMax, then the cast); no alignment or divisibility requirement
 * (vector kernels when inner % lanes == 0, or inner == 1 and C % lanes == 0, with 16-byte aligned x).
 * ------------------------------------------------------------------------ */
int32_t cb_quantize_per_axis_int8(const void* x, int32_t dtype, int64_t outer, int64_t C, int64_t inner, float eps, void* q,
                                  float* scale, float* scratch, void* stream);
int32_t cb_dequantize_per_axis_int8(const void* q, const float* scale, int64_t outer, int64_t C, int64_t inner,
                                    int32_t out_dtype, void* y, void* stream);

/* ------------------------------------------------------------------------
 * INT8 per-group with the groups along a NON-LAST axis, in place: x contiguous, viewed as
 * [outer, C, inner]; group_size consecutive indices of C form a group at every (outer, inner)
 * position; group_size in (0, 4096] must divide C.  Same arithmetic per group as
 * cb_quantize_per_group_int8 and the same scale order as the reference's route
 *   cublade/quantization/quantizers.py:122-132 (movedim(ch_axis, -1).contiguous().view(-1, G), kernel,
 *   view back, movedim(-1, ch_axis).contiguous()), cublade/quantization/dequantizers.py:58-72
 * i.e. scale fp32[outer * inner * C / group_size] with index (o * inner + i) * (C / group_size) + c / group_size,
 * so codes, scales and dequantized values equal that route's bit for bit -- without its two
 * transposing copies (3 bytes of HBM traffic per element instead of 9).  No alignment requirement
 * (vector kernels when inner is a multiple of the 16-byte lane count and x is 16-byte aligned).
 * ------------------------------------------------------------------------ */
int32_t cb_quantize_per_group_axis_int8(const void* x, int32_t dtype, int64_t outer, int64_t C, int64_t inner,
                                        int64_t group_size, float eps, void* q, float* scale, void* stream);
int32_t cb_dequantize_per_group_axis_int8(const void* q, const float* scale, int64_t outer, int64_t C, int64_t inner,
                                          int64_t group_size, int32_t out_dtype, void* y, void* stream);

/* ------------------------------------------------------------------------
 * Fused RMSNorm -> per-row (per-token) quantize: one pass over x, 3 bytes of HBM traffic per
 * element instead of the 7 of "RMSNorm kernel, then per-channel quantize kernel".
 * The reference announces the op (README.md:20, "upcoming RMSNorm-fused-quant work" for which its
 * DTypeTraits / Pack16 headers, cublade/kernels/cuda/quantization/int8_pack.cuh:23-100, are meant)
 * but does not implement it; the second half is the arithmetic of
 * cublade/kernels/cuda/quantization/quantize_int8.cu:173-297 (per-channel, axis 0).
 *   x [rows, hidden] CB_F16 / CB_BF16, contiguous.  gamma [hidden] of the same dtype or NULL.
 *   r = 1 / sqrt(mean(x^2) + rms_eps);  n = T(x * r);  y = T(n * gamma);
 *   inv = qmax / max(max|y|, q_eps);  q = code(float(y) * inv);  scale[row] = 1 / inv
 *   code_kind 0: int8 (qmax 127, codes in [-127, 127]); 1: e4m3 (qmax 448).
 *   q [rows, hidden] bytes; scale fp32[rows]; y_out [rows, hidden] in x's dtype receives y, or NULL;
 *   rstd_out fp32[rows] receives r, or NULL.
 * Any hidden and alignment are served; rows of hidden % 8 == 0, hidden <= 16384 with 16-byte
 * aligned pointers take the register-resident one-pass kernel.
 * ------------------------------------------------------------------------ */
int32_t cb_rmsnorm_quantize(const void* x, int32_t dtype, int64_t rows, int64_t hidden, const void* gamma, float rms_eps,
                            float q_eps, int32_t code_kind, void* q, float* scale, void* y_out, float* rstd_out,
                            void* stream);

/* ------------------------------------------------------------------------
 * LLM.int8 W8A16 linear for callers that cannot allocate device memory.
 * No counterpart in the reference (which allocates freely through torch).
 *
 * Same result as: cb_gather_columns(x, normal_cols) ; cb_gather_columns(x, outlier_cols) ;
 * cb_w8a16_linear(...), but the two re-packed activation buffers live in a 16 MiB array that is
 * part of the library's device image (every GPU that loads the library holds it until exit), so
 * the call needs nothing but its inputs and its output and makes no cudaMalloc / cudaFree.
 *   x [M, K] activations (act_dtype, row stride ldx);  normal_cols int64[K - KO] and
 *   outlier_cols int64[KO] are DEVICE arrays of column indices;  wq int8 [N, K - KO];
 *   wo [N, KO] in act_dtype;  y [M, N].
 * Limit: M * (round_up(K - KO, 8) + round_up(KO, 8)) * 2 bytes <= cb_static_scratch_bytes(),
 *   otherwise CB_ERR_RANGE with an explanatory cb_static_last_error(); nothing is launched.
 *   What the two buffers leave of the array is handed to the GEMM as its workspace.
 * The first call on a device resolves the array's address; issue it before any stream capture.
 * All calls on a device share the array: it keeps the last call's contents (each call writes
 * what it reads, nothing must be pre-zeroed) and calls that overlap on the GPU race on it.
 * ------------------------------------------------------------------------ */
size_t cb_static_scratch_bytes(void);
const char* cb_static_last_error(void);
int32_t cb_w8a16_linear_outlier_static(const void* x, int64_t M, int64_t K, int64_t ldx, const int64_t* normal_cols,
                                       const int64_t* outlier_cols, int64_t KO, const void* wq, int64_t N,
                                       const void* scales, int32_t scales_dtype, const void* bias, int32_t bias_dtype,
                                       const void* wo, void* y, int64_t ldy, int32_t act_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CUBLADE_B200_H_ */
