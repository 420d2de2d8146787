// extern "C" surface of libcublade_b200.so: argument validation, error text,
// launch accounting.  The declarations and the reference interface each entry
// point replaces live in include/cublade_b200.h.

#include "../../include/cublade_b200.h"
#include "launch.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>

namespace {

thread_local char g_err[512] = "";
std::atomic<int64_t> g_launches{0};

int32_t fail(cb_status st, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return (int32_t)st;
}

int32_t cuda_result(cudaError_t e, const char* what, int launches) {
    if (e != cudaSuccess) return fail(CB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    g_launches.fetch_add(launches, std::memory_order_relaxed);
    return CB_OK;
}

}  // namespace

namespace cb {
// entry points that live in other translation units account for their launches here
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
}  // namespace cb

namespace {

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool is_half_like(int32_t dt) { return dt == CB_F16 || dt == CB_BF16; }
inline bool is_float_like(int32_t dt) { return dt == CB_F16 || dt == CB_BF16 || dt == CB_F32; }

int32_t quantize_per_tensor(const char* name, const void* x, int32_t dtype, int64_t n, float eps, int code, void* q,
                            float* scale, float* amax, void* stream) {
    if (!scale || !amax || n < 0 || (n > 0 && (!x || !q))) return fail(CB_ERR_ARGUMENT, "%s: null pointer or n < 0", name);
    cudaStream_t s = as_stream(stream);
    // phase 1 writes one partial maximum per CTA into the scratch (no atomics, nothing to zero),
    // phase 2 folds them; for n == 0 the single slot is cleared so the scale is that of amax = 0
    int nparts = 0;
    cudaError_t e = cb::launch_amax_partials(x, dtype, n, amax, &nparts, s);
    if (e != cudaSuccess) return cuda_result(e, name, 0);
    if (nparts == 0) {
        e = cudaMemsetAsync(amax, 0, sizeof(float), s);
        if (e != cudaSuccess) return cuda_result(e, name, 0);
    }
    e = cb::launch_cast_tensor(x, dtype, n, amax, nparts, eps, code, q, scale, s);
    return cuda_result(e, name, n > 0 ? 2 : 1);
}

}  // namespace

extern "C" {

int32_t cb_version(void) { return 100; }
const char* cb_last_error(void) { return g_err; }
int64_t cb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int32_t cb_per_tensor_scratch_floats(void) { return cb::per_tensor_scratch_floats(); }

int32_t cb_quantize_per_tensor_fp8(const void* x, int32_t dtype, int64_t n, float eps, void* q, float* scale,
                                   float* amax_scratch, void* stream) {
    if (!is_half_like(dtype)) return fail(CB_ERR_DTYPE, "cb_quantize_per_tensor_fp8: x must be float16 or bfloat16");
    return quantize_per_tensor("cb_quantize_per_tensor_fp8", x, dtype, n, eps, cb::kCodeE4M3, q, scale, amax_scratch,
                               stream);
}

int32_t cb_quantize_per_tensor_int8(const void* x, int32_t dtype, int64_t n, float eps, void* q, float* scale,
                                    float* amax_scratch, void* stream) {
    if (!is_float_like(dtype))
        return fail(CB_ERR_DTYPE, "cb_quantize_per_tensor_int8: x must be float16, bfloat16 or float32");
    return quantize_per_tensor("cb_quantize_per_tensor_int8", x, dtype, n, eps, cb::kCodeInt8, q, scale, amax_scratch,
                               stream);
}

int32_t cb_amax_abs(const void* x, int32_t dtype, int64_t n, float* amax, void* stream) {
    if (!is_float_like(dtype)) return fail(CB_ERR_DTYPE, "cb_amax_abs: bad dtype");
    if (!amax || n < 0 || (n > 0 && !x)) return fail(CB_ERR_ARGUMENT, "cb_amax_abs: null pointer or n < 0");
    return cuda_result(cb::launch_amax_tensor(x, dtype, n, amax, as_stream(stream)), "cb_amax_abs", n > 0 ? 1 : 0);
}

int32_t cb_peer_exchange_state_bytes(void) { return cb::peer_exchange_state_words() * 8; }
int32_t cb_peer_exchange_max_ranks(void) { return cb::peer_exchange_max_ranks(); }

int32_t cb_amax_peer_exchange(const float* local_amax, const void* const* peer_state, int32_t rank, int32_t world,
                              float* out_amax, void* stream) {
    const char* name = "cb_amax_peer_exchange";
    if (!local_amax || !peer_state || !out_amax) return fail(CB_ERR_ARGUMENT, "%s: null pointer", name);
    if (world < 1 || world > cb::peer_exchange_max_ranks() || rank < 0 || rank >= world)
        return fail(CB_ERR_RANGE, "%s: rank %d / world %d outside 1..%d", name, (int)rank, (int)world,
                    cb::peer_exchange_max_ranks());
    return cuda_result(cb::launch_amax_peer_exchange(local_amax, peer_state, rank, world, out_amax, as_stream(stream)),
                       name, 1);
}

int32_t cb_cast_per_tensor(const void* x, int32_t dtype, int64_t n, const float* amax, float eps, int32_t code_kind,
                           void* q, float* scale, void* stream) {
    if (!is_float_like(dtype)) return fail(CB_ERR_DTYPE, "cb_cast_per_tensor: bad dtype");
    if (code_kind != cb::kCodeInt8 && code_kind != cb::kCodeE4M3)
        return fail(CB_ERR_ARGUMENT, "cb_cast_per_tensor: code_kind must be 0 (int8) or 1 (e4m3)");
    if (code_kind == cb::kCodeE4M3 && !is_half_like(dtype))
        return fail(CB_ERR_DTYPE, "cb_cast_per_tensor: e4m3 needs float16 or bfloat16 input");
    if (!amax || !scale || n < 0 || (n > 0 && (!x || !q)))
        return fail(CB_ERR_ARGUMENT, "cb_cast_per_tensor: null pointer or n < 0");
    return cuda_result(cb::launch_cast_tensor(x, dtype, n, amax, 0, eps, code_kind, q, scale, as_stream(stream)),
                       "cb_cast_per_tensor", 1);
}

int32_t cb_quantize_per_channel_int8(const void* x, int32_t dtype, int64_t C, int64_t F, float eps, void* q,
                                     float* scale, void* stream) {
    if (!is_float_like(dtype))
        return fail(CB_ERR_DTYPE, "cb_quantize_per_channel_int8: x must be float16, bfloat16 or float32");
    if (C < 0 || F < 0) return fail(CB_ERR_ARGUMENT, "cb_quantize_per_channel_int8: negative size");
    if ((F * cb::dtype_size(dtype)) % 16 != 0)
        return fail(CB_ERR_ALIGNMENT,
                    "per-channel quant requires inner stride F * element_size to be a multiple of 16; got F=%lld "
                    "element_size=%d",
                    (long long)F, cb::dtype_size(dtype));
    if (C == 0 || F == 0) return CB_OK;
    if (!x || !q || !scale) return fail(CB_ERR_ARGUMENT, "cb_quantize_per_channel_int8: null pointer");
    return cuda_result(cb::launch_quant_segments(x, dtype, C, F, eps, cb::kCodeInt8, q, scale, as_stream(stream)),
                       "cb_quantize_per_channel_int8", 1);
}

int32_t cb_quantize_per_group_int8(const void* x, int32_t dtype, int64_t num_groups, int64_t group_size, float eps,
                                   void* q, float* scale, void* stream) {
    if (!is_float_like(dtype))
        return fail(CB_ERR_DTYPE, "cb_quantize_per_group_int8: x must be float16, bfloat16 or float32");
    if (group_size <= 0 || group_size > 4096) return fail(CB_ERR_RANGE, "group_size must be in (0, 4096]");
    if (num_groups < 0) return fail(CB_ERR_ARGUMENT, "cb_quantize_per_group_int8: negative size");
    if (num_groups == 0) return CB_OK;
    if (!x || !q || !scale) return fail(CB_ERR_ARGUMENT, "cb_quantize_per_group_int8: null pointer");
    return cuda_result(
        cb::launch_quant_segments(x, dtype, num_groups, group_size, eps, cb::kCodeInt8, q, scale, as_stream(stream)),
        "cb_quantize_per_group_int8", 1);
}

static int32_t dequant_common(const char* name, const void* q, int code, const float* scale, int64_t n,
                              int64_t seg_len, int32_t out_dtype, void* y, void* stream) {
    if (!is_half_like(out_dtype)) return fail(CB_ERR_DTYPE, "%s: out_dtype must be float16 or bfloat16", name);
    if (n < 0) return fail(CB_ERR_ARGUMENT, "%s: negative size", name);
    if (n == 0) return CB_OK;
    if (!q || !scale || !y) return fail(CB_ERR_ARGUMENT, "%s: null pointer", name);
    return cuda_result(cb::launch_dequant(q, code, scale, n, seg_len, out_dtype, y, as_stream(stream)), name, 1);
}

int32_t cb_dequantize_per_tensor_fp8(const void* q, const float* scale, int64_t n, int32_t out_dtype, void* y,
                                     void* stream) {
    return dequant_common("cb_dequantize_per_tensor_fp8", q, cb::kCodeE4M3, scale, n, 0, out_dtype, y, stream);
}

int32_t cb_dequantize_per_tensor_int8(const void* q, const float* scale, int64_t n, int32_t out_dtype, void* y,
                                      void* stream) {
    return dequant_common("cb_dequantize_per_tensor_int8", q, cb::kCodeInt8, scale, n, 0, out_dtype, y, stream);
}

int32_t cb_dequantize_per_channel_int8(const void* q, const float* scale, int64_t C, int64_t F, int32_t out_dtype,
                                       void* y, void* stream) {
    if (C < 0 || F < 0) return fail(CB_ERR_ARGUMENT, "cb_dequantize_per_channel_int8: negative size");
    if (F % 8 != 0)
        return fail(CB_ERR_ALIGNMENT,
                    "per-channel dequant requires inner stride F to be a multiple of 8; got F=%lld", (long long)F);
    return dequant_common("cb_dequantize_per_channel_int8", q, cb::kCodeInt8, scale, C * F, F, out_dtype, y, stream);
}

int32_t cb_dequantize_per_group_int8(const void* q, const float* scale, int64_t num_groups, int64_t group_size,
                                     int32_t out_dtype, void* y, void* stream) {
    if (group_size <= 0 || group_size > 4096) return fail(CB_ERR_RANGE, "group_size must be in (0, 4096]");
    if (num_groups < 0) return fail(CB_ERR_ARGUMENT, "cb_dequantize_per_group_int8: negative size");
    return dequant_common("cb_dequantize_per_group_int8", q, cb::kCodeInt8, scale, num_groups * group_size,
                          group_size, out_dtype, y, stream);
}

size_t cb_w8a16_workspace_bytes(int64_t M, int64_t N, int64_t K) { return cb::w8a16_workspace_bytes(M, N, K); }

int32_t cb_w8a16_linear(const void* x, int64_t M, int64_t K, int64_t ldx, const void* wq, int64_t N,
                        const void* scales, int32_t scales_dtype, const void* bias, int32_t bias_dtype,
                        const void* xo, int64_t ldxo, const void* wo, int64_t KO, void* y, int64_t ldy,
                        int32_t act_dtype, void* workspace, size_t workspace_bytes, int32_t path, void* stream) {
    if (!is_half_like(act_dtype)) return fail(CB_ERR_DTYPE, "cb_w8a16_linear: activations must be float16 or bfloat16");
    if (!is_float_like(scales_dtype)) return fail(CB_ERR_DTYPE, "cb_w8a16_linear: bad scales dtype");
    if (bias && !is_float_like(bias_dtype)) return fail(CB_ERR_DTYPE, "cb_w8a16_linear: bad bias dtype");
    if (M < 0 || N < 0 || K < 0 || KO < 0) return fail(CB_ERR_ARGUMENT, "cb_w8a16_linear: negative size");
    if (M == 0 || N == 0) return CB_OK;
    if (!x || !wq || !scales || !y) return fail(CB_ERR_ARGUMENT, "cb_w8a16_linear: null pointer");
    if (KO > 0 && (!xo || !wo)) return fail(CB_ERR_ARGUMENT, "cb_w8a16_linear: KO > 0 needs xo and wo");
    if (ldx < K || ldy < N || (KO > 0 && ldxo < KO)) return fail(CB_ERR_ARGUMENT, "cb_w8a16_linear: row stride too small");
    if (path < 0 || path > 3) return fail(CB_ERR_ARGUMENT, "cb_w8a16_linear: path must be 0, 1, 2 or 3");
    const size_t need = cb::w8a16_workspace_bytes(M, N, K);
    if (need > 0 && (!workspace || workspace_bytes < need))
        return fail(CB_ERR_WORKSPACE, "cb_w8a16_linear: workspace of %zu bytes required", need);
    cb::W8A16Args a;
    a.x = x; a.M = M; a.K = K; a.ldx = ldx;
    a.wq = static_cast<const int8_t*>(wq); a.N = N;
    a.scales = scales; a.scales_dtype = scales_dtype;
    a.bias = bias; a.bias_dtype = bias_dtype;
    a.xo = KO > 0 ? xo : nullptr; a.wo = KO > 0 ? wo : nullptr; a.KO = KO; a.ldxo = ldxo;
    a.y = y; a.ldy = ldy; a.act_dtype = act_dtype;
    a.workspace = workspace; a.workspace_bytes = workspace_bytes;
    cudaError_t e = cb::launch_w8a16(a, path, as_stream(stream));
    if (e == cudaErrorNotSupported)
        return fail(CB_ERR_UNSUPPORTED, "cb_w8a16_linear: shape/alignment not supported by the requested path");
    return cuda_result(e, "cb_w8a16_linear", 1);
}

int32_t cb_device_error_state(uint32_t* host_flag, void* stream) {
    if (!host_flag) return fail(CB_ERR_ARGUMENT, "cb_device_error_state: null pointer");
    unsigned int v = 0;
    cudaError_t e = cb::w8a16_tc_read_error(&v, as_stream(stream));
    if (e != cudaSuccess) return cuda_result(e, "cb_device_error_state", 0);
    *host_flag = v;
    return CB_OK;
}

int32_t cb_gather_columns(const void* src, int64_t M, int64_t ld_src, const int64_t* cols, int64_t ncols, void* dst,
                          int64_t ld_dst, int32_t elem_size, void* stream) {
    if (M < 0 || ncols < 0) return fail(CB_ERR_ARGUMENT, "cb_gather_columns: negative size");
    if (elem_size != 2 && elem_size != 4) return fail(CB_ERR_ARGUMENT, "cb_gather_columns: elem_size must be 2 or 4");
    if (M == 0 || ncols == 0) return CB_OK;
    if (!src || !cols || !dst) return fail(CB_ERR_ARGUMENT, "cb_gather_columns: null pointer");
    return cuda_result(cb::launch_gather_cols(src, M, ld_src, cols, ncols, ncols, dst, ld_dst, elem_size,
                                              as_stream(stream)),
                       "cb_gather_columns", 1);
}

int32_t cb_gather_columns_padded(const void* src, int64_t M, int64_t ld_src, const int64_t* cols, int64_t ncols,
                                 int64_t ncols_padded, void* dst, int64_t ld_dst, int32_t elem_size, void* stream) {
    if (M < 0 || ncols < 0 || ncols_padded < ncols || ld_dst < ncols_padded)
        return fail(CB_ERR_ARGUMENT, "cb_gather_columns_padded: need 0 <= ncols <= ncols_padded <= ld_dst");
    if (elem_size != 2 && elem_size != 4) return fail(CB_ERR_ARGUMENT, "cb_gather_columns_padded: elem_size must be 2 or 4");
    if (M == 0 || ncols_padded == 0) return CB_OK;
    if (!src || (ncols > 0 && !cols) || !dst) return fail(CB_ERR_ARGUMENT, "cb_gather_columns_padded: null pointer");
    return cuda_result(cb::launch_gather_cols(src, M, ld_src, cols, ncols, ncols_padded, dst, ld_dst, elem_size,
                                              as_stream(stream)),
                       "cb_gather_columns_padded", 1);
}

size_t cb_gemm_workspace_bytes(int64_t N, int64_t K, int32_t in_kind) {
    if (N <= 0 || K <= 0 || in_kind < 0 || in_kind > 3) return 0;
    return cb::tc_gemm_workspace_bytes(N, K, in_kind);
}

int32_t cb_gemm(const void* a, const void* b, int64_t M, int64_t N, int64_t K, int32_t in_kind, void* c, int64_t ldc,
                int32_t out_kind, void* workspace, size_t workspace_bytes, void* stream) {
    if (in_kind < 0 || in_kind > 3) return fail(CB_ERR_DTYPE, "cb_gemm: in_kind must be 0 (fp16), 1 (bf16), 2 (int8) or 3 (uint8)");
    const bool integer = in_kind >= 2;
    if (integer ? out_kind != 2 : !(out_kind == 0 || (out_kind == 1 && in_kind == 0)))
        return fail(CB_ERR_DTYPE, "cb_gemm: accumulator type does not go with the input type "
                                  "(fp16 -> fp32 or fp16, bf16 -> fp32, int8 / uint8 -> int32)");
    if (M < 0 || N < 0 || K < 0) return fail(CB_ERR_ARGUMENT, "cb_gemm: negative size");
    if (M == 0 || N == 0) return CB_OK;
    if (K == 0) return fail(CB_ERR_ARGUMENT, "cb_gemm: K must be positive");
    if (!a || !b || !c) return fail(CB_ERR_ARGUMENT, "cb_gemm: null pointer");
    if (ldc < N) return fail(CB_ERR_ARGUMENT, "cb_gemm: ldc < N");
    return cuda_result(cb::launch_tc_gemm(a, b, M, N, K, in_kind, c, ldc, out_kind, workspace, workspace_bytes,
                                          as_stream(stream)),
                       "cb_gemm", 2);
}

int32_t cb_matmul(const void* a, const void* b, int64_t M, int64_t N, int64_t K, int32_t in_kind, void* c, int64_t ldc,
                  int32_t activation, void* workspace, size_t workspace_bytes, void* stream) {
    if (in_kind < 0 || in_kind > 2) return fail(CB_ERR_DTYPE, "cb_matmul: in_kind must be 0 (fp16), 1 (bf16) or 2 (int8)");
    if (activation != 0 && activation != 1) return fail(CB_ERR_ARGUMENT, "cb_matmul: activation must be 0 (none) or 1 (leaky_relu)");
    if (M < 0 || N < 0 || K < 0) return fail(CB_ERR_ARGUMENT, "cb_matmul: negative size");
    if (M == 0 || N == 0) return CB_OK;
    if (K == 0) return fail(CB_ERR_ARGUMENT, "cb_matmul: K must be positive");
    if (!a || !b || !c) return fail(CB_ERR_ARGUMENT, "cb_matmul: null pointer");
    if (ldc < N) return fail(CB_ERR_ARGUMENT, "cb_matmul: ldc < N");
    // C has the input type for the float kinds (fp32 accumulation, one rounding), int32 for int8; the activation is
    // ignored for int8 as in the reference wrapper
    const int out_kind = in_kind == 0 ? 1 : in_kind == 1 ? 3 : 2;
    return cuda_result(cb::launch_tc_gemm(a, b, M, N, K, in_kind, c, ldc, out_kind, workspace, workspace_bytes,
                                          as_stream(stream), in_kind <= 1 ? activation : 0),
                       "cb_matmul", 2);
}

int32_t cb_w8a8_linear(const void* xq, const float* x_scales, int64_t M, int64_t K, const void* wq, int64_t N,
                       const void* w_scales, int32_t w_scales_dtype, const void* bias, int32_t bias_dtype, void* y,
                       int64_t ldy, int32_t out_dtype, void* stream) {
    if (out_dtype != CB_F16 && out_dtype != CB_BF16)
        return fail(CB_ERR_DTYPE, "cb_w8a8_linear: out_dtype must be float16 or bfloat16");
    if (!is_float_like(w_scales_dtype) || (bias && !is_float_like(bias_dtype)))
        return fail(CB_ERR_DTYPE, "cb_w8a8_linear: scales / bias must be float16, bfloat16 or float32");
    if (M < 0 || N < 0 || K < 0) return fail(CB_ERR_ARGUMENT, "cb_w8a8_linear: negative size");
    if (M == 0 || N == 0) return CB_OK;
    if (K == 0) return fail(CB_ERR_ARGUMENT, "cb_w8a8_linear: K must be positive");
    if (!xq || !x_scales || !wq || !w_scales || !y) return fail(CB_ERR_ARGUMENT, "cb_w8a8_linear: null pointer");
    if (ldy < N) return fail(CB_ERR_ARGUMENT, "cb_w8a8_linear: ldy < N");
    cb::W8A8Args a;
    a.xq = static_cast<const int8_t*>(xq); a.xs = x_scales; a.M = M; a.K = K;
    a.wq = static_cast<const int8_t*>(wq); a.N = N;
    a.ws = w_scales; a.ws_dtype = w_scales_dtype; a.bias = bias; a.bias_dtype = bias_dtype;
    a.y = y; a.ldy = ldy; a.out_dtype = out_dtype;
    return cuda_result(cb::launch_w8a8(a, as_stream(stream)), "cb_w8a8_linear", 1);
}

int32_t cb_w4_quantize_rows(const void* w, int32_t dtype, int64_t N, int64_t K, float eps, void* packed, float* scale_out,
                            void* stream) {
    if (!is_float_like(dtype)) return fail(CB_ERR_DTYPE, "cb_w4_quantize_rows: w must be float16, bfloat16 or float32");
    if (N < 0 || K < 0) return fail(CB_ERR_ARGUMENT, "cb_w4_quantize_rows: negative size");
    if (K % 8 != 0) return fail(CB_ERR_ARGUMENT, "cb_w4_quantize_rows: K must be a multiple of 8");
    if (N == 0 || K == 0) return CB_OK;
    if (!w || !packed || !scale_out) return fail(CB_ERR_ARGUMENT, "cb_w4_quantize_rows: null pointer");
    return cuda_result(cb::launch_w4_quantize_rows(w, dtype, N, K, eps, packed, scale_out, as_stream(stream)),
                       "cb_w4_quantize_rows", 1);
}

int32_t cb_w4_unpack(const void* packed, int64_t N, int64_t K, void* codes_int8, void* stream) {
    if (N < 0 || K < 0) return fail(CB_ERR_ARGUMENT, "cb_w4_unpack: negative size");
    if (K % 8 != 0) return fail(CB_ERR_ARGUMENT, "cb_w4_unpack: K must be a multiple of 8");
    if (N == 0 || K == 0) return CB_OK;
    if (!packed || !codes_int8) return fail(CB_ERR_ARGUMENT, "cb_w4_unpack: null pointer");
    if (reinterpret_cast<uintptr_t>(codes_int8) % 8) return fail(CB_ERR_ARGUMENT, "cb_w4_unpack: output must be 8-byte aligned");
    return cuda_result(cb::launch_w4_unpack(packed, N, K, static_cast<int8_t*>(codes_int8), as_stream(stream)),
                       "cb_w4_unpack", 1);
}

size_t cb_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K) { return cb::w4a16_workspace_bytes(M, N, K, false); }

int32_t cb_w4a16_linear(const void* x, int32_t act_dtype, int64_t M, int64_t K, int64_t ldx, const void* wq4, int64_t N,
                        const void* scales, int32_t scales_dtype, const void* bias, int32_t bias_dtype, void* y,
                        int64_t ldy, void* workspace, size_t workspace_bytes, void* stream) {
    if (!is_half_like(act_dtype)) return fail(CB_ERR_DTYPE, "cb_w4a16_linear: activations must be float16 or bfloat16");
    if (!is_float_like(scales_dtype) || (bias && !is_float_like(bias_dtype)))
        return fail(CB_ERR_DTYPE, "cb_w4a16_linear: scales / bias must be float16, bfloat16 or float32");
    if (M < 0 || N < 0 || K < 0) return fail(CB_ERR_ARGUMENT, "cb_w4a16_linear: negative size");
    if (M == 0 || N == 0) return CB_OK;
    if (K == 0 || K % 8 != 0) return fail(CB_ERR_ARGUMENT, "cb_w4a16_linear: K must be a positive multiple of 8");
    if (!x || !wq4 || !scales || !y) return fail(CB_ERR_ARGUMENT, "cb_w4a16_linear: null pointer");
    if (ldx < K || ldy < N) return fail(CB_ERR_ARGUMENT, "cb_w4a16_linear: row stride smaller than the row");
    cb::W4A16Args a;
    a.x = x; a.M = M; a.K = K; a.ldx = ldx; a.wq4 = wq4; a.N = N;
    a.scales = scales; a.scales_dtype = scales_dtype; a.bias = bias; a.bias_dtype = bias_dtype;
    a.y = y; a.ldy = ldy; a.act_dtype = act_dtype; a.workspace = workspace; a.workspace_bytes = workspace_bytes;
    int launches = 0;
    const cudaError_t e = cb::launch_w4a16(a, as_stream(stream), &launches);
    if (e == cudaErrorInvalidValue)
        return fail(CB_ERR_ARGUMENT, "cb_w4a16_linear: this shape needs cb_w4a16_workspace_bytes(M, N, K) bytes of 16-byte "
                                     "aligned workspace");
    return cuda_result(e, "cb_w4a16_linear", launches);
}

int32_t cb_quantize_per_axis_int8(const void* x, int32_t dtype, int64_t outer, int64_t C, int64_t inner, float eps, void* q,
                                  float* scale, float* scratch, void* stream) {
    if (!is_float_like(dtype)) return fail(CB_ERR_DTYPE, "cb_quantize_per_axis_int8: x must be float16, bfloat16 or float32");
    if (outer < 0 || C < 0 || inner < 0) return fail(CB_ERR_ARGUMENT, "cb_quantize_per_axis_int8: negative size");
    if (C == 0) return CB_OK;
    if (!scale || !scratch) return fail(CB_ERR_ARGUMENT, "cb_quantize_per_axis_int8: null scale or scratch");
    if (outer * inner > 0 && (!x || !q)) return fail(CB_ERR_ARGUMENT, "cb_quantize_per_axis_int8: null pointer");
    const int launches = outer * inner > 0 ? 3 : 1;
    return cuda_result(cb::launch_quant_axis(x, dtype, outer, C, inner, eps, q, scale, scratch, as_stream(stream)),
                       "cb_quantize_per_axis_int8", launches);
}

int32_t cb_dequantize_per_axis_int8(const void* q, const float* scale, int64_t outer, int64_t C, int64_t inner,
                                    int32_t out_dtype, void* y, void* stream) {
    if (out_dtype != CB_F16 && out_dtype != CB_BF16)
        return fail(CB_ERR_DTYPE, "cb_dequantize_per_axis_int8: out_dtype must be float16 or bfloat16");
    if (outer < 0 || C < 0 || inner < 0) return fail(CB_ERR_ARGUMENT, "cb_dequantize_per_axis_int8: negative size");
    if (outer * C * inner == 0) return CB_OK;
    if (!q || !scale || !y) return fail(CB_ERR_ARGUMENT, "cb_dequantize_per_axis_int8: null pointer");
    return cuda_result(cb::launch_dequant_axis(q, scale, outer, C, inner, out_dtype, y, as_stream(stream)),
                       "cb_dequantize_per_axis_int8", 1);
}

int32_t cb_quantize_per_group_axis_int8(const void* x, int32_t dtype, int64_t outer, int64_t C, int64_t inner,
                                        int64_t group_size, float eps, void* q, float* scale, void* stream) {
    const char* name = "cb_quantize_per_group_axis_int8";
    if (!is_float_like(dtype)) return fail(CB_ERR_DTYPE, "%s: x must be float16, bfloat16 or float32", name);
    if (group_size <= 0 || group_size > 4096) return fail(CB_ERR_RANGE, "group_size must be in (0, 4096]");
    if (outer < 0 || C < 0 || inner < 0) return fail(CB_ERR_ARGUMENT, "%s: negative size", name);
    if (C % group_size != 0) return fail(CB_ERR_ARGUMENT, "%s: group_size must divide C", name);
    if (outer * C * inner == 0) return CB_OK;
    if (!x || !q || !scale) return fail(CB_ERR_ARGUMENT, "%s: null pointer", name);
    return cuda_result(cb::launch_quant_group_axis(x, dtype, outer, C, inner, (int)group_size, eps, q, scale,
                                                   as_stream(stream)), name, 1);
}

int32_t cb_dequantize_per_group_axis_int8(const void* q, const float* scale, int64_t outer, int64_t C, int64_t inner,
                                          int64_t group_size, int32_t out_dtype, void* y, void* stream) {
    const char* name = "cb_dequantize_per_group_axis_int8";
    if (out_dtype != CB_F16 && out_dtype != CB_BF16) return fail(CB_ERR_DTYPE, "%s: out_dtype must be float16 or bfloat16", name);
    if (group_size <= 0 || group_size > 4096) return fail(CB_ERR_RANGE, "group_size must be in (0, 4096]");
    if (outer < 0 || C < 0 || inner < 0) return fail(CB_ERR_ARGUMENT, "%s: negative size", name);
    if (C % group_size != 0) return fail(CB_ERR_ARGUMENT, "%s: group_size must divide C", name);
    if (outer * C * inner == 0) return CB_OK;
    if (!q || !scale || !y) return fail(CB_ERR_ARGUMENT, "%s: null pointer", name);
    return cuda_result(cb::launch_dequant_group_axis(q, scale, outer, C, inner, (int)group_size, out_dtype, y,
                                                     as_stream(stream)), name, 1);
}

int32_t cb_rmsnorm_quantize(const void* x, int32_t dtype, int64_t rows, int64_t hidden, const void* gamma, float rms_eps,
                            float q_eps, int32_t code_kind, void* q, float* scale, void* y_out, float* rstd_out,
                            void* stream) {
    if (dtype != CB_F16 && dtype != CB_BF16)
        return fail(CB_ERR_DTYPE, "cb_rmsnorm_quantize: x must be float16 or bfloat16");
    if (code_kind != 0 && code_kind != 1) return fail(CB_ERR_ARGUMENT, "cb_rmsnorm_quantize: code_kind must be 0 (int8) or 1 (e4m3)");
    if (rows < 0 || hidden < 0) return fail(CB_ERR_ARGUMENT, "cb_rmsnorm_quantize: negative size");
    if (rows == 0 || hidden == 0) return CB_OK;
    if (!x || !q || !scale) return fail(CB_ERR_ARGUMENT, "cb_rmsnorm_quantize: null pointer");
    if (rows > 0x7fffffffLL) return fail(CB_ERR_RANGE, "cb_rmsnorm_quantize: more than 2^31 - 1 rows");
    return cuda_result(cb::launch_rmsnorm_quant(x, dtype, rows, hidden, gamma, rms_eps, q_eps,
                                                code_kind == 1 ? cb::kCodeE4M3 : cb::kCodeInt8, q, scale, y_out,
                                                rstd_out, as_stream(stream)),
                       "cb_rmsnorm_quantize", 1);
}

}  // extern "C"
