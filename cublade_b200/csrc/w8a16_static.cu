// cb_w8a16_linear_outlier_static: the LLM.int8 form of the W8A16 linear for callers that cannot
// allocate device memory.
//
// The ordinary route (cb_gather_columns twice into caller-allocated buffers, then cb_w8a16_linear)
// needs scratch for the re-packed activations: [M, K - KO] "normal" columns and [M, KO] outlier
// columns.  Some callers have nowhere to get that scratch from: a serving loop that runs inside a
// frozen memory pool, a plugin that is handed only its input and output tensors, code replayed
// under a runtime that forbids cudaMalloc on its hot path.  For them the scratch lives in this
// file as a fixed array in device memory, reserved when the library is loaded on a GPU and held
// until the process exits.  The entry point calls no cudaMalloc / cudaFree and no allocating
// library routine.
//
// Limits and rules (also in include/cublade_b200.h):
//   * M * (round_up(K - KO, 8) + round_up(KO, 8)) 16-bit elements must fit in kScratchBytes
//     (16 MiB); larger requests are refused with CB_ERR_RANGE and nothing is launched;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress);
//     make that first call outside any stream capture;
//   * all calls on one device share the array and it keeps the previous call's contents: every
//     element a call reads it has written first (nothing needs to start at zero), but two calls
//     that overlap on the GPU (different streams) race on it -- serialise them.

#include "../../include/cublade_b200.h"
#include "launch.h"

#include <cstdio>

namespace {

constexpr size_t kScratchBytes = 16u << 20;

// Device-resident scratch.  In host code this name is only a handle for cudaGetSymbolAddress;
// the pointer handed to kernels is the looked-up device address.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

unsigned char* scratch_for_current_device(cudaError_t* err) {
    // one slot per device; two host threads that fill a slot at the same time store the same address
    static unsigned char* cached[64] = {nullptr};
    int dev = 0;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= 64) {
        *err = cudaErrorInvalidDevice;
        return nullptr;
    }
    if (!cached[dev]) {
        void* p = nullptr;
        *err = cudaGetSymbolAddress(&p, g_scratch);
        if (*err != cudaSuccess) return nullptr;
        cached[dev] = static_cast<unsigned char*>(p);
    }
    return cached[dev];
}

thread_local char g_static_err[256] = "";

}  // namespace

extern "C" {

const char* cb_static_last_error(void) { return g_static_err; }

size_t cb_static_scratch_bytes(void) { return kScratchBytes; }

int32_t cb_w8a16_linear_outlier_static(const void* x, int64_t M, int64_t K, int64_t ldx, const int64_t* normal_cols,
                                       const int64_t* outlier_cols, int64_t KO, const void* wq, int64_t N,
                                       const void* scales, int32_t scales_dtype, const void* bias, int32_t bias_dtype,
                                       const void* wo, void* y, int64_t ldy, int32_t act_dtype, void* stream) {
    auto fail = [](int32_t code, const char* msg) {
        snprintf(g_static_err, sizeof(g_static_err), "%s", msg);
        return code;
    };
    if (act_dtype != CB_F16 && act_dtype != CB_BF16)
        return fail(CB_ERR_DTYPE, "cb_w8a16_linear_outlier_static: activations must be float16 or bfloat16");
    auto float_like = [](int32_t dt) { return dt == CB_F16 || dt == CB_BF16 || dt == CB_F32; };
    if (!float_like(scales_dtype))
        return fail(CB_ERR_DTYPE, "cb_w8a16_linear_outlier_static: bad scales dtype");
    if (bias && !float_like(bias_dtype))
        return fail(CB_ERR_DTYPE, "cb_w8a16_linear_outlier_static: bad bias dtype");
    if (M < 0 || N < 0 || K < 0 || KO < 0 || KO > K)
        return fail(CB_ERR_ARGUMENT, "cb_w8a16_linear_outlier_static: bad sizes");
    if (M == 0 || N == 0) return CB_OK;
    if (ldx < K || ldy < N)
        return fail(CB_ERR_ARGUMENT, "cb_w8a16_linear_outlier_static: row stride too small (need ldx >= K, ldy >= N)");
    if (!x || !wq || !scales || !y || (K - KO > 0 && !normal_cols) || (KO > 0 && (!outlier_cols || !wo)))
        return fail(CB_ERR_ARGUMENT, "cb_w8a16_linear_outlier_static: null pointer");
    const int64_t kn = K - KO;
    const int64_t ld_n = (kn + 7) / 8 * 8, ld_o = (KO + 7) / 8 * 8;
    // compared in divided form: M * (ld_n + ld_o) * 2 cannot wrap for any int64 sizes this way
    const bool fits = ld_n + ld_o == 0 || (uint64_t)M <= (uint64_t)(kScratchBytes / 2u) / (uint64_t)(ld_n + ld_o);
    const size_t need = fits ? (size_t)M * (size_t)(ld_n + ld_o) * 2u : ~(size_t)0;
    if (!fits) {
        snprintf(g_static_err, sizeof(g_static_err),
                 "cb_w8a16_linear_outlier_static: needs %zu bytes of scratch, the built-in scratch holds %zu "
                 "(M * (K rounded up per column set) * 2 must not exceed it); use cb_w8a16_linear with your own buffers",
                 need, kScratchBytes);
        return CB_ERR_RANGE;
    }
    cudaError_t e;
    unsigned char* scratch = scratch_for_current_device(&e);
    if (!scratch) {
        snprintf(g_static_err, sizeof(g_static_err), "cb_w8a16_linear_outlier_static: scratch lookup failed: %s",
                 cudaGetErrorString(e));
        return CB_ERR_CUDA;
    }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    void* xn = scratch;                                   // [M, ld_n]
    void* xo = scratch + (size_t)M * (size_t)ld_n * 2u;   // [M, ld_o]   (offset is a multiple of 16 bytes)
    int launches = 1;
    if (kn > 0) {
        e = cb::launch_gather_cols(x, M, ldx, normal_cols, kn, kn, xn, ld_n, 2, s);
        if (e != cudaSuccess) return fail(CB_ERR_CUDA, cudaGetErrorString(e));
        ++launches;
    }
    if (KO > 0) {
        e = cb::launch_gather_cols(x, M, ldx, outlier_cols, KO, KO, xo, ld_o, 2, s);
        if (e != cudaSuccess) return fail(CB_ERR_CUDA, cudaGetErrorString(e));
        ++launches;
    }
    cb::W8A16Args a;
    a.x = xn; a.M = M; a.K = kn; a.ldx = ld_n;
    a.wq = static_cast<const int8_t*>(wq); a.N = N;
    a.scales = scales; a.scales_dtype = scales_dtype;
    a.bias = bias; a.bias_dtype = bias_dtype;
    a.xo = KO > 0 ? xo : nullptr; a.wo = KO > 0 ? wo : nullptr; a.KO = KO; a.ldxo = ld_o;
    a.y = y; a.ldy = ldy; a.act_dtype = act_dtype;
    // what is left of the array behind the two re-packed buffers serves as the K-split workspace of the
    // tensor-core kernel; when it is too small that kernel simply does not split
    const size_t used = (need + 255u) & ~(size_t)255u;
    a.workspace = used < kScratchBytes ? scratch + used : nullptr;
    a.workspace_bytes = used < kScratchBytes ? kScratchBytes - used : 0;
    e = cb::launch_w8a16(a, 0, s);
    if (e != cudaSuccess) return fail(CB_ERR_CUDA, cudaGetErrorString(e));
    cb::count_launches(launches);
    return CB_OK;
}

}  // extern "C"
