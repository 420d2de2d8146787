// W8A16 dispatch: the weight-streaming kernel (w8a16_stream.cu) for skinny activations, the
// tcgen05 CTA-pair kernel (w8a16_tc2.cu) for tall ones, the single-CTA tcgen05 kernel
// (w8a16_tc.cu) when a pair cannot be used.
#include "launch.h"

namespace cb {

cudaError_t launch_w8a16_stream(const W8A16Args& a, cudaStream_t s);
cudaError_t launch_w8a16_tc(const W8A16Args& a, cudaStream_t s);
bool w8a16_tc_supported(const W8A16Args& a);
cudaError_t launch_w8a16_tc_pair(const W8A16Args& a, cudaStream_t s);
bool w8a16_tc_pair_supported(const W8A16Args& a);

// Rows of activations from which the tensor-core kernels are used when the shape allows it.
constexpr int64_t kTcMinM = 17;  // measured: the streaming kernel wins up to 16 rows, the tensor-core kernel from 17

size_t w8a16_tc_workspace_bytes(int64_t M, int64_t N, int64_t K);

// Scratch for the split-K round of the single-CTA tensor-core kernel (0 when no shape of this
// size would use it).  The kernels that do not need it ignore the pointer.
size_t w8a16_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    return M >= kTcMinM ? w8a16_tc_workspace_bytes(M, N, K) : 0;
}

cudaError_t launch_w8a16(const W8A16Args& a, int path, cudaStream_t s) {
    if (path == 1) return launch_w8a16_stream(a, s);
    if (path == 2) return w8a16_tc_pair_supported(a) ? launch_w8a16_tc_pair(a, s) : cudaErrorNotSupported;
    if (path == 3) return w8a16_tc_supported(a) ? launch_w8a16_tc(a, s) : cudaErrorNotSupported;
    if (a.M >= kTcMinM) {
        // measured on B200 (N = 14336, K = 4096): the single-CTA kernel is ahead of the CTA-pair kernel at every M tried
        // (M = 416 / 2048 / 8192: 51 / 200 / 906 us against 55 / 211 / 932 us)
        if (w8a16_tc_supported(a)) return launch_w8a16_tc(a, s);
        if (w8a16_tc_pair_supported(a)) return launch_w8a16_tc_pair(a, s);
    }
    return launch_w8a16_stream(a, s);
}

}  // namespace cb
