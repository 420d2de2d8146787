// W8A16 dispatch: picks the weight-streaming kernel (w8a16_stream.cu) for skinny
// activations and the tcgen05 tensor-core kernel (w8a16_tc.cu) for tall ones.
#include "launch.h"

namespace cb {

cudaError_t launch_w8a16_stream(const W8A16Args& a, cudaStream_t s);
cudaError_t launch_w8a16_tc(const W8A16Args& a, cudaStream_t s);
bool w8a16_tc_supported(const W8A16Args& a);

// Rows of activations from which the tensor-core kernel is used when the shape allows it.
constexpr int64_t kTcMinM = 65;

size_t w8a16_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }

cudaError_t launch_w8a16(const W8A16Args& a, int path, cudaStream_t s) {
    if (path == 1) return launch_w8a16_stream(a, s);
    if (path == 2) return w8a16_tc_supported(a) ? launch_w8a16_tc(a, s) : cudaErrorNotSupported;
    if (a.M >= kTcMinM && w8a16_tc_supported(a)) return launch_w8a16_tc(a, s);
    return launch_w8a16_stream(a, s);
}

}  // namespace cb
