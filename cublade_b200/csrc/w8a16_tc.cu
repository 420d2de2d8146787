// placeholder until the tcgen05 kernel lands
#include "launch.h"
namespace cb {
bool w8a16_tc_supported(const W8A16Args&) { return false; }
cudaError_t launch_w8a16_tc(const W8A16Args&, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace cb
