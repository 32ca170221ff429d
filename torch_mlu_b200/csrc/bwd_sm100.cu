#include "kernels.h"
namespace sdpa_b200 {
size_t bwd_workspace_bytes(const sdpa_b200_params& p) { return 0; }
int launch_bwd(const sdpa_b200_params& p, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  set_error("backward not built yet");
  return SDPA_B200_UNSUPPORTED;
}
}
