// placeholder until the tcgen05 backward lands: declines every shape so the launcher uses the CUDA-core path
#include "fdma_internal.h"
namespace fdma {
bool tc_bwd_supported(const fdma_bwd_params&) { return false; }
size_t tc_bwd_workspace_bytes(const fdma_bwd_params&) { return 0; }
int tc_bwd(const fdma_bwd_params&, cudaStream_t) { return FDMA_ERR_UNSUPPORTED; }
}  // namespace fdma
