#include "bwd_exact.cuh"
namespace flare {
size_t bwd_exact_workspace_bytes(const flare_bwd_args_t&) { return 0; }
int bwd_exact(const flare_bwd_args_t&, cudaStream_t) { return FLARE_ERR_UNSUPPORTED; }
}  // namespace flare
