// Exact (fp32, CUDA-core) backward pass (see bwd_exact.cu).
#pragma once
#include "flare_common.cuh"

namespace flare {

size_t bwd_exact_workspace_bytes(const flare_bwd_args_t& a);
int bwd_exact(const flare_bwd_args_t& a, cudaStream_t stream);

}  // namespace flare
