// Exact (fp32, CUDA-core) backward pass (see bwd_exact.cu).
#pragma once
#include "flare_common.cuh"

namespace flare {

size_t bwd_exact_workspace_bytes(const flare_bwd_args_t& a);
// gate (may be null): device word; with a gate every kernel of the pass returns at once unless the word is non-zero
int bwd_exact(const flare_bwd_args_t& a, cudaStream_t stream, const int* gate = nullptr);

// Exclusive prefix states of the sequence segments [s * seg_len, (s + 1) * seg_len) of a forward problem (empty initial
// state): slot s of seg_m / seg_d [lanes][nseg][M] and seg_u [lanes][nseg][M][Dv] receives the state after all tokens
// before segment s.  Uses the forward kernels (defined with them).
// `init` (may be null) is the state before the first segment.
int segment_prefix_states(const flare_fwd_args_t* f, int nseg, int seg_len, float* seg_m, float* seg_d, float* seg_u,
                          const flare_state_t* init, cudaStream_t stream, const int* gate = nullptr);

}  // namespace flare
