// Tensor-core (tcgen05 + TMEM + TMA) backward pass (see bwd_tc.cu).
#pragma once
#include "flare_common.cuh"

namespace flare {

// Per-chunk prefix states kept by the tensor-core forward for the backward pass (chunks of 128 tokens over the
// whole sequence): u bf16 [lanes][nch][M][Dv], c / d fp32 [lanes][nch][M].
struct ChunkStates {
  void* u;
  float *c, *d;
  int nch;
};

// true when flare_backward takes the tensor-core kernels for this problem
bool bwd_tc_supported(const flare_bwd_args_t& a);
size_t bwd_tc_workspace_bytes(const flare_bwd_args_t& a);
int bwd_tc(const flare_bwd_args_t& a, cudaStream_t stream);

// Forward on the tensor path that also writes y, the decode log-sum-exp and the per-chunk prefix states
// (defined with the forward dispatch).
int forward_keep_states(const flare_fwd_args_t* a, const ChunkStates& keep, cudaStream_t stream);
// kernels launched so far by the current forward / backward call of this thread (measurement hook)
void count_launches(int n);

}  // namespace flare
