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

// Layout of flare_fwd_args_t::keep for a problem (all offsets in bytes; total == 0: the problem keeps nothing)
struct KeepLayout {
  size_t off_gate, off_u, off_c, off_d, total;
  int nch;
};
KeepLayout keep_layout(const flare_fwd_args_t& f);

// true when flare_backward takes the tensor-core kernels for this problem
bool bwd_tc_supported(const flare_bwd_args_t& a);
size_t bwd_tc_workspace_bytes(const flare_bwd_args_t& a);
int bwd_tc(const flare_bwd_args_t& a, cudaStream_t stream);

// Forward on the tensor path that also writes y, the decode log-sum-exp and the per-chunk prefix states
// (defined with the forward dispatch).
// `gate` (may be null): per-call gate words, 1 + lanes ints, zeroed by the caller (see TcParams::gate).
int forward_keep_states(const flare_fwd_args_t* a, const ChunkStates& keep, int* gate, cudaStream_t stream);
// diagnostic buffer set with flare_set_trace_buffer (null in normal use)
long long* trace_buffer();
// kernels launched so far by the current forward / backward call of this thread (measurement hook)
void count_launches(int n);

}  // namespace flare
