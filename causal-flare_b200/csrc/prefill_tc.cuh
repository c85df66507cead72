// Tensor-core chunked prefill (see prefill_tc.cu).
#pragma once
#include "flare_common.cuh"

namespace flare {

struct TcParams {
  void* y;  // bf16 [B, N, H, Dv] (strided) or null
  int64_t y_stride_b, y_stride_n, y_stride_h;
  const void* q;  // bf16 latent bank [H, M, Dk]
  int64_t q_stride_h, q_stride_m;
  int N, H;
  int M;   // latents, <= 512; groups of 128 go to separate CTAs
  int Dv;  // value width (64 or 128); each CTA handles 64 columns
  float scale;
  int seg_len;
  // carry-in / carry-out states, indexed lane * lane_stride + seg * seg_stride (in states)
  const float *in_m, *in_d, *in_u;
  int64_t in_lane_stride, in_seg_stride;
  float *out_m, *out_d, *out_u;
  int64_t out_lane_stride, out_seg_stride;
  // more than 128 latents: per-group partial read-outs (each normalised over its own latents), fp16
  // [groups][B][N][H][Dv], and the log2 of each group's weight mass, fp32 [groups][B][N][H]; the launch merges them
  // into y afterwards
  void* part_y;
  float* part_lw;
  // the read-out rows leave through tiled bulk stores (set by the launch when the output's strides allow it and no
  // per-row lengths are given); otherwise every thread stores its own row
  int y_tma;
  // Two latent groups on the wide instance: the two CTAs of a lane form a thread-block cluster and merge their
  // partial read-outs on chip (each finalises one 64-column value block); no partials in global memory, no merge
  // kernel.  Set by the launch.
  int cluster_merge;
  int out_mode;  // 0: none, 1: every segment, 2: last segment only
  int nseg_total;
  const int32_t* lens;       // [B] tokens per batch row (right padding beyond), or null
  int block;                 // 1 = token-causal; 16, 32, 64, 128 = block-causal
  float power;               // stablemax exponent (stablemax encoder only)
  float *lse_dec, *lse_enc;  // optional outputs, fp32 natural log: [B, H, N] and [B, H, N / block, M]
  // Training: per-chunk prefix states for the backward pass (chunk = 128 tokens, index over the whole sequence):
  // dump_u bf16 [lanes][dump_nch][M][Dv] numerator before the chunk in the chunk's frame, dump_c / dump_d fp32
  // [lanes][dump_nch][M] that frame (log2 units) and the denominator before the chunk.  Null: nothing is kept.
  void* dump_u;
  float *dump_c, *dump_d;
  int dump_nch;
  // Optional per-call gate words (in the caller's workspace, zeroed before the launch): gate[0] is raised when any
  // token of the call left the numeric domain of these kernels, gate[1 + lane] for the (batch, head) lane it is in.
  int* gate;
  int* err;                  // device error word (bit 0: a wait gave up, bit 1: numeric domain exceeded)
  long long* trace;  // optional diagnostic cycle stamps of CTA (0, 0), see TC_TRACE; null in normal use
};

bool prefill_tc_supported(const flare_fwd_args_t* a);
// CTAs the kernel launches per (lane, segment)
int prefill_tc_ctas_per_lane(const flare_fwd_args_t* a);
// scratch for the partial read-outs of the latent groups (0 for M <= 128), and the byte offset of the weight-mass
// array inside it
size_t prefill_tc_partial_bytes(const flare_fwd_args_t* a);
size_t prefill_tc_partial_lw_offset(const flare_fwd_args_t* a);
// launches segments 0 .. nseg_grid-1
int launch_prefill_tc(const flare_fwd_args_t* a, const TcParams& p, int nseg_grid, cudaStream_t stream);
// device address (current device) of the error word shared by all tensor-core kernels
int tc_error_word(int** device_address);
// reads (and optionally clears) the device-side error flag of the tensor-core kernels; synchronises
int prefill_tc_error_flag(int* host_value, bool reset);

}  // namespace flare
