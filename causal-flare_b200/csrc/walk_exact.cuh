// Parameters and launcher of the exact sequential-walk kernel (see walk_exact.cu).
#pragma once
#include "flare_common.cuh"

namespace flare {

struct WalkParams {
  const void *q, *k, *v, *qd, *kd;
  void* y;
  const int32_t* mask;
  // carry-in state of (lane, segment): index = lane * in_lane_stride + seg * in_seg_stride (in states)
  const float *in_m, *in_d, *in_u;
  int64_t in_lane_stride, in_seg_stride;
  // carry-out state; out_mode 0: none, 1: every segment writes its own slot, 2: only the last segment
  float *out_m, *out_d, *out_u;
  int64_t out_lane_stride, out_seg_stride;
  int out_mode;
  int nseg_total;
  float* lse_dec;
  float* lse_enc;
  int B, N, H, M, Dk, Dv;
  int64_t q_stride_h, q_stride_m;
  int64_t k_stride_b, k_stride_n, k_stride_h;
  int64_t v_stride_b, v_stride_n, v_stride_h;
  int64_t qd_stride_b, qd_stride_n, qd_stride_h;
  int64_t kd_stride_h, kd_stride_m;
  int64_t y_stride_b, y_stride_n, y_stride_h;
  int seg_len;
  int write_y;
  float scale, power;
  int dtype, variant, block_size;
  // Optional gate: a CTA does nothing unless gate[lane * gate_stride] != 0 (gate_stride 0: one word for the whole
  // call, 1: one word per (batch, head) lane).  Used when these kernels stand by behind the tensor-core path and
  // only run for calls (lanes) whose inputs left that path's numeric domain.  Null: always run.
  const int* gate;
  int gate_stride;
};

// grid.y = nseg_grid segments are launched (segments 0 .. nseg_grid-1)
int launch_walk_exact(const WalkParams& p, int nseg_grid, cudaStream_t stream);
int walk_exact_dd(int M, int Dv);

// defined once per MM_MAX in {2, 8, 16, 32, 64}, each in its own translation unit
template <int MM_MAX>
int launch_walk_mm(const WalkParams& p, int dd, dim3 grid, size_t smem, cudaStream_t stream);

}  // namespace flare
