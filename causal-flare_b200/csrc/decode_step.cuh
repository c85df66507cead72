// Parameters and launcher of the single-token decode kernel (see decode_step.cu).
#pragma once
#include "flare_common.cuh"

namespace flare {

struct DecodeParams {
  const void *q, *k, *v, *qd, *kd;
  void* y;
  const int32_t* mask;
  float *m, *d, *u;
  int B, H, M, Dk, Dv;
  int64_t q_stride_h, q_stride_m;
  int64_t k_stride_b, k_stride_h;
  int64_t v_stride_b, v_stride_h;
  int64_t qd_stride_b, qd_stride_h;
  int64_t kd_stride_h, kd_stride_m;
  float scale;
  int dtype;
};

bool decode_step_supported(int M, int Dk, int Dv);
int launch_decode_step(const DecodeParams& p, cudaStream_t stream);

}  // namespace flare
