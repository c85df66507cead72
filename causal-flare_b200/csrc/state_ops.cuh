// Associative combination of online-softmax states (see state_ops.cu).
#pragma once
#include "flare_common.cuh"

namespace flare {

struct FoldParams {
  // optional left operand (all null: the empty state); one state per lane
  const float *a_m, *a_d, *a_u;
  // `count` states per lane, state j of lane l at index l * lane_stride + j * seg_stride
  float *s_m, *s_d, *s_u;
  int64_t lane_stride, seg_stride;
  int count;
  // mode 0: s[j] <- a (+) s[0] (+) ... (+) s[j-1] in place (exclusive scan; s[count-1] is only written)
  // mode 1: o <- a (+) s[0] (+) ... (+) s[count-1]
  int mode;
  float *o_m, *o_d, *o_u;
  int64_t lanes;
  int M, Dv;
  int stablemax;  // the empty state has m = 0 instead of -inf
  const int* gate;  // optional: the kernel does nothing unless *gate != 0
};

int launch_fold(const FoldParams& p, cudaStream_t stream);

// fp16 <-> bf16 copy of a tensor of rows: n0 x n1 x n2 rows of d contiguous 2-byte elements (d a multiple of 8, row
// starts 16-byte aligned), row (i0, i1, i2) at element offset i0 * s0 + i1 * s1 + i2 * s2 on either side.
struct CastParams {
  const void* in;
  void* out;
  int64_t n0, n1, n2;
  int d;
  int64_t is0, is1, is2;
  int64_t os0, os1, os2;
  int to_f16;  // 1: bf16 -> fp16, 0: fp16 -> bf16
};

int launch_cast_rows(const CastParams& p, cudaStream_t stream);

}  // namespace flare
