// Fold / exclusive scan of (m, d, u) states: the chunk-state scan of the segmented prefill, the carry-in
// merge, and the cross-GPU prefix fold all use this one kernel.
//
// (m_a, d_a, u_a) (+) (m_b, d_b, u_b) = (m, d_a e^{m_a-m} + d_b e^{m_b-m}, u_a e^{m_a-m} + u_b e^{m_b-m}),
// m = max(m_a, m_b); a side whose max is -inf contributes with factor 0 (factor 1 if both are -inf).
#include "state_ops.cuh"

namespace flare {

namespace {

constexpr int NT = 128;
constexpr int LAT_PER_CTA = NT / 32;
constexpr int DCH = 8;  // value columns per lane per pass (32 * DCH columns per pass)

__device__ __forceinline__ void merge_factors(float ma, float mb, float& mn, float& fa, float& fb) {
  mn = fmaxf(ma, mb);
  if (mn == kNegInf) {
    fa = 1.f;
    fb = 1.f;
  } else {
    fa = (ma == kNegInf) ? 0.f : __expf(ma - mn);
    fb = (mb == kNegInf) ? 0.f : __expf(mb - mn);
  }
}

__global__ void __launch_bounds__(NT) fold_kernel(const FoldParams p) {
  if (p.gate != nullptr && *p.gate == 0) return;
  const int64_t lane_id = blockIdx.x;
  const int m = blockIdx.y * LAT_PER_CTA + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (m >= p.M) return;
  const int M = p.M, Dv = p.Dv;
  for (int dv0 = 0; dv0 < Dv; dv0 += 32 * DCH) {
    float rm = p.a_m ? p.a_m[lane_id * M + m] : (p.stablemax ? 0.f : kNegInf);
    float rd = p.a_d ? p.a_d[lane_id * M + m] : 0.f;
    float ru[DCH];
#pragma unroll
    for (int j = 0; j < DCH; ++j) {
      const int dv = dv0 + lane + 32 * j;
      ru[j] = (p.a_u && dv < Dv) ? p.a_u[(lane_id * M + m) * Dv + dv] : 0.f;
    }
    // the statistics are rewritten only in the last column pass: earlier passes still need the originals
    const bool first = (dv0 + 32 * DCH >= Dv) && lane == 0;
    for (int j = 0; j < p.count; ++j) {
      const int64_t sidx = lane_id * p.lane_stride + (int64_t)j * p.seg_stride;
      const bool have_b = (p.mode == 1) || (j < p.count - 1);
      float bm = kNegInf, bd = 0.f, bu[DCH];
      if (have_b) {
        bm = p.s_m[sidx * M + m];
        bd = p.s_d[sidx * M + m];
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          const int dv = dv0 + lane + 32 * c;
          bu[c] = dv < Dv ? p.s_u[(sidx * M + m) * Dv + dv] : 0.f;
        }
      }
      if (p.mode == 0) {
        // all lanes of the warp have read slot j before anyone overwrites it
        __syncwarp();
        if (first) {
          p.s_m[sidx * M + m] = rm;
          p.s_d[sidx * M + m] = rd;
        }
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          const int dv = dv0 + lane + 32 * c;
          if (dv < Dv) p.s_u[(sidx * M + m) * Dv + dv] = ru[c];
        }
      }
      if (have_b) {
        float mn, fa, fb;
        merge_factors(rm, bm, mn, fa, fb);
        rm = mn;
        rd = rd * fa + bd * fb;
#pragma unroll
        for (int c = 0; c < DCH; ++c) ru[c] = ru[c] * fa + bu[c] * fb;
      }
    }
    if (p.mode == 1) {
      if (first) {
        p.o_m[lane_id * M + m] = rm;
        p.o_d[lane_id * M + m] = rd;
      }
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        const int dv = dv0 + lane + 32 * c;
        if (dv < Dv) p.o_u[(lane_id * M + m) * Dv + dv] = ru[c];
      }
    }
  }
}

}  // namespace

int launch_fold(const FoldParams& p, cudaStream_t stream) {
  if (p.lanes <= 0 || p.count <= 0) return FLARE_OK;
  dim3 grid((unsigned)p.lanes, (p.M + LAT_PER_CTA - 1) / LAT_PER_CTA);
  LaunchTimer timer("fold_kernel", stream);
  fold_kernel<<<grid, NT, 0, stream>>>(p);
  FLARE_CUDA_CHECK(cudaGetLastError());
  return FLARE_OK;
}

}  // namespace flare
