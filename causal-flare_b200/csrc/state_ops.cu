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

template <bool TO_F16>
__global__ void __launch_bounds__(256) cast_rows_kernel(const CastParams p) {
  const int c8n = p.d >> 3;
  const int64_t total = p.n0 * p.n1 * p.n2 * c8n;
  const uint16_t* in = reinterpret_cast<const uint16_t*>(p.in);
  uint16_t* out = reinterpret_cast<uint16_t*>(p.out);
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int c8 = (int)(idx % c8n);
    int64_t r = idx / c8n;
    const int64_t i2 = r % p.n2;
    r /= p.n2;
    const int64_t i1 = r % p.n1;
    const int64_t i0 = r / p.n1;
    uint4 x = *reinterpret_cast<const uint4*>(in + i0 * p.is0 + i1 * p.is1 + i2 * p.is2 + c8 * 8);
    uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (TO_F16) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
        const __half2 h = __floats2half2_rn(f.x, f.y);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        const __nv_bfloat162 h = __floats2bfloat162_rn(f.x, f.y);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(out + i0 * p.os0 + i1 * p.os1 + i2 * p.os2 + c8 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace

int launch_cast_rows(const CastParams& p, cudaStream_t stream) {
  const int64_t total = p.n0 * p.n1 * p.n2 * (p.d >> 3);
  if (total <= 0) return FLARE_OK;
  if (p.d % 8) return FLARE_ERR_BAD_SHAPE;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  LaunchTimer timer(p.to_f16 ? "cast_rows_kernel<bf16 to fp16>" : "cast_rows_kernel<fp16 to bf16>", stream);
  if (p.to_f16)
    cast_rows_kernel<true><<<(unsigned)blocks, 256, 0, stream>>>(p);
  else
    cast_rows_kernel<false><<<(unsigned)blocks, 256, 0, stream>>>(p);
  FLARE_CUDA_CHECK(cudaGetLastError());
  return FLARE_OK;
}

int launch_fold(const FoldParams& p, cudaStream_t stream) {
  if (p.lanes <= 0 || p.count <= 0) return FLARE_OK;
  dim3 grid((unsigned)p.lanes, (p.M + LAT_PER_CTA - 1) / LAT_PER_CTA);
  LaunchTimer timer("fold_kernel", stream);
  fold_kernel<<<grid, NT, 0, stream>>>(p);
  FLARE_CUDA_CHECK(cudaGetLastError());
  return FLARE_OK;
}

}  // namespace flare
