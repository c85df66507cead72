// Device helpers shared by the exact forward walk and the exact backward kernels: tile staging,
// fp32 score tiles, decode softmax over the latents, warp reduce-scatter.
#pragma once
#include "flare_common.cuh"

namespace flare {
namespace walk {

constexpr int BT = 16;   // tokens per tile
constexpr int NT = 256;  // threads per CTA
constexpr int NW = NT / 32;

struct Smem {
  float* ks;     // [BT][ldk]   key rows (also decode queries under weight sharing)
  float* qds;    // [BT][ldk]   decode query rows when q_dec is separate
  float* vs;     // [BT][dvt]
  float* s;      // [BT][mp]    encode scores -> eta
  float* a;      // [BT][mp]    decode scores -> softmax -> read-out weight
  float* g;      // [BT][mp]    gamma
  float* m_run;  // [mp]
  float* d_run;  // [mp]
  float* dinv;   // [mp]
  float* ypart;  // [NW][BT][dvt]
  int* valid;    // [BT]
};

static __device__ __forceinline__ Smem carve(float* base, int ldk, int dvt, int mp) {
  Smem sm;
  sm.ks = base; base += BT * ldk;
  sm.qds = base; base += BT * ldk;
  sm.vs = base; base += BT * dvt;
  sm.s = base; base += BT * mp;
  sm.a = base; base += BT * mp;
  sm.g = base; base += BT * mp;
  sm.m_run = base; base += mp;
  sm.d_run = base; base += mp;
  sm.dinv = base; base += mp;
  sm.ypart = base; base += NW * BT * dvt;
  sm.valid = reinterpret_cast<int*>(base);
  return sm;
}

// rows [t0, t0+BT) of a [.., N, .., D] tensor -> fp32 smem tile; rows >= t_end are zero.
static __device__ __forceinline__ void load_rows(float* dst, int ld, const void* src, int dtype, int64_t row0_off,
                                          int64_t stride_n, int t0, int t_end, int D, int d0, int dcount) {
  const int chunks = dcount / 8;
  for (int idx = threadIdx.x; idx < BT * chunks; idx += NT) {
    const int t = idx / chunks, c = idx % chunks;
    float x[8];
    if (t0 + t < t_end && d0 + c * 8 < D) {
      load8(src, dtype, row0_off + (int64_t)(t0 + t) * stride_n + d0 + c * 8, x);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = 0.f;
    }
    float4* o = reinterpret_cast<float4*>(dst + t * ld + c * 8);
    o[0] = make_float4(x[0], x[1], x[2], x[3]);
    o[1] = make_float4(x[4], x[5], x[6], x[7]);
  }
}

// out[t][m] = scale * <tok[t,:], lat[m,:]> for the 16 tokens of the tile and all M latents.  A thread owns one latent
// and TPG consecutive tokens; TPG is chosen so that all NT threads have work (M = 64: 4 tokens, M >= 128: 8 tokens).
template <int TPG>
static __device__ __forceinline__ void score_tile_impl(float* out, int mp, const float* tok, int ldk, const void* lat,
                                                       int dtype, int64_t lat_off, int64_t lat_stride_m, int M, int Dk,
                                                       float scale) {
  constexpr int GROUPS = BT / TPG;
  for (int idx = threadIdx.x; idx < GROUPS * M; idx += NT) {
    const int m = idx % M, th = idx / M;
    float acc[TPG];
#pragma unroll
    for (int i = 0; i < TPG; ++i) acc[i] = 0.f;
    const int64_t row = lat_off + (int64_t)m * lat_stride_m;
    for (int d0 = 0; d0 < Dk; d0 += 8) {
      float qv[8];
      load8(lat, dtype, row + d0, qv);
#pragma unroll
      for (int tt = 0; tt < TPG; ++tt) {
        const float4* kr = reinterpret_cast<const float4*>(tok + (th * TPG + tt) * ldk + d0);
        const float4 k0 = kr[0], k1 = kr[1];
        acc[tt] += qv[0] * k0.x + qv[1] * k0.y + qv[2] * k0.z + qv[3] * k0.w + qv[4] * k1.x + qv[5] * k1.y +
                   qv[6] * k1.z + qv[7] * k1.w;
      }
    }
#pragma unroll
    for (int tt = 0; tt < TPG; ++tt) out[(th * TPG + tt) * mp + m] = acc[tt] * scale;
  }
}

static __device__ __forceinline__ void score_tile(float* out, int mp, const float* tok, int ldk, const void* lat, int dtype,
                                           int64_t lat_off, int64_t lat_stride_m, int M, int Dk, float scale) {
  if (2 * M >= NT) score_tile_impl<8>(out, mp, tok, ldk, lat, dtype, lat_off, lat_stride_m, M, Dk, scale);
  else if (4 * M >= NT) score_tile_impl<4>(out, mp, tok, ldk, lat, dtype, lat_off, lat_stride_m, M, Dk, scale);
  else if (8 * M >= NT) score_tile_impl<2>(out, mp, tok, ldk, lat, dtype, lat_off, lat_stride_m, M, Dk, scale);
  else score_tile_impl<1>(out, mp, tok, ldk, lat, dtype, lat_off, lat_stride_m, M, Dk, scale);
}

// a[t][:] <- softmax over latents of src[t][:]; one warp per token.  Invalid tokens get zeros.
static __device__ __forceinline__ void decode_softmax(float* a, const float* src, int mp, int M, const int* valid,
                                               float* lse_out /* may be null: [BT] global slice */, int t0, int t_end) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = warp; t < BT; t += NW) {
    if (!valid[t]) {
      for (int m = lane; m < M; m += 32) a[t * mp + m] = 0.f;
      if (lse_out != nullptr && t0 + t < t_end && lane == 0) lse_out[t] = 0.f;
      continue;
    }
    float mx = kNegInf;
    for (int m = lane; m < M; m += 32) mx = fmaxf(mx, src[t * mp + m]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int m = lane; m < M; m += 32) {
      const float e = __expf(src[t * mp + m] - mx);
      a[t * mp + m] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int m = lane; m < M; m += 32) a[t * mp + m] *= inv;
    if (lse_out != nullptr && lane == 0) lse_out[t] = mx + logf(sum);
  }
}


// Sum v[i] over the 32 lanes of the warp for every i in [0, N); afterwards lane l holds the total of
// element (l mod N) in v[0] when N <= 32, and of elements (l, l + 32) in v[0], v[32] when N == 64.
// N - 1 + log2(32 / N) shuffles instead of 5 N.
template <int N>
static __device__ __forceinline__ void warp_reduce_scatter(float (&v)[N], int lane) {
  static_assert(N == 2 || N == 4 || N == 8 || N == 16 || N == 32 || N == 64, "N must be a power of two <= 64");
  constexpr int W = N > 32 ? 32 : N;
#pragma unroll
  for (int base = 0; base < N; base += 32) {
#pragma unroll
    for (int s = W / 2; s >= 1; s >>= 1) {
      const bool upper = (lane & s) != 0;
#pragma unroll
      for (int k = 0; k < s; ++k) {
        const float send = upper ? v[base + k] : v[base + k + s];
        const float keep = upper ? v[base + k + s] : v[base + k];
        v[base + k] = keep + __shfl_xor_sync(0xffffffffu, send, s);
      }
    }
#pragma unroll
    for (int o = W; o < 32; o <<= 1) v[base] += __shfl_xor_sync(0xffffffffu, v[base], o);
  }
}

}  // namespace walk
}  // namespace flare
