// Exact (fp32, CUDA-core) backward of causal FLARE: softmax / stablemax encoders, token-causal or
// block-causal read-out, shared or separate decode weights.  Nothing is saved by the forward; the
// forward recurrence is replayed here.
//
// With e[t,m] the normalised encoder weight of token t at its read-out time (softmax exp(s - L_t),
// stablemax sigma(s)/D_t) the read-out state obeys z_t = (1 - e_t) z_{t-1} + e_t v_t, hence
//   p[t,m]   = <z_t[m,:], dY_t>                        g[t,:] = softmax_m(a[t,:])
//   b_t[m,:] = g dY_t + (1 - e_{t+1}) b_{t+1}           c_t[m] = g p + (1 - e_{t+1}) c_{t+1}
//   dV_t     = sum_m e b_t[m,:]
//   dS_enc   = e * slope * (<b_t[m,:], v_t> - c_t[m])    slope = 1 | sigma'(s)/sigma(s)
//   dS_dec   = g (p - sum_m g p)
//   dK = scale dS Q,  dQ = scale sum_{b,t} dS^T k_t  (decode-side products go to dQ_dec / dK_dec when separate)
// For block-causal read-out the state is read at block ends, so e, b, c are per block.
//
// Kernels: (1) replay: forward walk that stores e, g and the partial p of its Dv tile;
// (2) reverse: reverse walk carrying (b, c), emits dV and the dS planes; (3) rows: dK / dQ_dec = dS Lat;
// (4) latents: per-split partial dQ / dK_dec = dS^T Rows; (5) fixed-order sum of the partials
// (deterministic: no atomics anywhere).
#include "bwd_exact.cuh"

#include <string.h>

#include "walk_device.cuh"
#include "walk_exact.cuh"

namespace flare {

using namespace walk;

struct BwdParams {
  const void *q, *k, *v, *qd, *kd, *dy;
  int B, N, H, M, Dk, Dv;
  int64_t q_stride_h, q_stride_m;
  int64_t k_stride_b, k_stride_n, k_stride_h;
  int64_t v_stride_b, v_stride_n, v_stride_h;
  int64_t qd_stride_b, qd_stride_n, qd_stride_h;
  int64_t kd_stride_h, kd_stride_m;
  int64_t dy_stride_b, dy_stride_n, dy_stride_h;
  float scale, power;
  int dtype, variant, block_size;
  // workspace planes, each [lanes][N][M] fp32
  float* E;    // normalised encoder weight
  float* G;    // decode softmax
  float* W2;   // E * slope (stablemax), aliases E for softmax
  float* P;    // [DT] planes: partial p of every Dv tile
  float* dSe;  // [DT] planes: partial encode-score gradient (plane 0 also carries -c and, if shared, dS_dec)
  float* dSd;  // decode-score gradient, null when the weights are shared
  int DT;
  int64_t plane;  // lanes * N * M
  void* dv_out;   // [B, N, H, Dv] contiguous, input dtype
  // Sequence segments (token-causal read-out only; nseg == 1: one CTA walks the whole sequence).  grid.z walks
  // segments seg_first .. ; the replay starts every segment from its exclusive prefix state, the reverse walk from
  // the carries (b, c) of the segment to its right.
  int seg_len, nseg, seg_first;
  const float *in_m, *in_d, *in_u;   // [lanes][nseg][M], [lanes][nseg][M], [lanes][nseg][M][Dv]
  float *seg_b, *seg_c, *seg_gam;    // [lanes][nseg][M][Dv], [lanes][nseg][M], [lanes][nseg][M]
  // Written by the replay when nseg > 1: X[t, m] = g[t, m] * prod_{tau = a+1 .. t} (1 - e[tau, m]) (a = first token of
  // the segment of t), the weight with which g dY_t and g p enter the carries (b, c) at the segment's first token;
  // seg_gam receives the product of all decays of the segment.
  float* X;                          // [lanes][N][M]
  // Block-causal read-out with segments: decay of every block, rho[j, m] = 1 - sum_{t in block j} e[t, m]; the decays
  // in X and seg_gam are then per block.
  float* RHO;                        // [lanes][N / block_size][M]
  // Span of a longer sequence (sequence parallelism): carries entering from the tokens after the span, or null
  const float *carry_b, *carry_c, *carry_rho;  // [lanes][M][Dv], [lanes][M], [lanes][M] (decay of the first token after)
  // Optional gate word: every kernel of this pass returns at once unless *gate != 0 (the pass then stands by behind
  // the tensor-core backward and only runs when that one reported inputs outside its numeric domain).
  const int* gate;
};

// defined once per MM_MAX in {2, 8, 16, 32, 64}, each in its own translation unit; stage 0 = replay, 1 = reverse
template <int MM_MAX>
int launch_bwd_mm(const BwdParams& p, int dd, dim3 grid, size_t smem1, size_t smem2, cudaStream_t stream, int stage);

namespace {

#ifdef FLARE_WALK_MM
// --------------------------------------------------------------------------------------------------
// (1) forward replay
// --------------------------------------------------------------------------------------------------
template <int MM_MAX, int DD>
__global__ void __launch_bounds__(NT, (MM_MAX * DD <= 32) ? 2 : 1) bwd_replay_kernel(const BwdParams p) {
  if (p.gate != nullptr && *p.gate == 0) return;
  extern __shared__ __align__(16) float smem_raw[];
  const int lane_id = blockIdx.x, dt = blockIdx.y;
  const int b = lane_id / p.H, h = lane_id % p.H;
  constexpr int dvt = 32 * DD;
  const int dv0 = dt * dvt;
  const int M = p.M, Dk = p.Dk, Dv = p.Dv, N = p.N;
  const int mp = M + 4, ldk = Dk + 4;
  float* base = smem_raw;
  float* ks = base; base += BT * ldk;
  float* qds = base; base += BT * ldk;
  float* vs = base; base += BT * dvt;
  float* dos = base; base += BT * dvt;
  float* s_s = base; base += BT * mp;   // scores -> eta
  float* a_s = base; base += BT * mp;   // decode softmax
  float* g_s = base; base += BT * mp;   // gamma
  float* r_s = base; base += BT * mp;   // 1 / d_t
  float* m_run = base; base += mp;
  float* d_run = base; base += mp;
  float* dinv = base; base += mp;
  float* gp_run = base; base += mp;  // running product of the decays since the segment's first token
  float* m0_s = base; base += mp;    // block-causal: running max / denominator at the start of the current block
  float* d0_s = base; base += mp;
  int* valid = reinterpret_cast<int*>(base);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mm = M / NW;
  const bool shared_w = p.qd == nullptr && p.kd == nullptr;
  const bool stablemax = p.variant == FLARE_STABLEMAX;
  const int dtype = p.dtype;

  const int seg = p.seg_first + blockIdx.z;
  const int tbeg = seg * p.seg_len, tend = min(N, tbeg + p.seg_len);
  const bool carry_in = p.in_u != nullptr;  // slot 0 holds the state before the sequence / span (possibly empty)
  const int64_t st = (int64_t)lane_id * p.nseg + seg;  // index of this segment's prefix state

  float U[MM_MAX][DD];
#pragma unroll
  for (int mi = 0; mi < MM_MAX; ++mi)
#pragma unroll
    for (int j = 0; j < DD; ++j) {
      const int m = warp * mm + mi, col = dv0 + lane + 32 * j;
      U[mi][j] = (carry_in && mi < mm && col < Dv) ? p.in_u[(st * M + m) * Dv + col] : 0.f;
    }
  for (int m = tid; m < M; m += NT) {
    m_run[m] = carry_in ? p.in_m[st * M + m] : (stablemax ? 0.f : kNegInf);
    d_run[m] = carry_in ? p.in_d[st * M + m] : 0.f;
    gp_run[m] = 1.0f;
  }
  __syncthreads();

  const int64_t k_off = (int64_t)b * p.k_stride_b + (int64_t)h * p.k_stride_h;
  const int64_t v_off = (int64_t)b * p.v_stride_b + (int64_t)h * p.v_stride_h;
  const int64_t qd_off = (int64_t)b * p.qd_stride_b + (int64_t)h * p.qd_stride_h;
  const int64_t dy_off = (int64_t)b * p.dy_stride_b + (int64_t)h * p.dy_stride_h;
  const int64_t q_off = (int64_t)h * p.q_stride_h;
  const int64_t kd_off = (int64_t)h * p.kd_stride_h;
  const int64_t row_base = (int64_t)lane_id * N;  // row index into the [lanes][N][M] planes
  float* Ppart = p.P + (int64_t)dt * p.plane;

  auto set_valid = [&](int t0) {
    if (tid < BT) valid[tid] = (t0 + tid) < N;
  };

  // p[t, m] for the tokens of the staged tile: sum over this tile's value columns, then across lanes
  auto emit_p = [&](int t0, int t, const float* rinv_row /* [mp] 1/d per latent */) {
    float pp[MM_MAX];
#pragma unroll
    for (int mi = 0; mi < MM_MAX; ++mi) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < DD; ++j) acc += U[mi][j] * dos[t * dvt + lane + 32 * j];
      pp[mi] = acc;
    }
    warp_reduce_scatter<MM_MAX>(pp, lane);
    constexpr int W = MM_MAX > 32 ? 32 : MM_MAX;
    const int li = lane & (W - 1);
#pragma unroll
    for (int rep = 0; rep < (MM_MAX + 31) / 32; ++rep) {
      const int mi = li + 32 * rep;
      if (lane < W && mi < mm) {
        const int m = warp * mm + mi;
        Ppart[(row_base + t0 + t) * M + m] = pp[32 * rep] * rinv_row[m];
      }
    }
  };

  if (p.block_size <= 1) {
    for (int t0 = tbeg; t0 < tend; t0 += BT) {
      __syncthreads();
      set_valid(t0);
      load_rows(ks, ldk, p.k, dtype, k_off, p.k_stride_n, t0, N, Dk, 0, Dk);
      load_rows(vs, dvt, p.v, dtype, v_off, p.v_stride_n, t0, N, Dv, dv0, dvt);
      load_rows(dos, dvt, p.dy, dtype, dy_off, p.dy_stride_n, t0, N, Dv, dv0, dvt);
      if (p.qd != nullptr) load_rows(qds, ldk, p.qd, dtype, qd_off, p.qd_stride_n, t0, N, Dk, 0, Dk);
      __syncthreads();
      score_tile(s_s, mp, ks, ldk, p.q, dtype, q_off, p.q_stride_m, M, Dk, p.scale);
      if (!shared_w)
        score_tile(a_s, mp, p.qd ? qds : ks, ldk, p.kd ? p.kd : p.q, dtype, p.kd ? kd_off : q_off,
                   p.kd ? p.kd_stride_m : p.q_stride_m, M, Dk, p.scale);
      __syncthreads();
      decode_softmax(a_s, shared_w ? s_s : a_s, mp, M, valid, nullptr, t0, N);
      __syncthreads();
      for (int m = tid; m < M; m += NT) {
        float mr = m_run[m], dr = d_run[m], gp = gp_run[m];
        for (int t = 0; t < BT; ++t) {
          if (!valid[t]) continue;
          const float s = s_s[t * mp + m];
          float gam, eta;
          if (stablemax) {
            gam = 1.f;
            eta = stablemax_sigma(s, p.power);
            dr += eta;
          } else {
            const float mn = fmaxf(mr, s);
            gam = (mr == kNegInf) ? 0.f : __expf(mr - mn);
            eta = __expf(s - mn);
            dr = dr * gam + eta;
            mr = mn;
          }
          const float rinv = 1.0f / dr;
          g_s[t * mp + m] = gam;
          s_s[t * mp + m] = eta;
          r_s[t * mp + m] = rinv;
          if (dt == 0) {
            const int64_t o = (row_base + t0 + t) * M + m;
            const float e = eta * rinv;
            p.E[o] = e;
            p.G[o] = a_s[t * mp + m];
            if (stablemax) p.W2[o] = e * stablemax_slope_ratio(s, p.power);
            if (p.X != nullptr) {
              if (t0 + t != tbeg) gp *= 1.0f - e;  // the segment's first token carries no decay
              p.X[o] = a_s[t * mp + m] * gp;
            }
          }
        }
        m_run[m] = mr;
        d_run[m] = dr;
        gp_run[m] = gp;
      }
      __syncthreads();
#pragma unroll 1
      for (int t = 0; t < BT; ++t) {
        if (!valid[t]) continue;
        float vv[DD];
#pragma unroll
        for (int j = 0; j < DD; ++j) vv[j] = vs[t * dvt + lane + 32 * j];
#pragma unroll
        for (int mi = 0; mi < MM_MAX; ++mi) {
          if (mi < mm) {
            const int m = warp * mm + mi;
            const float gam = g_s[t * mp + m], eta = s_s[t * mp + m];
#pragma unroll
            for (int j = 0; j < DD; ++j) U[mi][j] = U[mi][j] * gam + eta * vv[j];
          }
        }
        emit_p(t0, t, r_s + t * mp);
      }
    }
    if (p.X != nullptr && dt == 0) {
      // product of all decays of the segment, including the one of the next segment's first token
      __syncthreads();
      for (int m = tid; m < M; m += NT)
        p.seg_gam[st * M + m] = gp_run[m];
    }
  } else {
    const int bs = p.block_size;
    for (int blk0 = tbeg; blk0 < tend; blk0 += bs) {
      const int blk_end = blk0 + bs;
      __syncthreads();
      for (int m = tid; m < M; m += NT) {
        m0_s[m] = m_run[m];
        d0_s[m] = d_run[m];
      }
      for (int t0 = blk0; t0 < blk_end; t0 += BT) {
        __syncthreads();
        set_valid(t0);
        load_rows(ks, ldk, p.k, dtype, k_off, p.k_stride_n, t0, N, Dk, 0, Dk);
        load_rows(vs, dvt, p.v, dtype, v_off, p.v_stride_n, t0, N, Dv, dv0, dvt);
        __syncthreads();
        score_tile(s_s, mp, ks, ldk, p.q, dtype, q_off, p.q_stride_m, M, Dk, p.scale);
        __syncthreads();
        for (int m = tid; m < M; m += NT) {
          float mr = m_run[m], dr = d_run[m];
          for (int t = 0; t < BT; ++t) {
            const float s = s_s[t * mp + m];
            const float mn = fmaxf(mr, s);
            const float gam = (mr == kNegInf) ? 0.f : __expf(mr - mn);
            const float eta = __expf(s - mn);
            dr = dr * gam + eta;
            mr = mn;
            g_s[t * mp + m] = gam;
            s_s[t * mp + m] = eta;
          }
          m_run[m] = mr;
          d_run[m] = dr;
        }
        __syncthreads();
#pragma unroll 1
        for (int t = 0; t < BT; ++t) {
          float vv[DD];
#pragma unroll
          for (int j = 0; j < DD; ++j) vv[j] = vs[t * dvt + lane + 32 * j];
#pragma unroll
          for (int mi = 0; mi < MM_MAX; ++mi) {
            if (mi < mm) {
              const int m = warp * mm + mi;
              const float gam = g_s[t * mp + m], eta = s_s[t * mp + m];
#pragma unroll
              for (int j = 0; j < DD; ++j) U[mi][j] = U[mi][j] * gam + eta * vv[j];
            }
          }
        }
      }
      __syncthreads();
      for (int m = tid; m < M; m += NT) {
        const float di = 1.0f / d_run[m];
        dinv[m] = di;
        if (p.X != nullptr) {
          // decay of this block = denominator before the block over the one after it, in the block-end frame
          const float rho = (m0_s[m] == kNegInf) ? 0.f : d0_s[m] * __expf(m0_s[m] - m_run[m]) * di;
          if (blk0 != tbeg) gp_run[m] *= rho;  // the segment's first block carries no decay
          if (dt == 0) p.RHO[((int64_t)lane_id * (N / bs) + blk0 / bs) * M + m] = rho;
        }
      }
      for (int t0 = blk0; t0 < blk_end; t0 += BT) {
        __syncthreads();
        set_valid(t0);
        load_rows(ks, ldk, p.k, dtype, k_off, p.k_stride_n, t0, N, Dk, 0, Dk);
        load_rows(dos, dvt, p.dy, dtype, dy_off, p.dy_stride_n, t0, N, Dv, dv0, dvt);
        if (p.qd != nullptr) load_rows(qds, ldk, p.qd, dtype, qd_off, p.qd_stride_n, t0, N, Dk, 0, Dk);
        __syncthreads();
        score_tile(s_s, mp, ks, ldk, p.q, dtype, q_off, p.q_stride_m, M, Dk, p.scale);
        if (!shared_w)
          score_tile(a_s, mp, p.qd ? qds : ks, ldk, p.kd ? p.kd : p.q, dtype, p.kd ? kd_off : q_off,
                     p.kd ? p.kd_stride_m : p.q_stride_m, M, Dk, p.scale);
        __syncthreads();
        decode_softmax(a_s, shared_w ? s_s : a_s, mp, M, valid, nullptr, t0, N);
        __syncthreads();
        if (dt == 0) {
          for (int idx = tid; idx < BT * M; idx += NT) {
            const int t = idx / M, m = idx % M;
            const int64_t o = (row_base + t0 + t) * M + m;
            p.E[o] = __expf(s_s[t * mp + m] - m_run[m]) * dinv[m];
            p.G[o] = a_s[t * mp + m];
            if (p.X != nullptr) p.X[o] = a_s[t * mp + m] * gp_run[m];
          }
        }
#pragma unroll 1
        for (int t = 0; t < BT; ++t) emit_p(t0, t, dinv);
      }
    }
    if (p.X != nullptr && dt == 0) {
      __syncthreads();
      for (int m = tid; m < M; m += NT) p.seg_gam[st * M + m] = gp_run[m];
    }
  }
}

// --------------------------------------------------------------------------------------------------
// (2) reverse walk
// --------------------------------------------------------------------------------------------------
template <int MM_MAX, int DD>
__global__ void __launch_bounds__(NT, (MM_MAX * DD <= 32) ? 2 : 1) bwd_reverse_kernel(const BwdParams p) {
  if (p.gate != nullptr && *p.gate == 0) return;
  extern __shared__ __align__(16) float smem_raw[];
  const int lane_id = blockIdx.x, dt = blockIdx.y;
  const int b = lane_id / p.H, h = lane_id % p.H;
  constexpr int dvt = 32 * DD;
  const int dv0 = dt * dvt;
  const int M = p.M, Dv = p.Dv, N = p.N;
  const int mp = M + 4;
  const bool stablemax = p.variant == FLARE_STABLEMAX;
  const bool shared_w = p.dSd == nullptr;
  float* base = smem_raw;
  float* vs = base; base += BT * dvt;
  float* dos = base; base += BT * dvt;
  float* e_s = base; base += BT * mp;
  float* g_s = base; base += BT * mp;
  float* p_s = base; base += BT * mp;   // p -> dS_dec
  float* c_s = base; base += BT * mp;
  float* bv_s = base; base += BT * mp;
  float* w_s = stablemax ? base : e_s;
  if (stablemax) base += BT * mp;
  float* rho_in = base; base += mp;     // decay applied when stepping from the next tile / block into this one
  float* c_run = base; base += mp;
  float* esum = base; base += mp;
  float* gp = base; base += BT;
  float* dvpart = base; base += NW * BT * dvt;
  int* valid = reinterpret_cast<int*>(base);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mm = M / NW;
  const int dtype = p.dtype;

  const int seg = p.seg_first + blockIdx.z;
  const int tbeg = seg * p.seg_len, tend = min(N, tbeg + p.seg_len);
  const int64_t row_base = (int64_t)lane_id * N;
  const int64_t st = (int64_t)lane_id * p.nseg + seg;
  // carries from the segment to the right (zero at the end of the sequence and in the carries-only mode)
  // carries from the segment to the right; for the last segment, from the tokens after the span (if any)
  const bool carry_in = p.nseg > 1 && tend < N;
  const bool span_carry = tend >= N && p.carry_b != nullptr;

  float Bc[MM_MAX][DD];
#pragma unroll
  for (int mi = 0; mi < MM_MAX; ++mi)
#pragma unroll
    for (int j = 0; j < DD; ++j) {
      const int m = warp * mm + mi, col = dv0 + lane + 32 * j;
      Bc[mi][j] = (mi >= mm || col >= Dv) ? 0.f
                  : carry_in            ? p.seg_b[(st * M + m) * Dv + col]
                  : span_carry          ? p.carry_b[((int64_t)lane_id * M + m) * Dv + col]
                                        : 0.f;
    }
  for (int m = tid; m < M; m += NT) {
    // decay of the first step = 1 - e of the first token of the segment to the right
    rho_in[m] = tend >= N ? (span_carry ? p.carry_rho[(int64_t)lane_id * M + m] : 0.f)
                : p.block_size <= 1 ? 1.0f - p.E[(row_base + tend) * M + m]
                                    : p.RHO[((int64_t)lane_id * (N / p.block_size) + tend / p.block_size) * M + m];
    c_run[m] = carry_in ? p.seg_c[st * M + m] : span_carry ? p.carry_c[(int64_t)lane_id * M + m] : 0.f;
    esum[m] = 0.f;
  }

  const int64_t v_off = (int64_t)b * p.v_stride_b + (int64_t)h * p.v_stride_h;
  const int64_t dy_off = (int64_t)b * p.dy_stride_b + (int64_t)h * p.dy_stride_h;
  float* dSe_part = p.dSe + (int64_t)dt * p.plane;

  auto load_plane = [&](float* dst, const float* src, int t0, int parts) {
    const int q4 = M / 4;
    for (int idx = tid; idx < BT * q4; idx += NT) {
      const int t = idx / q4, c = (idx % q4) * 4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t0 + t < N) {
        for (int part = 0; part < parts; ++part) {
          const float4 x = *reinterpret_cast<const float4*>(src + (int64_t)part * p.plane + (row_base + t0 + t) * M + c);
          acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
      }
      *reinterpret_cast<float4*>(dst + t * mp + c) = acc;
    }
  };
  auto set_valid = [&](int t0) {
    if (tid < BT) valid[tid] = (t0 + tid) < N;
  };
  auto compute_gp = [&]() {
    for (int t = warp; t < BT; t += NW) {
      float acc = 0.f;
      for (int m = lane; m < M; m += 32) acc += g_s[t * mp + m] * p_s[t * mp + m];
      acc = warp_sum(acc);
      if (lane == 0) gp[t] = acc;
    }
  };
  float dvacc[BT][DD];
  auto zero_dv = [&]() {
#pragma unroll
    for (int t = 0; t < BT; ++t)
#pragma unroll
      for (int j = 0; j < DD; ++j) dvacc[t][j] = 0.f;
  };
  // <b[m,:], v_t> over this tile's value columns -> bv_s[t][m]
  auto emit_bv = [&](int t) {
    float pp[MM_MAX];
#pragma unroll
    for (int mi = 0; mi < MM_MAX; ++mi) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < DD; ++j) acc += Bc[mi][j] * vs[t * dvt + lane + 32 * j];
      pp[mi] = acc;
    }
    warp_reduce_scatter<MM_MAX>(pp, lane);
    constexpr int W = MM_MAX > 32 ? 32 : MM_MAX;
    const int li = lane & (W - 1);
#pragma unroll
    for (int rep = 0; rep < (MM_MAX + 31) / 32; ++rep) {
      const int mi = li + 32 * rep;
      if (lane < W && mi < mm) bv_s[t * mp + warp * mm + mi] = pp[32 * rep];
    }
  };
  // dS planes and dV of the staged tile
  auto finish_tile = [&](int t0, const float* c_of /* [BT][mp] or per-latent [mp] */, int c_ld) {
#pragma unroll
    for (int t = 0; t < BT; ++t)
#pragma unroll
      for (int j = 0; j < DD; ++j) dvpart[(warp * BT + t) * dvt + lane + 32 * j] = dvacc[t][j];
    __syncthreads();
    for (int idx = tid; idx < BT * M; idx += NT) {
      const int t = idx / M, m = idx % M;
      if (t0 + t >= N) continue;
      const int64_t o = (row_base + t0 + t) * M + m;
      float ds = w_s[t * mp + m] * (bv_s[t * mp + m] - (dt == 0 ? c_of[t * c_ld + m] : 0.f));
      if (dt == 0) {
        if (shared_w) ds += p_s[t * mp + m];
        else p.dSd[o] = p_s[t * mp + m];
      }
      dSe_part[o] = ds;
    }
    const int q4 = dvt / 4;
    for (int idx = tid; idx < BT * q4; idx += NT) {
      const int t = idx / q4, c = (idx % q4) * 4;
      if (t0 + t >= N || dv0 + c >= Dv) continue;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float4 x = *reinterpret_cast<const float4*>(dvpart + (w * BT + t) * dvt + c);
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
      }
      store4(p.dv_out, dtype, (((int64_t)b * N + t0 + t) * p.H + h) * Dv + dv0 + c, acc.x, acc.y, acc.z, acc.w);
    }
  };

  if (p.block_size <= 1) {
    const int last_tile = ((tend - 1) / BT) * BT;
    for (int t0 = last_tile; t0 >= tbeg; t0 -= BT) {
      __syncthreads();
      set_valid(t0);
      load_rows(vs, dvt, p.v, dtype, v_off, p.v_stride_n, t0, N, Dv, dv0, dvt);
      load_rows(dos, dvt, p.dy, dtype, dy_off, p.dy_stride_n, t0, N, Dv, dv0, dvt);
      load_plane(e_s, p.E, t0, 1);
      load_plane(g_s, p.G, t0, 1);
      load_plane(p_s, p.P, t0, p.DT);
      if (stablemax) load_plane(w_s, p.W2, t0, 1);
      __syncthreads();
      compute_gp();
      // reverse scan of c per latent
      for (int m = tid; m < M; m += NT) {
        float c = c_run[m], rho = rho_in[m];
        for (int t = BT - 1; t >= 0; --t) {
          if (!valid[t]) continue;
          c = g_s[t * mp + m] * p_s[t * mp + m] + rho * c;
          c_s[t * mp + m] = c;
          rho = 1.0f - e_s[t * mp + m];
        }
        c_run[m] = c;
      }
      __syncthreads();
      for (int idx = tid; idx < BT * M; idx += NT) {
        const int t = idx / M, m = idx % M;
        p_s[t * mp + m] = g_s[t * mp + m] * (p_s[t * mp + m] - gp[t]);
      }
      zero_dv();
#pragma unroll
      for (int t = BT - 1; t >= 0; --t) {
        if (!valid[t]) continue;
        const bool next_in_tile = (t + 1 < BT) && valid[t + 1 < BT ? t + 1 : t];
        float dd[DD];
#pragma unroll
        for (int j = 0; j < DD; ++j) dd[j] = dos[t * dvt + lane + 32 * j];
#pragma unroll
        for (int mi = 0; mi < MM_MAX; ++mi) {
          if (mi < mm) {
            const int m = warp * mm + mi;
            const float rho = next_in_tile ? 1.0f - e_s[(t + 1 < BT ? t + 1 : t) * mp + m] : rho_in[m];
            const float g = g_s[t * mp + m], e = e_s[t * mp + m];
#pragma unroll
            for (int j = 0; j < DD; ++j) {
              Bc[mi][j] = Bc[mi][j] * rho + g * dd[j];
              dvacc[t][j] += e * Bc[mi][j];
            }
          }
        }
        emit_bv(t);
      }
      __syncthreads();
      for (int m = tid; m < M; m += NT) rho_in[m] = 1.0f - e_s[m];  // token 0 of this tile is always valid
      finish_tile(t0, c_s, mp);
    }
  } else {
    const int bs = p.block_size;
    for (int blk0 = tend - bs; blk0 >= tbeg; blk0 -= bs) {
      const int blk_end = blk0 + bs;
      // pass 1: fold the whole block into the carries
      __syncthreads();
      for (int m = tid; m < M; m += NT) {
        c_run[m] *= rho_in[m];
        esum[m] = 0.f;
      }
#pragma unroll
      for (int mi = 0; mi < MM_MAX; ++mi) {
        if (mi < mm) {
          const float rho = rho_in[warp * mm + mi];
#pragma unroll
          for (int j = 0; j < DD; ++j) Bc[mi][j] *= rho;
        }
      }
      for (int t0 = blk0; t0 < blk_end; t0 += BT) {
        __syncthreads();
        load_rows(dos, dvt, p.dy, dtype, dy_off, p.dy_stride_n, t0, N, Dv, dv0, dvt);
        load_plane(e_s, p.E, t0, 1);
        load_plane(g_s, p.G, t0, 1);
        load_plane(p_s, p.P, t0, p.DT);
        __syncthreads();
        for (int m = tid; m < M; m += NT) {
          float c = c_run[m], es = esum[m];
          for (int t = 0; t < BT; ++t) {
            c += g_s[t * mp + m] * p_s[t * mp + m];
            es += e_s[t * mp + m];
          }
          c_run[m] = c;
          esum[m] = es;
        }
#pragma unroll 1
        for (int t = 0; t < BT; ++t) {
          float dd[DD];
#pragma unroll
          for (int j = 0; j < DD; ++j) dd[j] = dos[t * dvt + lane + 32 * j];
#pragma unroll
          for (int mi = 0; mi < MM_MAX; ++mi) {
            if (mi < mm) {
              const float g = g_s[t * mp + warp * mm + mi];
#pragma unroll
              for (int j = 0; j < DD; ++j) Bc[mi][j] += g * dd[j];
            }
          }
        }
      }
      // pass 2: gradients of every token of the block
      for (int t0 = blk0; t0 < blk_end; t0 += BT) {
        __syncthreads();
        set_valid(t0);
        load_rows(vs, dvt, p.v, dtype, v_off, p.v_stride_n, t0, N, Dv, dv0, dvt);
        load_plane(e_s, p.E, t0, 1);
        load_plane(g_s, p.G, t0, 1);
        load_plane(p_s, p.P, t0, p.DT);
        __syncthreads();
        compute_gp();
        __syncthreads();
        for (int idx = tid; idx < BT * M; idx += NT) {
          const int t = idx / M, m = idx % M;
          p_s[t * mp + m] = g_s[t * mp + m] * (p_s[t * mp + m] - gp[t]);
        }
        zero_dv();
#pragma unroll
        for (int t = 0; t < BT; ++t) {
#pragma unroll
          for (int mi = 0; mi < MM_MAX; ++mi) {
            if (mi < mm) {
              const float e = e_s[t * mp + warp * mm + mi];
#pragma unroll
              for (int j = 0; j < DD; ++j) dvacc[t][j] += e * Bc[mi][j];
            }
          }
          emit_bv(t);
        }
        __syncthreads();
        finish_tile(t0, c_run, 0);
      }
      __syncthreads();
      for (int m = tid; m < M; m += NT) rho_in[m] = 1.0f - esum[m];
    }
  }
}

#else
// --------------------------------------------------------------------------------------------------
// (3) token-row gradients: out[b, t, h, :] = scale * sum_src (sum_parts dS_src[t, :]) Lat_src[h]
// --------------------------------------------------------------------------------------------------
struct RowsParams {
  const float* ds[2];
  int parts[2];
  const void* lat[2];
  int64_t lat_stride_h[2], lat_stride_m[2];
  int nsrc;
  int64_t plane;
  void* out;  // [B, N, H, Dk] contiguous
  int B, N, H, M, Dk, dtype;
  float scale;
  const int* gate;  // optional: nothing is done unless *gate != 0
};

constexpr int RT = 64;    // token rows per CTA
constexpr int RM = 32;    // latents per shared-memory stage
constexpr int RC = 128;   // output columns per CTA (grid.z tiles wider rows)

// Register-tiled fp32 product: 256 threads, thread (ty, tx) owns rows ty*4 .. +3 and columns tx*8 .. +7 of the
// RT x RC output tile; per latent 6 shared-memory loads feed 32 FMAs.
__global__ void __launch_bounds__(NT) bwd_rows_kernel(const RowsParams p) {
  if (p.gate != nullptr && *p.gate == 0) return;
  __shared__ __align__(16) float ds_s[RT][RM + 4];
  __shared__ __align__(16) float lat_s[RM][RC];
  const int lane_id = blockIdx.x, t0 = blockIdx.y * RT, c0 = blockIdx.z * RC;
  const int b = lane_id / p.H, h = lane_id % p.H;
  const int M = p.M, Dk = p.Dk, N = p.N;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  for (int src = 0; src < p.nsrc; ++src) {
    for (int m0 = 0; m0 < M; m0 += RM) {
      __syncthreads();
      // dS tile (summed over the value-tile partials), zero outside the sequence / the latent range
      for (int idx = tid; idx < RT * (RM / 4); idx += NT) {
        const int t = idx / (RM / 4), c = (idx % (RM / 4)) * 4;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t0 + t < N && m0 + c < M) {
          for (int part = 0; part < p.parts[src]; ++part) {
            const float4 x = __ldcs(reinterpret_cast<const float4*>(p.ds[src] + (int64_t)part * p.plane +
                                                                    ((int64_t)lane_id * N + t0 + t) * M + m0 + c));
            a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
          }
        }
        *reinterpret_cast<float4*>(&ds_s[t][c]) = a;
      }
      // latent rows m0 .. m0 + RM - 1, columns c0 .. c0 + RC - 1, as fp32
      for (int idx = tid; idx < RM * (RC / 8); idx += NT) {
        const int m = idx / (RC / 8), c = (idx % (RC / 8)) * 8;
        float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (m0 + m < M && c0 + c < Dk)
          load8(p.lat[src], p.dtype, (int64_t)h * p.lat_stride_h[src] + (int64_t)(m0 + m) * p.lat_stride_m[src] + c0 + c, x);
        *reinterpret_cast<float4*>(&lat_s[m][c]) = make_float4(x[0], x[1], x[2], x[3]);
        *reinterpret_cast<float4*>(&lat_s[m][c + 4]) = make_float4(x[4], x[5], x[6], x[7]);
      }
      __syncthreads();
#pragma unroll 4
      for (int m = 0; m < RM; ++m) {
        const float4 l0 = *reinterpret_cast<const float4*>(&lat_s[m][tx * 8]);
        const float4 l1 = *reinterpret_cast<const float4*>(&lat_s[m][tx * 8 + 4]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float d = ds_s[ty * 4 + i][m];
          acc[i][0] += d * l0.x; acc[i][1] += d * l0.y; acc[i][2] += d * l0.z; acc[i][3] += d * l0.w;
          acc[i][4] += d * l1.x; acc[i][5] += d * l1.y; acc[i][6] += d * l1.z; acc[i][7] += d * l1.w;
        }
      }
    }
  }
  const int c = c0 + tx * 8;
  if (c < Dk) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = t0 + ty * 4 + i;
      if (t < N) {
        const int64_t o = (((int64_t)b * N + t) * p.H + h) * Dk + c;
        store4(p.out, p.dtype, o, acc[i][0] * p.scale, acc[i][1] * p.scale, acc[i][2] * p.scale, acc[i][3] * p.scale);
        store4(p.out, p.dtype, o + 4, acc[i][4] * p.scale, acc[i][5] * p.scale, acc[i][6] * p.scale, acc[i][7] * p.scale);
      }
    }
  }
}

// --------------------------------------------------------------------------------------------------
// (4) latent gradients: partial[split][h][m][dk] = scale * sum_src sum_{rows in split} dS_src[r, m] Rows_src[r, dk]
// --------------------------------------------------------------------------------------------------
struct LatParams {
  const float* ds[2];
  int parts[2];
  const void* rows[2];
  int64_t rows_stride_b[2], rows_stride_n[2], rows_stride_h[2];
  int nsrc;
  int64_t plane;
  float* partial;  // [splits][H][M][Dk]
  int B, N, H, M, Dk, dtype;
  int rows_per_split, splits;
  float scale;
  const int* gate;  // optional: nothing is done unless *gate != 0
};

constexpr int LM = 64;    // latents per CTA
constexpr int LDK = 128;  // score columns per CTA

constexpr int LT = 32;    // token rows per shared-memory stage

__global__ void __launch_bounds__(NT) bwd_lat_kernel(const LatParams p) {
  if (p.gate != nullptr && *p.gate == 0) return;
  __shared__ __align__(16) float ds_s[LT][LM + 4];
  __shared__ __align__(16) float rw_s[LT][LDK + 4];
  const int mtiles = (p.M + LM - 1) / LM;
  const int h = blockIdx.x / mtiles, m0 = (blockIdx.x % mtiles) * LM;
  const int split = blockIdx.y, dk0 = blockIdx.z * LDK;
  const int tid = threadIdx.x, tm = tid / 16, td = tid % 16;
  const int M = p.M, Dk = p.Dk, N = p.N;
  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  const int64_t total_rows = (int64_t)p.B * N;
  const int64_t r_begin = (int64_t)split * p.rows_per_split;
  const int64_t r_end = min(total_rows, r_begin + p.rows_per_split);
  for (int src = 0; src < p.nsrc; ++src) {
    for (int64_t r0 = r_begin; r0 < r_end; r0 += LT) {
      __syncthreads();
      // dS tile: LT rows x LM latents, 128-bit loads, summed over the value-tile partials
      for (int idx = tid; idx < LT * (LM / 4); idx += NT) {
        const int t = idx / (LM / 4), c = (idx % (LM / 4)) * 4;
        const int64_t r = r0 + t;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < r_end && m0 + c < M) {
          const int64_t bb = r / N, tt = r - bb * N;
          const float* src_p = p.ds[src] + ((bb * p.H + h) * N + tt) * M + m0 + c;
          for (int part = 0; part < p.parts[src]; ++part) {
            const float4 x = __ldcs(reinterpret_cast<const float4*>(src_p + (int64_t)part * p.plane));
            a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
          }
        }
        *reinterpret_cast<float4*>(&ds_s[t][c]) = a;
      }
      // token rows: LT rows x LDK columns, 8 elements per load
      for (int idx = tid; idx < LT * (LDK / 8); idx += NT) {
        const int t = idx / (LDK / 8), c = (idx % (LDK / 8)) * 8;
        const int64_t r = r0 + t;
        float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (r < r_end && dk0 + c < Dk) {
          const int64_t bb = r / N, tt = r - bb * N;
          load8(p.rows[src], p.dtype,
                bb * p.rows_stride_b[src] + tt * p.rows_stride_n[src] + (int64_t)h * p.rows_stride_h[src] + dk0 + c, x);
        }
        *reinterpret_cast<float4*>(&rw_s[t][c]) = make_float4(x[0], x[1], x[2], x[3]);
        *reinterpret_cast<float4*>(&rw_s[t][c + 4]) = make_float4(x[4], x[5], x[6], x[7]);
      }
      __syncthreads();
#pragma unroll 8
      for (int t = 0; t < LT; ++t) {
        float dsv[4], rv[8];
        const float4 d4 = *reinterpret_cast<const float4*>(&ds_s[t][tm * 4]);
        dsv[0] = d4.x; dsv[1] = d4.y; dsv[2] = d4.z; dsv[3] = d4.w;
#pragma unroll
        for (int j = 0; j < 8; ++j) rv[j] = rw_s[t][td + 16 * j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] += dsv[i] * rv[j];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int m = m0 + tm * 4 + i, dk = dk0 + td + 16 * j;
      if (m < M && dk < Dk) p.partial[(((int64_t)split * p.H + h) * M + m) * Dk + dk] = acc[i][j] * p.scale;
    }
}

// (5) out[i] = sum_split partial[split][i], fixed order
__global__ void bwd_sum_splits_kernel(float* out, const float* partial, int64_t n, int splits, const int* gate) {
  if (gate != nullptr && *gate == 0) return;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0.f;
  for (int s = 0; s < splits; ++s) acc += partial[(int64_t)s * n + i];
  out[i] = acc;
}

size_t replay_smem(int M, int Dk, int dd) {
  const int mp = M + 4, ldk = Dk + 4, dvt = 32 * dd;
  return ((size_t)2 * BT * ldk + 2 * BT * dvt + (size_t)4 * BT * mp + 6 * mp) * 4 + BT * sizeof(int);
}
size_t reverse_smem(int M, int dd, bool stablemax) {
  const int mp = M + 4, dvt = 32 * dd;
  return ((size_t)2 * BT * dvt + (size_t)(stablemax ? 6 : 5) * BT * mp + 3 * mp + BT + (size_t)NW * BT * dvt) * 4 +
         BT * sizeof(int);
}

struct BwdPlan {
  int dd, DT, splits, rows_per_split;
  int nseg, seg_len;  // sequence segments of the replay / reverse walks (token-causal read-out only)
  int64_t plane;
  size_t off_E, off_G, off_W2, off_P, off_dSe, off_dSd, off_part_q, off_part_kd, total;
  size_t off_seg_m, off_seg_d, off_seg_u, off_seg_b, off_seg_c, off_seg_gam, off_X, off_RHO;
};

// a span of a longer sequence: prefix state, carries from the right or a summary wanted
bool span_mode(const flare_bwd_args_t& a) {
  return a.fwd.state_in.u != nullptr || a.carry_b != nullptr || a.span_b0 != nullptr || a.phase != 0;
}

BwdPlan plan_backward(const flare_bwd_args_t& a) {
  const flare_fwd_args_t& f = a.fwd;
  BwdPlan pl;
  pl.dd = walk_exact_dd(f.M, f.Dv);
  pl.DT = (f.Dv + 32 * pl.dd - 1) / (32 * pl.dd);
  // The walks are sequential in the tokens; with few (lane, value tile) CTAs the sequence is cut into segments that
  // run concurrently (prefix states for the replay, carries (b, c) for the reverse walk, see bwd_exact()).
  // Measured at B=4, N=4096, H=16, M=64, D=128 (ms per training step): 2 segments 6.09, 4: 3.87, 8: 3.91, 16: 3.95;
  // narrower value tiles (more CTAs, repeated score work) are slower once the sequence is segmented (5.1-8.9).
  pl.nseg = 1;
  pl.seg_len = f.N;
  {
    // segments are whole 128-token chunks (forward kernels) and whole blocks (block-causal read-out)
    int unit = 128;
    if (f.block_size > 1) {
      int a = f.block_size, b = 128;
      while (b != 0) { const int t = a % b; a = b; b = t; }
      unit = f.block_size / a * 128;
    }
    const int min_seg = unit > 256 ? unit : 256;
    const int64_t ctas = (int64_t)f.B * f.H * pl.DT, target = 4LL * sm_count();
    int nseg = (int)((target + ctas - 1) / ctas);
    const int max_seg = f.N / min_seg;
    if (nseg > max_seg) nseg = max_seg;
    if (nseg > 1) {
      int seg_len = (f.N + nseg - 1) / nseg;
      seg_len = (seg_len + unit - 1) / unit * unit;
      pl.seg_len = seg_len;
      pl.nseg = (f.N + seg_len - 1) / seg_len;
    }
  }
  pl.plane = (int64_t)f.B * f.H * f.N * f.M;
  const bool stablemax = f.variant == FLARE_STABLEMAX;
  const bool shared_w = f.q_dec == nullptr && f.k_dec == nullptr;
  const int64_t rows = (int64_t)f.B * f.N;
  const int mt = (f.M + LM - 1) / LM, dkc = (f.Dk + LDK - 1) / LDK;
  int64_t splits = (2LL * sm_count() + (int64_t)f.H * mt * dkc - 1) / ((int64_t)f.H * mt * dkc);
  const int64_t max_splits = (rows + 255) / 256;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  int64_t rps = (rows + splits - 1) / splits;
  rps = (rps + LT - 1) / LT * LT;
  splits = (rows + rps - 1) / rps;
  pl.splits = (int)splits;
  pl.rows_per_split = (int)rps;
  size_t off = 0;
  auto take = [&](size_t floats) {
    const size_t o = off;
    off += align_up(floats * 4, 256);
    return o;
  };
  const size_t plane = (size_t)pl.plane;
  pl.off_E = take(plane);
  pl.off_G = take(plane);
  pl.off_W2 = stablemax ? take(plane) : pl.off_E;
  pl.off_P = take(plane * pl.DT);
  pl.off_dSe = take(plane * pl.DT);
  pl.off_dSd = shared_w ? 0 : take(plane);
  const size_t lat = (size_t)f.H * f.M * f.Dk;
  pl.off_part_q = take(lat * pl.splits);
  pl.off_part_kd = f.k_dec ? take(lat * pl.splits) : 0;
  pl.off_seg_m = pl.off_seg_d = pl.off_seg_u = pl.off_seg_b = pl.off_seg_c = pl.off_seg_gam = pl.off_X = pl.off_RHO = 0;
  if (pl.nseg > 1 || span_mode(a)) {
    const size_t ls = (size_t)f.B * f.H * pl.nseg;
    pl.off_seg_m = take(ls * f.M);
    pl.off_seg_d = take(ls * f.M);
    pl.off_seg_u = take(ls * f.M * f.Dv);
    pl.off_seg_b = take(ls * f.M * f.Dv);
    pl.off_seg_c = take(ls * f.M);
    pl.off_seg_gam = take(ls * f.M);
    pl.off_X = take(plane);
    pl.off_RHO = f.block_size > 1 ? take((size_t)f.B * f.H * (f.N / f.block_size) * f.M) : 0;
  }
  pl.total = off;
  return pl;
}

#endif

}  // namespace

#ifdef FLARE_WALK_MM
template <int MM_MAX, int DD>
static int launch_bwd_one(const BwdParams& p, dim3 grid, size_t smem1, size_t smem2, cudaStream_t stream, int stage) {
  if (stage == 0) {
    auto k1 = bwd_replay_kernel<MM_MAX, DD>;
    FLARE_CUDA_CHECK(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
    LaunchTimer timer("bwd_replay_kernel", stream);
    k1<<<grid, NT, smem1, stream>>>(p);
  } else {
    auto k2 = bwd_reverse_kernel<MM_MAX, DD>;
    FLARE_CUDA_CHECK(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
    LaunchTimer timer("bwd_reverse_kernel", stream);
    k2<<<grid, NT, smem2, stream>>>(p);
  }
  FLARE_CUDA_CHECK(cudaGetLastError());
  return FLARE_OK;
}

template <>
int launch_bwd_mm<FLARE_WALK_MM>(const BwdParams& p, int dd, dim3 grid, size_t smem1, size_t smem2, cudaStream_t stream,
                                 int stage) {
  constexpr int MM_MAX = FLARE_WALK_MM;
  if (dd == 1) return launch_bwd_one<MM_MAX, 1>(p, grid, smem1, smem2, stream, stage);
  if (dd == 2) {
    if constexpr (MM_MAX * 2 <= 64) return launch_bwd_one<MM_MAX, 2>(p, grid, smem1, smem2, stream, stage);
  }
  if (dd == 4) {
    if constexpr (MM_MAX * 4 <= 64) return launch_bwd_one<MM_MAX, 4>(p, grid, smem1, smem2, stream, stage);
  }
  return FLARE_ERR_UNSUPPORTED;
}
#else

// Carries of a segment for a zero carry-in, as products over its tokens (no sequential walk):
//   b0[m, :] = sum_t X[t, m] dY_t,   c0[m] = sum_t X[t, m] p[t, m].
// Register-tiled like the latent-gradient kernel: 64 latents x 128 value columns per CTA; grid.y = segment.
__global__ void __launch_bounds__(NT) bwd_seg_carry_kernel(const float* __restrict__ X, const float* __restrict__ P,
                                                           int p_parts, int64_t plane, const void* dy, int dtype, int64_t dy_stride_b,
                                                           int64_t dy_stride_n, int64_t dy_stride_h, float* seg_b,
                                                           float* seg_c, float* seg_gam, int nseg, int seg_len, int N,
                                                           int H, int M, int Dv, const int* gate) {
  if (gate != nullptr && *gate == 0) return;
  __shared__ __align__(16) float x_s[LT][LM + 4];
  __shared__ __align__(16) float dy_s[LT][LDK + 4];
  const int mtiles = (M + LM - 1) / LM;
  const int lane_id = blockIdx.x / mtiles, m0 = (blockIdx.x % mtiles) * LM;
  const int seg = blockIdx.y, dv0 = blockIdx.z * LDK;
  const int b = lane_id / H, h = lane_id % H;
  const int tid = threadIdx.x, tm = tid / 16, td = tid % 16;
  const int tbeg = seg * seg_len, tend = min(N, tbeg + seg_len);
  const int64_t row_base = (int64_t)lane_id * N;
  const int64_t st = (int64_t)lane_id * nseg + seg;
  float acc[4][8], cacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  for (int t0 = tbeg; t0 < tend; t0 += LT) {
    __syncthreads();
    for (int idx = tid; idx < LT * (LM / 4); idx += NT) {
      const int t = idx / (LM / 4), c = (idx % (LM / 4)) * 4;
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t0 + t < tend && m0 + c < M) {
        const int64_t o = (row_base + t0 + t) * M + m0 + c;
        x = __ldcs(reinterpret_cast<const float4*>(X + o));
        if (dv0 == 0) {
          // c0 partial of this thread's four latents for this token (threads of other rows add theirs below)
          float4 pp = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int part = 0; part < p_parts; ++part) {
            const float4 y = __ldcs(reinterpret_cast<const float4*>(P + (int64_t)part * plane + o));
            pp.x += y.x; pp.y += y.y; pp.z += y.z; pp.w += y.w;
          }
          // stash x * p behind the x values of the same row: columns LM/4 apart are not used, so keep it in registers
          // of the loading thread and reduce through shared memory after the loop instead
          cacc[0] += x.x * pp.x; cacc[1] += x.y * pp.y; cacc[2] += x.z * pp.z; cacc[3] += x.w * pp.w;
        }
      }
      *reinterpret_cast<float4*>(&x_s[t][c]) = x;
    }
    for (int idx = tid; idx < LT * (LDK / 8); idx += NT) {
      const int t = idx / (LDK / 8), c = (idx % (LDK / 8)) * 8;
      float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (t0 + t < tend && dv0 + c < Dv)
        load8(dy, dtype, (int64_t)b * dy_stride_b + (int64_t)(t0 + t) * dy_stride_n + (int64_t)h * dy_stride_h + dv0 + c, x);
      *reinterpret_cast<float4*>(&dy_s[t][c]) = make_float4(x[0], x[1], x[2], x[3]);
      *reinterpret_cast<float4*>(&dy_s[t][c + 4]) = make_float4(x[4], x[5], x[6], x[7]);
    }
    __syncthreads();
#pragma unroll 8
    for (int t = 0; t < LT; ++t) {
      const float4 d4 = *reinterpret_cast<const float4*>(&x_s[t][tm * 4]);
      const float dsv[4] = {d4.x, d4.y, d4.z, d4.w};
      float rv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) rv[j] = dy_s[t][td + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] += dsv[i] * rv[j];
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int m = m0 + tm * 4 + i, dv = dv0 + td + 16 * j;
      if (m < M && dv < Dv) seg_b[(st * M + m) * Dv + dv] = acc[i][j];
    }
  if (dv0 == 0) {
    // c0: the loading threads hold partial sums for columns (tid % 16) * 4 .. + 3 over the rows tid / 16 + 16 k
    __syncthreads();
    float* red = &dy_s[0][0];  // [16 row groups][LM]
    if (tid < LT * (LM / 4) && tid < NT) {
      const int rg = tid / (LM / 4), c = (tid % (LM / 4)) * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) red[rg * LM + c + i] = cacc[i];
    }
    __syncthreads();
    if (tid < LM && m0 + tid < M) {
      float c0 = 0.f;
      for (int rg = 0; rg < NT / (LM / 4); ++rg) c0 += red[rg * LM + tid];
      seg_c[st * M + m0 + tid] = c0;
    }
  }
}

// Right-to-left scan of the segment carries.  On entry slot s holds (b, c) at the first token of segment s for a zero
// carry-in and seg_gam the product of its internal decays; with rho_next(s) = decay of the first token (block) after
// segment s, b(s) = own(s) + gam(s) rho_next(s) b(s + 1).  write_slots: slot s receives the carry that enters segment
// s from the right (what the reverse walk starts from).  The totals of the whole span (b, c at its first token for the
// given right-hand carry, the product of all its decays, the decay of its own first token) go to the span_* outputs
// when those are given.
__global__ void __launch_bounds__(256) bwd_seg_scan_kernel(float* seg_b, float* seg_c, const float* seg_gam, int nseg,
                                                           int seg_len, int64_t lanes, int N, int M, int Dv,
                                                           const float* __restrict__ E, const float* __restrict__ RHO,
                                                           int block_size, const float* carry_b, const float* carry_c,
                                                           const float* carry_rho, int write_slots, float* span_b0,
                                                           float* span_c0, float* span_gam, float* span_rho_first,
                                                           const int* gate) {
  if (gate != nullptr && *gate == 0) return;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t per_lane = (int64_t)M * (Dv + 1);  // Dv columns of b, then c
  if (idx >= lanes * per_lane) return;
  const int64_t lane_id = idx / per_lane;
  const int r = (int)(idx % per_lane);
  const int m = r / (Dv + 1), col = r % (Dv + 1);
  auto decay_at = [&](int t) -> float {  // decay of the token (block) that starts at t
    return block_size <= 1 ? 1.0f - E[(lane_id * N + t) * M + m]
                           : RHO[(lane_id * (N / block_size) + t / block_size) * M + m];
  };
  float run = 0.f;
  if (carry_b != nullptr) run = col < Dv ? carry_b[(lane_id * M + m) * Dv + col] : carry_c[lane_id * M + m];
  float gprod = 1.0f;
  for (int s = nseg - 1; s >= 0; --s) {
    const int64_t st = lane_id * nseg + s;
    float* slot = col < Dv ? seg_b + (st * M + m) * Dv + col : seg_c + st * M + m;
    const float own = *slot;
    const int t_next = (s + 1) * seg_len;
    const float rho_next = t_next < N ? decay_at(t_next) : (carry_rho != nullptr ? carry_rho[lane_id * M + m] : 0.f);
    const float gam = seg_gam[st * M + m];
    if (write_slots) *slot = run;
    run = own + gam * rho_next * run;
    gprod *= gam * (t_next < N ? rho_next : 1.0f);  // internal decays only
  }
  if (span_b0 != nullptr) {
    if (col < Dv) {
      span_b0[(lane_id * M + m) * Dv + col] = run;
    } else {
      span_c0[lane_id * M + m] = run;
      span_gam[lane_id * M + m] = gprod;
      span_rho_first[lane_id * M + m] = decay_at(0);
    }
  }
}

size_t bwd_exact_workspace_bytes(const flare_bwd_args_t& a) {
  if (a.fwd.B == 0 || a.fwd.N == 0) return 0;
  return plan_backward(a).total;
}

int bwd_exact(const flare_bwd_args_t& a, cudaStream_t stream, const int* gate) {
  const flare_fwd_args_t& f = a.fwd;
  if (f.B == 0 || f.N == 0) return FLARE_OK;
  if (f.M > 512) return FLARE_ERR_UNSUPPORTED;
  const BwdPlan pl = plan_backward(a);
  if (f.workspace == nullptr || f.workspace_bytes < pl.total || (reinterpret_cast<uintptr_t>(f.workspace) & 15u))
    return FLARE_ERR_WORKSPACE;
  char* ws = reinterpret_cast<char*>(f.workspace);
  const bool stablemax = f.variant == FLARE_STABLEMAX;
  const bool shared_w = f.q_dec == nullptr && f.k_dec == nullptr;
  BwdParams p;
  memset(&p, 0, sizeof(p));
  p.q = f.q; p.k = f.k; p.v = f.v; p.qd = f.q_dec; p.kd = f.k_dec; p.dy = a.dy;
  p.B = f.B; p.N = f.N; p.H = f.H; p.M = f.M; p.Dk = f.Dk; p.Dv = f.Dv;
  p.q_stride_h = f.q_stride_h; p.q_stride_m = f.q_stride_m;
  p.k_stride_b = f.k_stride_b; p.k_stride_n = f.k_stride_n; p.k_stride_h = f.k_stride_h;
  p.v_stride_b = f.v_stride_b; p.v_stride_n = f.v_stride_n; p.v_stride_h = f.v_stride_h;
  p.qd_stride_b = f.qd_stride_b; p.qd_stride_n = f.qd_stride_n; p.qd_stride_h = f.qd_stride_h;
  p.kd_stride_h = f.kd_stride_h; p.kd_stride_m = f.kd_stride_m;
  p.dy_stride_b = a.dy_stride_b; p.dy_stride_n = a.dy_stride_n; p.dy_stride_h = a.dy_stride_h;
  p.scale = f.scale; p.power = f.power; p.dtype = f.dtype; p.variant = f.variant; p.block_size = f.block_size;
  p.E = reinterpret_cast<float*>(ws + pl.off_E);
  p.G = reinterpret_cast<float*>(ws + pl.off_G);
  p.W2 = reinterpret_cast<float*>(ws + pl.off_W2);
  p.P = reinterpret_cast<float*>(ws + pl.off_P);
  p.dSe = reinterpret_cast<float*>(ws + pl.off_dSe);
  p.dSd = shared_w ? nullptr : reinterpret_cast<float*>(ws + pl.off_dSd);
  p.DT = pl.DT; p.plane = pl.plane; p.dv_out = a.dv;
  p.nseg = pl.nseg; p.seg_len = pl.seg_len; p.seg_first = 0;
  const int64_t lanes = (int64_t)f.B * f.H;
  const bool seg_mode = pl.nseg > 1 || span_mode(a);
  if (a.phase < 0 || a.phase > 2 || (a.span_b0 != nullptr && !(a.span_c0 && a.span_gam && a.span_rho_first)) ||
      (a.carry_b != nullptr && !(a.carry_c && a.carry_rho)) || (span_mode(a) && f.block_size > 1 && f.N % f.block_size))
    return FLARE_ERR_BAD_POINTER;
  float *seg_m = nullptr, *seg_d = nullptr, *seg_u = nullptr;
  if (seg_mode) {
    seg_m = reinterpret_cast<float*>(ws + pl.off_seg_m);
    seg_d = reinterpret_cast<float*>(ws + pl.off_seg_d);
    seg_u = reinterpret_cast<float*>(ws + pl.off_seg_u);
    p.in_m = seg_m; p.in_d = seg_d; p.in_u = seg_u;
    p.seg_b = reinterpret_cast<float*>(ws + pl.off_seg_b);
    p.seg_c = reinterpret_cast<float*>(ws + pl.off_seg_c);
    p.seg_gam = reinterpret_cast<float*>(ws + pl.off_seg_gam);
    p.X = reinterpret_cast<float*>(ws + pl.off_X);
    p.RHO = f.block_size > 1 ? reinterpret_cast<float*>(ws + pl.off_RHO) : nullptr;
  }
  p.carry_b = a.carry_b; p.carry_c = a.carry_c; p.carry_rho = a.carry_rho;
  p.gate = gate;

  const int mm = f.M / NW;
  const size_t smem1 = replay_smem(f.M, f.Dk, pl.dd), smem2 = reverse_smem(f.M, pl.dd, stablemax);
  if (smem1 > 227 * 1024 || smem2 > 227 * 1024) return FLARE_ERR_UNSUPPORTED;
  auto walk = [&](int stage, int seg_first, int seg_count) -> int {
    BwdParams q = p;
    q.seg_first = seg_first;
    dim3 grid(f.B * f.H, pl.DT, seg_count);
    if (mm <= 2) return launch_bwd_mm<2>(q, pl.dd, grid, smem1, smem2, stream, stage);
    if (mm <= 8) return launch_bwd_mm<8>(q, pl.dd, grid, smem1, smem2, stream, stage);
    if (mm <= 16) return launch_bwd_mm<16>(q, pl.dd, grid, smem1, smem2, stream, stage);
    if (mm <= 32) return launch_bwd_mm<32>(q, pl.dd, grid, smem1, smem2, stream, stage);
    return launch_bwd_mm<64>(q, pl.dd, grid, smem1, smem2, stream, stage);
  };
  const int64_t nscan = lanes * f.M * (f.Dv + 1);
  auto scan = [&](bool write_slots, bool with_carry, bool summary) -> int {
    LaunchTimer timer("bwd_seg_scan_kernel", stream);
    bwd_seg_scan_kernel<<<(unsigned)((nscan + 255) / 256), 256, 0, stream>>>(
        p.seg_b, p.seg_c, p.seg_gam, pl.nseg, pl.seg_len, lanes, f.N, f.M, f.Dv, p.E, p.RHO, f.block_size,
        with_carry ? a.carry_b : nullptr, with_carry ? a.carry_c : nullptr, with_carry ? a.carry_rho : nullptr,
        write_slots ? 1 : 0, summary ? a.span_b0 : nullptr, a.span_c0, a.span_gam, a.span_rho_first, gate);
    FLARE_CUDA_CHECK(cudaGetLastError());
    return FLARE_OK;
  };
  int rcw = FLARE_OK;
  if (a.phase != 2) {
    if (seg_mode) {
      // exclusive prefix state of every segment, from the forward kernels (slot 0: the state before the span)
      rcw = segment_prefix_states(&f, pl.nseg, pl.seg_len, seg_m, seg_d, seg_u,
                                  f.state_in.u != nullptr ? &f.state_in : nullptr, stream, gate);
      if (rcw != FLARE_OK) return rcw;
    }
    rcw = walk(0, 0, pl.nseg);  // replay: planes e, g, p (and X, the carry weights, when segmented)
    if (rcw != FLARE_OK) return rcw;
    if (seg_mode) {
      // carries of every segment for a zero carry-in, as products over the planes
      const int mt = (f.M + LM - 1) / LM;
      dim3 g((unsigned)(lanes * mt), pl.nseg, (f.Dv + LDK - 1) / LDK);
      LaunchTimer timer("bwd_seg_carry_kernel", stream);
      bwd_seg_carry_kernel<<<g, NT, 0, stream>>>(p.X, p.P, pl.DT, pl.plane, a.dy, f.dtype, a.dy_stride_b, a.dy_stride_n,
                                                 a.dy_stride_h, p.seg_b, p.seg_c, p.seg_gam, pl.nseg, pl.seg_len, f.N,
                                                 f.H, f.M, f.Dv, gate);
      FLARE_CUDA_CHECK(cudaGetLastError());
      if (a.span_b0 != nullptr) {
        rcw = scan(false, false, true);  // summary of the span for a zero carry-in from the right
        if (rcw != FLARE_OK) return rcw;
      }
    }
    if (a.phase == 1) return FLARE_OK;
  }
  if (seg_mode) {
    rcw = scan(true, true, false);  // right-to-left scan: every segment's true carry-in
    if (rcw != FLARE_OK) return rcw;
  }
  rcw = walk(1, 0, pl.nseg);  // reverse walk: dV and the dS planes
  if (rcw != FLARE_OK) return rcw;

  // ---- dK (+ dQ_dec): products of the dS planes with the latent banks ------------------------------
  auto rows_launch = [&](RowsParams& r) -> int {
    r.plane = pl.plane; r.B = f.B; r.N = f.N; r.H = f.H; r.M = f.M; r.Dk = f.Dk; r.dtype = f.dtype; r.scale = f.scale;
    r.gate = gate;
    dim3 g(f.B * f.H, (f.N + RT - 1) / RT, (f.Dk + RC - 1) / RC);
    LaunchTimer timer("bwd_rows_kernel", stream);
    bwd_rows_kernel<<<g, NT, 0, stream>>>(r);
    FLARE_CUDA_CHECK(cudaGetLastError());
    return FLARE_OK;
  };
  {
    RowsParams r;
    memset(&r, 0, sizeof(r));
    r.out = a.dk;
    r.ds[0] = p.dSe; r.parts[0] = pl.DT; r.lat[0] = f.q; r.lat_stride_h[0] = f.q_stride_h; r.lat_stride_m[0] = f.q_stride_m;
    r.nsrc = 1;
    if (!shared_w && f.q_dec == nullptr) {  // decode queries are the keys: their gradient lands on K
      r.ds[1] = p.dSd; r.parts[1] = 1; r.lat[1] = f.k_dec; r.lat_stride_h[1] = f.kd_stride_h; r.lat_stride_m[1] = f.kd_stride_m;
      r.nsrc = 2;
    }
    int rc = rows_launch(r);
    if (rc != FLARE_OK) return rc;
  }
  if (f.q_dec != nullptr) {
    RowsParams r;
    memset(&r, 0, sizeof(r));
    r.out = a.dq_dec;
    r.ds[0] = p.dSd; r.parts[0] = 1;
    r.lat[0] = f.k_dec ? f.k_dec : f.q;
    r.lat_stride_h[0] = f.k_dec ? f.kd_stride_h : f.q_stride_h;
    r.lat_stride_m[0] = f.k_dec ? f.kd_stride_m : f.q_stride_m;
    r.nsrc = 1;
    int rc = rows_launch(r);
    if (rc != FLARE_OK) return rc;
  }

  // ---- dQ (+ dK_dec): split partial sums, then a fixed-order reduction -------------------------------
  const int mt = (f.M + LM - 1) / LM, dkc = (f.Dk + LDK - 1) / LDK;
  const int64_t lat_n = (int64_t)f.H * f.M * f.Dk;
  auto lat_launch = [&](LatParams& l, float* partial, float* out) -> int {
    l.plane = pl.plane; l.B = f.B; l.N = f.N; l.H = f.H; l.M = f.M; l.Dk = f.Dk; l.dtype = f.dtype; l.scale = f.scale;
    l.gate = gate;
    l.rows_per_split = pl.rows_per_split; l.splits = pl.splits; l.partial = partial;
    dim3 g(f.H * mt, pl.splits, dkc);
    {
      LaunchTimer timer("bwd_lat_kernel", stream);
      bwd_lat_kernel<<<g, NT, 0, stream>>>(l);
    }
    FLARE_CUDA_CHECK(cudaGetLastError());
    LaunchTimer timer("bwd_sum_splits_kernel", stream);
    bwd_sum_splits_kernel<<<(unsigned)((lat_n + 255) / 256), 256, 0, stream>>>(out, partial, lat_n, pl.splits, gate);
    FLARE_CUDA_CHECK(cudaGetLastError());
    return FLARE_OK;
  };
  {
    LatParams l;
    memset(&l, 0, sizeof(l));
    l.ds[0] = p.dSe; l.parts[0] = pl.DT; l.rows[0] = f.k;
    l.rows_stride_b[0] = f.k_stride_b; l.rows_stride_n[0] = f.k_stride_n; l.rows_stride_h[0] = f.k_stride_h;
    l.nsrc = 1;
    if (!shared_w && f.k_dec == nullptr) {  // decode keys are the latent queries: their gradient lands on Q
      l.ds[1] = p.dSd; l.parts[1] = 1; l.rows[1] = f.q_dec;
      l.rows_stride_b[1] = f.qd_stride_b; l.rows_stride_n[1] = f.qd_stride_n; l.rows_stride_h[1] = f.qd_stride_h;
      l.nsrc = 2;
    }
    int rc = lat_launch(l, reinterpret_cast<float*>(ws + pl.off_part_q), a.dq);
    if (rc != FLARE_OK) return rc;
  }
  if (f.k_dec != nullptr) {
    LatParams l;
    memset(&l, 0, sizeof(l));
    l.ds[0] = p.dSd; l.parts[0] = 1;
    l.rows[0] = f.q_dec ? f.q_dec : f.k;
    l.rows_stride_b[0] = f.q_dec ? f.qd_stride_b : f.k_stride_b;
    l.rows_stride_n[0] = f.q_dec ? f.qd_stride_n : f.k_stride_n;
    l.rows_stride_h[0] = f.q_dec ? f.qd_stride_h : f.k_stride_h;
    l.nsrc = 1;
    int rc = lat_launch(l, reinterpret_cast<float*>(ws + pl.off_part_kd), a.dk_dec);
    if (rc != FLARE_OK) return rc;
  }
  return FLARE_OK;
}
#endif

}  // namespace flare
