// Exact (fp32, CUDA-core) sequential walk over the tokens of one (batch, head) lane.
//
// This is the general path of the library: any dtype, any M/Dk/Dv that are multiples of 16,
// separate decode weights, attention masks, carry-in / carry-out state, token-causal or
// block-causal read-out, softmax or stablemax encoder weights.  It evaluates the online
// recurrence token by token, so it is exact for arbitrarily sharp score distributions.
//
// Work split: grid = (lane, segment, Dv tile).  A CTA walks the tokens of its segment in tiles
// of 16: (1) stage the K/V rows in shared memory as fp32, (2) all 16 x M scores with fp32 FMAs,
// (3) decode softmax over the latents, one warp per token, (4) per-latent running statistics,
// one thread per latent, (5) the state replay: warp w owns latents [w*M/8, (w+1)*M/8), lane l owns
// value columns l, l+32, ... of the tile; state and per-token output partials live in registers,
// (6) cross-warp reduction of the output partials through shared memory.
#include "walk_exact.cuh"
#include "walk_device.cuh"

namespace flare {

using namespace walk;

template <int MM_MAX, int DD>
__global__ void __launch_bounds__(NT, (MM_MAX * DD <= 32) ? 2 : 1) walk_exact_kernel(const WalkParams p) {
  extern __shared__ __align__(16) float smem_raw[];
  const int lane_id = blockIdx.x;  // (b, h) lane
  if (p.gate != nullptr && p.gate[(int64_t)lane_id * p.gate_stride] == 0) return;
  const int seg = blockIdx.y;
  const int b = lane_id / p.H, h = lane_id % p.H;
  const int dvt = 32 * DD;
  const int dv0 = blockIdx.z * dvt;
  const int M = p.M, Dk = p.Dk, Dv = p.Dv;
  const int mp = M + 4, ldk = Dk + 4;
  Smem sm = carve(smem_raw, ldk, dvt, mp);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mm = M / NW;  // latents per warp
  const bool shared_w = (p.qd == nullptr && p.kd == nullptr);
  const bool stablemax = p.variant == FLARE_STABLEMAX;
  const int dtype = p.dtype;

  const int seg_begin = seg * p.seg_len;
  const int seg_end = min(p.N, seg_begin + p.seg_len);

  // ---- carry-in state ------------------------------------------------------------------------
  float U[MM_MAX][DD];
  {
    const int64_t sidx = (int64_t)lane_id * p.in_lane_stride + (int64_t)seg * p.in_seg_stride;
    for (int m = tid; m < M; m += NT) {
      sm.m_run[m] = p.in_m ? p.in_m[sidx * M + m] : (stablemax ? 0.f : kNegInf);
      sm.d_run[m] = p.in_d ? p.in_d[sidx * M + m] : 0.f;
    }
#pragma unroll
    for (int mi = 0; mi < MM_MAX; ++mi)
#pragma unroll
      for (int j = 0; j < DD; ++j) {
        const int dv = dv0 + lane + 32 * j;
        U[mi][j] = (p.in_u && mi < mm && dv < Dv) ? p.in_u[(sidx * M + warp * mm + mi) * Dv + dv] : 0.f;
      }
  }
  __syncthreads();

  const int64_t k_off = (int64_t)b * p.k_stride_b + (int64_t)h * p.k_stride_h;
  const int64_t v_off = (int64_t)b * p.v_stride_b + (int64_t)h * p.v_stride_h;
  const int64_t qd_off = (int64_t)b * p.qd_stride_b + (int64_t)h * p.qd_stride_h;
  const int64_t y_off = (int64_t)b * p.y_stride_b + (int64_t)h * p.y_stride_h;
  const int64_t q_off = (int64_t)h * p.q_stride_h;
  const int64_t kd_off = (int64_t)h * p.kd_stride_h;
  const int dcount_v = dvt;

  auto set_valid = [&](int t0) {
    if (tid < BT) {
      const int t = t0 + tid;
      int ok = t < seg_end;
      if (ok && p.mask != nullptr) ok = p.mask[(int64_t)b * p.N + t] != 0;
      sm.valid[tid] = ok;
    }
  };

  // Per-latent running statistics for the 16 tokens of the tile: s -> eta, g <- gamma.
  // ar_weights: also turn the decode softmax in a[] into the read-out weight softmax / d_t.
  auto stats_scan = [&](bool ar_weights) {
    for (int m = tid; m < M; m += NT) {
      float mr = sm.m_run[m], dr = sm.d_run[m];
#pragma unroll 4
      for (int t = 0; t < BT; ++t) {
        if (!sm.valid[t]) continue;
        const float s = sm.s[t * mp + m];
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
        sm.g[t * mp + m] = gam;
        sm.s[t * mp + m] = eta;
        if (ar_weights) sm.a[t * mp + m] *= 1.0f / (dr > 0.f ? dr : 1.f);
      }
      sm.m_run[m] = mr;
      sm.d_run[m] = dr;
    }
  };

  float yacc[BT][DD];
  auto zero_y = [&]() {
#pragma unroll
    for (int t = 0; t < BT; ++t)
#pragma unroll
      for (int j = 0; j < DD; ++j) yacc[t][j] = 0.f;
  };

  // state update and/or read-out for the tile currently staged in shared memory
  auto replay = [&](bool update, bool readout) {
#pragma unroll
    for (int t = 0; t < BT; ++t) {
      if (!sm.valid[t]) continue;
      float vv[DD];
#pragma unroll
      for (int j = 0; j < DD; ++j) vv[j] = sm.vs[t * dvt + lane + 32 * j];
#pragma unroll
      for (int mi = 0; mi < MM_MAX; ++mi) {
        if (mi < mm) {
          const int m = warp * mm + mi;
          if (update) {
            const float gam = sm.g[t * mp + m], eta = sm.s[t * mp + m];
#pragma unroll
            for (int j = 0; j < DD; ++j) U[mi][j] = U[mi][j] * gam + eta * vv[j];
          }
          if (readout) {
            const float w = sm.a[t * mp + m];
#pragma unroll
            for (int j = 0; j < DD; ++j) yacc[t][j] += w * U[mi][j];
          }
        }
      }
    }
  };

  auto store_y = [&](int t0) {
#pragma unroll
    for (int t = 0; t < BT; ++t)
#pragma unroll
      for (int j = 0; j < DD; ++j) sm.ypart[(warp * BT + t) * dvt + lane + 32 * j] = yacc[t][j];
    __syncthreads();
    const int q4 = dvt / 4;
    for (int idx = tid; idx < BT * q4; idx += NT) {
      const int t = idx / q4, c = (idx % q4) * 4;
      if (t0 + t >= seg_end || dv0 + c >= Dv) continue;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float4 x = *reinterpret_cast<const float4*>(sm.ypart + (w * BT + t) * dvt + c);
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
      }
      store4(p.y, dtype, y_off + (int64_t)(t0 + t) * p.y_stride_n + dv0 + c, acc.x, acc.y, acc.z, acc.w);
    }
  };

  if (p.block_size <= 1) {
    // ------------------------------ token-causal walk ----------------------------------------
    for (int t0 = seg_begin; t0 < seg_end; t0 += BT) {
      __syncthreads();
      set_valid(t0);
      load_rows(sm.ks, ldk, p.k, dtype, k_off, p.k_stride_n, t0, seg_end, Dk, 0, Dk);
      load_rows(sm.vs, dvt, p.v, dtype, v_off, p.v_stride_n, t0, seg_end, Dv, dv0, dcount_v);
      if (p.qd != nullptr) load_rows(sm.qds, ldk, p.qd, dtype, qd_off, p.qd_stride_n, t0, seg_end, Dk, 0, Dk);
      __syncthreads();
      score_tile(sm.s, mp, sm.ks, ldk, p.q, dtype, q_off, p.q_stride_m, M, Dk, p.scale);
      if (p.write_y && !shared_w) {
        score_tile(sm.a, mp, p.qd ? sm.qds : sm.ks, ldk, p.kd ? p.kd : p.q, dtype, p.kd ? kd_off : q_off,
                   p.kd ? p.kd_stride_m : p.q_stride_m, M, Dk, p.scale);
      }
      __syncthreads();
      if (p.write_y) {
        float* lse = (p.lse_dec != nullptr && blockIdx.z == 0) ? p.lse_dec + (int64_t)lane_id * p.N + t0 : nullptr;
        decode_softmax(sm.a, shared_w ? sm.s : sm.a, mp, M, sm.valid, lse, t0, seg_end);
        __syncthreads();
      }
      stats_scan(p.write_y != 0);
      __syncthreads();
      zero_y();
      replay(true, p.write_y != 0);
      if (p.write_y) store_y(t0);
    }
  } else {
    // ------------------------------ block-causal walk ----------------------------------------
    const int bs = p.block_size;
    for (int blk0 = seg_begin; blk0 < seg_end; blk0 += bs) {
      const int blk_end = min(seg_end, blk0 + bs);
      for (int t0 = blk0; t0 < blk_end; t0 += BT) {
        __syncthreads();
        set_valid(t0);
        load_rows(sm.ks, ldk, p.k, dtype, k_off, p.k_stride_n, t0, blk_end, Dk, 0, Dk);
        load_rows(sm.vs, dvt, p.v, dtype, v_off, p.v_stride_n, t0, blk_end, Dv, dv0, dcount_v);
        __syncthreads();
        score_tile(sm.s, mp, sm.ks, ldk, p.q, dtype, q_off, p.q_stride_m, M, Dk, p.scale);
        __syncthreads();
        stats_scan(false);
        __syncthreads();
        replay(true, false);
      }
      __syncthreads();
      for (int m = tid; m < M; m += NT) {
        const float dr = sm.d_run[m];
        sm.dinv[m] = 1.0f / (dr > 0.f ? dr : 1.f);
        if (p.lse_enc != nullptr && blockIdx.z == 0) {
          const int64_t nb = p.N / bs;
          p.lse_enc[((int64_t)lane_id * nb + blk0 / bs) * M + m] = logf(fmaxf(dr, 1e-20f)) + sm.m_run[m];
        }
      }
      if (!p.write_y) continue;
      for (int t0 = blk0; t0 < blk_end; t0 += BT) {
        __syncthreads();
        set_valid(t0);
        if (p.qd != nullptr) load_rows(sm.ks, ldk, p.qd, dtype, qd_off, p.qd_stride_n, t0, blk_end, Dk, 0, Dk);
        else load_rows(sm.ks, ldk, p.k, dtype, k_off, p.k_stride_n, t0, blk_end, Dk, 0, Dk);
        __syncthreads();
        score_tile(sm.a, mp, sm.ks, ldk, p.kd ? p.kd : p.q, dtype, p.kd ? kd_off : q_off,
                   p.kd ? p.kd_stride_m : p.q_stride_m, M, Dk, p.scale);
        __syncthreads();
        float* lse = (p.lse_dec != nullptr && blockIdx.z == 0) ? p.lse_dec + (int64_t)lane_id * p.N + t0 : nullptr;
        decode_softmax(sm.a, sm.a, mp, M, sm.valid, lse, t0, blk_end);
        __syncthreads();
        for (int idx = tid; idx < BT * M; idx += NT) {
          const int t = idx / M, m = idx % M;
          sm.a[t * mp + m] *= sm.dinv[m];
        }
        __syncthreads();
        zero_y();
        replay(false, true);
        store_y(t0);
      }
    }
  }

  // ---- carry-out state -------------------------------------------------------------------------
  const bool write_out = p.out_mode == 1 || (p.out_mode == 2 && seg == p.nseg_total - 1);
  if (write_out && p.out_u != nullptr) {
    __syncthreads();
    const int64_t sidx = (int64_t)lane_id * p.out_lane_stride + (int64_t)seg * p.out_seg_stride;
    if (blockIdx.z == 0) {
      for (int m = tid; m < M; m += NT) {
        p.out_m[sidx * M + m] = sm.m_run[m];
        p.out_d[sidx * M + m] = sm.d_run[m];
      }
    }
#pragma unroll
    for (int mi = 0; mi < MM_MAX; ++mi)
#pragma unroll
      for (int j = 0; j < DD; ++j) {
        const int dv = dv0 + lane + 32 * j;
        if (mi < mm && dv < Dv) p.out_u[(sidx * M + warp * mm + mi) * Dv + dv] = U[mi][j];
      }
  }
}

static size_t walk_exact_smem_bytes(int M, int Dk, int dd) {
  const int mp = M + 4, ldk = Dk + 4, dvt = 32 * dd;
  size_t floats = (size_t)2 * BT * ldk + (size_t)BT * dvt + (size_t)3 * BT * mp + 3 * mp + (size_t)NW * BT * dvt;
  return floats * 4 + BT * sizeof(int);
}

#ifdef FLARE_WALK_MM
// One translation unit per latents-per-warp bound, so the instantiations compile in parallel.
template <int MM_MAX, int DD>
static int launch_one(const WalkParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
  auto kern = walk_exact_kernel<MM_MAX, DD>;
  FLARE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  LaunchTimer timer(p.gate != nullptr ? "walk_exact_kernel (standby)" : "walk_exact_kernel", stream);
  kern<<<grid, NT, smem, stream>>>(p);
  FLARE_CUDA_CHECK(cudaGetLastError());
  return FLARE_OK;
}

template <>
int launch_walk_mm<FLARE_WALK_MM>(const WalkParams& p, int dd, dim3 grid, size_t smem, cudaStream_t stream) {
  constexpr int MM_MAX = FLARE_WALK_MM;
  if (dd == 1) return launch_one<MM_MAX, 1>(p, grid, smem, stream);
  if (dd == 2) {
    if constexpr (MM_MAX * 2 <= 64) return launch_one<MM_MAX, 2>(p, grid, smem, stream);
  }
  if (dd == 4) {
    if constexpr (MM_MAX * 4 <= 64) return launch_one<MM_MAX, 4>(p, grid, smem, stream);
  }
  return FLARE_ERR_UNSUPPORTED;
}
#else
int walk_exact_dd(int M, int Dv) {
  const int mm = M / NW;
  int dd = 1;
  while (dd < 4 && dd * 32 < Dv && mm * dd * 2 <= 64) dd *= 2;
  return dd;
}

int launch_walk_exact(const WalkParams& p, int nseg_grid, cudaStream_t stream) {
  if (p.M % 16 != 0 || p.M > 512) return FLARE_ERR_UNSUPPORTED;
  if (nseg_grid <= 0 || p.B * p.H <= 0) return FLARE_OK;
  const int mm = p.M / NW;
  const int dd = walk_exact_dd(p.M, p.Dv);
  const int dvt = 32 * dd;
  dim3 grid(p.B * p.H, nseg_grid, (p.Dv + dvt - 1) / dvt);
  const size_t smem = walk_exact_smem_bytes(p.M, p.Dk, dd);
  if (smem > 227 * 1024) return FLARE_ERR_UNSUPPORTED;
  if (mm <= 2) return launch_walk_mm<2>(p, dd, grid, smem, stream);
  if (mm <= 8) return launch_walk_mm<8>(p, dd, grid, smem, stream);
  if (mm <= 16) return launch_walk_mm<16>(p, dd, grid, smem, stream);
  if (mm <= 32) return launch_walk_mm<32>(p, dd, grid, smem, stream);
  return launch_walk_mm<64>(p, dd, grid, smem, stream);
}
#endif

}  // namespace flare
