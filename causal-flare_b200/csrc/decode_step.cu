// One decode token per (batch, head) lane: HBM-bound in-place update of the fp32 latent state.
//
// Per lane the kernel reads and writes u [M, Dv] fp32 once (128-bit accesses, streaming cache hints so the
// shared latent bank Q stays resident in L2), plus m, d [M].  Phases inside a CTA (one CTA per lane):
//   0. issue the first batch of state loads so they are in flight while scores are computed
//   1. scores s[m] = scale <q_m, k>, 8 lanes per latent, 16-byte loads of Q, 3-step shuffle reduction
//   2. running max / denominator update per latent, decode softmax over the M latents (block reductions)
//   3. stream u: u' = gamma u + eta v,  y += (softmax / d') u'; thread-private y columns, reduced once
#include "decode_step.cuh"

namespace flare {

namespace {

constexpr int NT = 256;
constexpr int NW = NT / 32;

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < NW; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
  return r;
}

// scores of all M latents against one token vector held in shared memory (fp32)
__device__ __forceinline__ void lane_scores(float* out, const float* tok, const void* lat, int dtype, int64_t lat_off,
                                            int64_t lat_stride_m, int M, int Dk, float scale) {
  const int grp = threadIdx.x >> 3, gl = threadIdx.x & 7;
  for (int m = grp; m < M; m += NT / 8) {
    float acc = 0.f;
    const int64_t row = lat_off + (int64_t)m * lat_stride_m;
    for (int d0 = gl * 8; d0 < Dk; d0 += 64) {
      float qv[8];
      load8(lat, dtype, row + d0, qv);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += qv[i] * tok[d0 + i];
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    if (gl == 0) out[m] = acc * scale;
  }
}

}  // namespace

// PRE: state vectors per thread issued before the score phase; UNR: state vectors in flight per thread in the
// streaming loop; MINB: CTAs per SM the register budget is held to
template <int PRE, int UNR, int MINB>
__global__ void __launch_bounds__(NT, MINB) decode_step_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) float smem[];
  const int lane_id = blockIdx.x;
  const int b = lane_id / p.H, h = lane_id % p.H;
  const int M = p.M, Dk = p.Dk, Dv = p.Dv;
  const int tid = threadIdx.x;
  const int dtype = p.dtype;
  const int dv4 = Dv >> 2;
  const int rows_per_pass = NT / dv4;
  const int col4 = tid % dv4, row0 = tid / dv4;

  float* s_sc = smem;           // [M] encode scores -> eta
  float* a_sc = s_sc + M;       // [M] decode scores -> read-out weight
  float* gam = a_sc + M;        // [M]
  float* ktok = gam + M;        // [Dk]
  float* qtok = ktok + Dk;      // [Dk]
  float* vtok = qtok + Dk;      // [Dv]
  float* red = vtok + Dv;       // [NW]
  float4* ypart = reinterpret_cast<float4*>(red + NW);  // [NT]

  if (p.mask != nullptr && p.mask[b] == 0) {
    // masked lane: state untouched, y = 0
    for (int i = tid; i < Dv; i += NT) store1(p.y, dtype, (int64_t)lane_id * Dv + i, 0.f);
    return;
  }

  float4* u4 = reinterpret_cast<float4*>(p.u + (int64_t)lane_id * M * Dv);
  const int total4 = M * dv4;

  // phase 0: first state vectors in flight
  float4 pre[PRE];
#pragma unroll
  for (int i = 0; i < PRE; ++i) {
    const int idx = tid + i * NT;
    pre[i] = idx < total4 ? __ldcs(u4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }

  // token vectors -> smem fp32
  for (int i = tid; i < Dk; i += NT) {
    ktok[i] = load1(p.k, dtype, (int64_t)b * p.k_stride_b + (int64_t)h * p.k_stride_h + i);
    if (p.qd != nullptr) qtok[i] = load1(p.qd, dtype, (int64_t)b * p.qd_stride_b + (int64_t)h * p.qd_stride_h + i);
  }
  for (int i = tid; i < Dv; i += NT) vtok[i] = load1(p.v, dtype, (int64_t)b * p.v_stride_b + (int64_t)h * p.v_stride_h + i);
  __syncthreads();

  // phase 1: scores
  lane_scores(s_sc, ktok, p.q, dtype, (int64_t)h * p.q_stride_h, p.q_stride_m, M, Dk, p.scale);
  const bool shared_w = p.qd == nullptr && p.kd == nullptr;
  if (!shared_w) {
    lane_scores(a_sc, p.qd ? qtok : ktok, p.kd ? p.kd : p.q, dtype,
                p.kd ? (int64_t)h * p.kd_stride_h : (int64_t)h * p.q_stride_h, p.kd ? p.kd_stride_m : p.q_stride_m, M,
                Dk, p.scale);
  }
  __syncthreads();

  // phase 2: decode softmax over latents and per-latent statistics
  float amax = kNegInf;
  for (int m = tid; m < M; m += NT) amax = fmaxf(amax, shared_w ? s_sc[m] : a_sc[m]);
  amax = block_reduce(amax, red, true);
  float asum = 0.f;
  for (int m = tid; m < M; m += NT) {
    const float e = __expf((shared_w ? s_sc[m] : a_sc[m]) - amax);
    a_sc[m] = e;
    asum += e;
  }
  asum = block_reduce(asum, red, false);
  const float ainv = 1.0f / asum;
  float* gm = p.m + (int64_t)lane_id * M;
  float* gd = p.d + (int64_t)lane_id * M;
  for (int m = tid; m < M; m += NT) {
    const float s = s_sc[m];
    const float mo = gm[m], dold = gd[m];
    const float mn = fmaxf(mo, s);
    const float g = (mo == kNegInf) ? 0.f : __expf(mo - mn);
    const float eta = __expf(s - mn);
    const float dn = dold * g + eta;
    gm[m] = mn;
    gd[m] = dn;
    gam[m] = g;
    s_sc[m] = eta;
    a_sc[m] = a_sc[m] * ainv / (dn > 0.f ? dn : 1.f);
  }
  __syncthreads();

  // phase 3: stream the state
  const float4 v4 = reinterpret_cast<const float4*>(vtok)[col4];
  float4 yacc = make_float4(0.f, 0.f, 0.f, 0.f);
  auto apply = [&](float4 x, int row, int idx) {
    const float g = gam[row], e = s_sc[row], w = a_sc[row];
    x.x = x.x * g + e * v4.x;
    x.y = x.y * g + e * v4.y;
    x.z = x.z * g + e * v4.z;
    x.w = x.w * g + e * v4.w;
    __stcs(u4 + idx, x);
    yacc.x += w * x.x;
    yacc.y += w * x.y;
    yacc.z += w * x.z;
    yacc.w += w * x.w;
  };
#pragma unroll
  for (int i = 0; i < PRE; ++i) {
    const int idx = tid + i * NT;
    if (idx < total4) apply(pre[i], row0 + i * rows_per_pass, idx);
  }
  int base = PRE * NT;
  for (; base + UNR * NT <= total4; base += UNR * NT) {
    float4 x[UNR];
#pragma unroll
    for (int i = 0; i < UNR; ++i) x[i] = __ldcs(u4 + base + tid + i * NT);
#pragma unroll
    for (int i = 0; i < UNR; ++i) apply(x[i], (base + tid + i * NT) / dv4, base + tid + i * NT);
  }
  for (; base < total4; base += NT) {
    const int idx = base + tid;
    if (idx < total4) apply(__ldcs(u4 + idx), idx / dv4, idx);
  }

  // reduce y over the row groups that share a column
  ypart[tid] = yacc;
  __syncthreads();
  if (tid < dv4) {
    float4 acc = ypart[tid];
    for (int r = 1; r < rows_per_pass; ++r) {
      const float4 x = ypart[tid + r * dv4];
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    store4(p.y, dtype, (int64_t)lane_id * Dv + tid * 4, acc.x, acc.y, acc.z, acc.w);
  }
}

bool decode_step_supported(int M, int Dk, int Dv) {
  const int dv4 = Dv / 4;
  if (dv4 > NT || (NT % dv4) != 0) return false;
  const size_t smem = (size_t)(3 * M + 2 * Dk + Dv + NW) * 4 + NT * 16;
  return smem <= 200 * 1024;
}

template <int PRE, int UNR, int MINB>
static int launch_variant(const DecodeParams& p, size_t smem, cudaStream_t stream) {
  auto kern = decode_step_kernel<PRE, UNR, MINB>;
  if (smem > 48 * 1024) FLARE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  LaunchTimer timer("decode_step_kernel", stream);
  kern<<<p.B * p.H, NT, smem, stream>>>(p);
  FLARE_CUDA_CHECK(cudaGetLastError());
  return FLARE_OK;
}

int launch_decode_step(const DecodeParams& p, cudaStream_t stream) {
  const size_t smem = (size_t)(3 * p.M + 2 * p.Dk + p.Dv + NW) * 4 + NT * 16;
  // Measured on B200 at B=64, H=32, M=256, D=128 (us per step): <2,4,8> 112.0, <8,8,4> 113.8, <4,8,4> 115.6,
  // <4,4,6> 116.8, <4,8,1> 141.9, <4,16,2> 157.8: occupancy (8 CTAs of 32 registers per SM) beats deeper unrolling.
  // Also measured and rejected: 128-thread CTAs at 16 per SM (121.7), and moving the state with bulk async copies
  // through a shared-memory ring (4 x 8 KB: 115.5, 4 x 16 KB: 131.3, 8 x 16 KB: 207.2) - the per-lane score and
  // softmax phases are hidden best by many resident CTAs, not by more bytes in flight per CTA.
  return launch_variant<2, 4, 8>(p, smem, stream);
}

}  // namespace flare
