// Tensor-core (tcgen05 + TMEM + TMA) backward of causal FLARE, bf16 operands, fp32 accumulation and statistics.
// Shape class: the one of the tensor-core forward (prefill_tc.cu) with shared decode weights: softmax encoder token-
// or block-causal (blocks of 16 / 32 / 64 / 128), stablemax encoder token-causal; (Dk, Dv) = (64, 64), (128, 128),
// (64, 128); M a multiple of 16, up to 256 (Dk = 128) or 512 (Dk = 64).
//
// Per (batch, head) lane, chunks of C = 128 tokens are walked from the last to the first.  The forward kernel has
// left, per chunk i, the frame c_i[m] (log2 units), the encoder denominator d_i[m] and the numerator U_i[m, :] (bf16)
// of the state BEFORE the chunk, and per token the decode log-sum-exp L_t; delta_t = <dY_t, y_t>.  With
//   E[m,t] = exp2(s2[m,t] - c_i[m])   (stablemax: sigma(s))        D[m,t] = d_i[m] + sum_{tau <= t} E[m,tau]
//   g[m,t] = exp2(s2[m,t] - L_t)      decode softmax               R[m,t] = g / D
//   A[tau,t] = <v_tau, dY_t>,  vis(tau, t) = tau <= t  (block-causal: tau <= end of the block of t; D at block ends)
// and the reverse carries G[m,:] = sum_{t in later chunks} R dY_t, Cc[m] = sum_{t later} R p (both in the frame c_i):
//   P    = U_i dY^T + E (A . vis)                          p = P / D = <z_t[m], dY_t>
//   X    = G V^T   + R (A . vis)^T
//   dS   = R (P - D delta_t)  +  E slope (X - Cc - sum_{t' >= t} R p)          slope = 1 | sigma'/sigma
//   dV   = E^T G + (E^T R . vis) dY
//   G   += R dY,  Cc += sum_t R p,  then both are rescaled by exp2(c_{i-1} - c_i) for the next chunk.
// dS is written per token as a hi and a lo bf16 row over the latents ([lane][t][2][m], dS = hi + lo, every warp store
// one contiguous segment); a second tensor-core kernel forms dK = scale dS^T Q per chunk and
// dQ = scale sum_t dS K per (lane, split) (fp32 partials, summed in fixed order: no atomics, deterministic).
//
// Main kernel, one CTA per (lane, group of 128 latents), 14 warps: 0-7 latent group (thread = latent = TMEM lane,
// the two warps of a lane quarter take 64 tokens each), 8-11 token group (thread = token = TMEM lane: causal masks of
// A and E^T R, dV store), 12 MMA issuer, 13 TMA producer.  Ten MMAs per chunk; every operand that the latent / token
// threads produce (E, R, masked A, G as bf16) is written once into a 128-byte-swizzled buffer and read K-major or
// MN-major as the product needs, so there is no transposition pass.
#include "bwd_tc.cuh"

#include <cuda.h>
#include <string.h>

#include "bwd_exact.cuh"
#include "prefill_tc.cuh"
#include "sm100_ptx.cuh"
#include "tc_device.cuh"

namespace flare {

using namespace sm100;
using tc::bf16_hi;
using tc::bf16_lo;
using tc::kmaj_step;
using tc::mnmaj_step;
using tc::sigma_fast;
using tc::swz_chunk_off;
using tc::warp_arrive;

struct BwdTcParams {
  const void* q;  // bf16 latent bank [H, M, Dk]
  int64_t q_stride_h, q_stride_m;
  int N, H, M;  // M: all latents
  int nch;      // chunks of 128 tokens per lane
  int npad;     // nch * 128
  int block;    // 1 or 16 / 32 / 64 / 128
  float scale, power;
  const float *chunk_c, *chunk_d;  // [lanes][nch][M]
  const float *tok_l2, *tok_delta;  // [lanes][npad]
  void* ds;      // bf16 [lanes][npad][2][M]: dS of every token as a hi row and a lo row over the latents (dS = hi + lo)
  void* dv;      // bf16 [B, N, H, Dv] contiguous, or (more than one latent group) bf16 [groups][B][N][H][Dv]
  int groups;
  int* gate;  // per-call gate word (may be null): raised when a carry turns non-finite (inputs outside the numeric domain)
  int* err;
  long long* trace;  // optional diagnostic cycle stamps of CTA (0, 0), see BT_TRACE; null in normal use
};

struct GradTcParams {
  int N, H, M, B;
  int nch, npad, groups;
  int nsplit, chunks_per_split;
  float scale;
  void* dk;        // bf16 [B, N, H, Dk] contiguous
  float* dq_part;  // fp32 [B * nsplit][H][M][Dk]
  int* err;
};

// one instance family per head-width combination, compiled in its own translation unit
template <int UNIT>
int launch_bwd_tc_unit(int mode, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdy, const CUtensorMap& tu,
                       const BwdTcParams& p, dim3 grid, cudaStream_t stream);

namespace {

constexpr int C = 128;
constexpr int LW = 4;                           // latent warps per lane quarter
constexpr int TOK = C / LW;                     // tokens per latent thread
constexpr int NT_MAIN = (4 * LW + 4 + 2) * 32;  // latent warps, token warps, MMA issuer, TMA producer
constexpr int W_TOKEN = 4 * LW, W_MMA = 4 * LW + 4, W_TMA = 4 * LW + 5;  // first token warp, issuer, producer
constexpr float kLog2e = 1.4426950408889634f;

// shared memory map of the main kernel (bytes; every operand buffer 1024-aligned for the 128B swizzle)
template <int DVB>
struct BL {
  static constexpr int OFF_KA = 0;                      // K tile [DKB][128 t][64]; later the masked A [2][128 tau][64 t]
  static constexpr int OFF_V = 32768;                   // [DVB][128 t][64]
  static constexpr int OFF_DY = OFF_V + DVB * 16384;    // [DVB][128 t][64]
  static constexpr int OFF_UR = OFF_DY + DVB * 16384;   // U_i [DVB][128 m][64] (the 32 KB slot keeps every buffer behind it 1024-aligned for both widths)
  static constexpr int OFF_GC = OFF_UR + 32768;         // G as bf16 [DVB][128 m][64]
  static constexpr int OFF_E = OFF_GC + DVB * 16384;    // [2 t-blocks][128 m][64 t]
  static constexpr int OFF_R = OFF_E + 32768;
  static constexpr int OFF_MISC = OFF_R + 32768;
  static constexpr int SMEM_BYTES = OFF_MISC + 3072;  // Misc + what the manual 1024-byte alignment may cost
  static_assert(SMEM_BYTES <= 232448, "shared memory");
};
// tensor-memory columns: T0 / T1 transient accumulators, T2 the masked E^T R as bf16 (A operand), TQ the latent bank
// as packed bf16 (A operand of the score product), TG the carry G (fp32)
constexpr uint32_t T0 = 0, T1 = 128, T2 = 256, TQ = 320, TG = 384, TM_COLS = 512;

struct Misc {
  uint64_t k_full, v_full, dy_full, u_full, q_ready;
  uint64_t s_ready, a_ready, px_ready, g_ready, wt_ready, dv_ready;
  uint64_t er_done, am_done, p_free, x_done, wm_done, dv_free, gc_done;
  uint64_t psum[4], prp[4];
  uint32_t tmem_base;
  volatile int abort_flag;
  float xch[LW][128];  // exchange between the token quarters of a latent row: sums of E, then sums of R p
};
static_assert(sizeof(Misc) <= 2560, "Misc must leave room for the alignment slack");

// waits between roles are long (thousands of cycles): one quick look, then suspend
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, Misc* misc) {
  return tc::wait_or_abort(bar, parity, &misc->abort_flag, 1);
}
// exchange between the four warps of a lane quarter, which run in step: poll
__device__ __forceinline__ bool wait_partner(uint64_t* bar, uint32_t parity, Misc* misc) {
  return tc::wait_or_abort(bar, parity, &misc->abort_flag, 48);
}

// optional cycle trace of CTA (0, 0): [role < 4][chunk step < 8][slot < 8] clock64 stamps (diagnostic hook)
#define BT_TRACE(role, step, slot)                                                             \
  do {                                                                                         \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (step) < 8)                \
      p.trace[((role) * 8 + (step)) * 8 + (slot)] = clock64();                                 \
  } while (0)

__device__ __forceinline__ float unpack8(const uint4& v, int j) {
  const uint32_t w = j < 2 ? v.x : (j < 4 ? v.y : (j < 6 ? v.z : v.w));
  return (j & 1) ? bf16_hi(w) : bf16_lo(w);
}
// slope sigma'(s) / sigma(s) = p / (1 + |s|) recovered from the (rounded) weight: 1 + |s| = E^(1/p) for s >= 0
// (E >= 1) and E^(-1/p) for s < 0
__device__ __forceinline__ float slope_from_sigma(float e, float p) {
  const float l = __log2f(e) * (1.0f / p);
  return p * ex2_approx(e >= 1.0f ? -l : l);
}

}  // namespace

#ifdef FLARE_BT_UNIT

// MODE 0: softmax encoder, token-causal; 1: block-causal read-out; 2: stablemax encoder, token-causal
template <int DKB, int DVB, int MODE>
__global__ void __launch_bounds__(NT_MAIN, 1)
bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
              const __grid_constant__ CUtensorMap tm_dy, const __grid_constant__ CUtensorMap tm_u, const BwdTcParams p) {
  using L = BL<DVB>;
  constexpr bool BLOCK = MODE == 1, STABLE = MODE == 2;
  constexpr int DV = DVB * 64;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + L::OFF_MISC);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lane_id = blockIdx.x, group = blockIdx.y;
  const int b = lane_id / p.H, h = lane_id % p.H;
  const int nch = p.nch;
  if ((int)(smem - smem_dyn) + L::OFF_MISC + (int)sizeof(Misc) > L::SMEM_BYTES) {
    // the dynamic shared memory window starts less aligned than this layout can absorb: report, do nothing
    if (tid == 0) atomicOr(p.err, 1);
    return;
  }

  if (tid == 0) {
    mbar_init(&misc->k_full, 1);
    mbar_init(&misc->v_full, 1);
    mbar_init(&misc->dy_full, 1);
    mbar_init(&misc->u_full, 1);
    mbar_init(&misc->q_ready, 4 * LW);
    mbar_init(&misc->s_ready, 1);
    mbar_init(&misc->a_ready, 1);
    mbar_init(&misc->px_ready, 1);
    mbar_init(&misc->g_ready, 1);
    mbar_init(&misc->wt_ready, 1);
    mbar_init(&misc->dv_ready, 1);
    mbar_init(&misc->er_done, 4 * LW);
    mbar_init(&misc->am_done, 4);
    mbar_init(&misc->p_free, 4 * LW);
    mbar_init(&misc->x_done, 4 * LW);
    mbar_init(&misc->wm_done, 4);
    mbar_init(&misc->dv_free, 4);
    mbar_init(&misc->gc_done, 4 * LW);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&misc->psum[i], LW);
      mbar_init(&misc->prp[i], LW);
    }
    misc->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == W_MMA) {
    tmem_alloc(&misc->tmem_base, TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = misc->tmem_base;
  bool ok = true;
  const int rows_here = min(128, p.M - group * 128);  // latents of this group
  const int ksm = (rows_here + 15) >> 4;              // 16-latent steps of a contraction over the latents

  if (warp == W_TMA) {
    // ======================================= TMA producer =======================================
    if (lane == 0) {
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      prefetch_tensormap(&tm_dy);
      prefetch_tensormap(&tm_u);
      for (int j = 0; ok && j < nch; ++j) {
        const int i = nch - 1 - j, t0 = i * C;
        const uint32_t pp = (j - 1) & 1;
        // K, V: free once the previous chunk's P / X products (which read the masked A and V) have run
        if (j > 0 && !(ok = wait_or_abort(&misc->px_ready, pp, misc))) break;
        mbar_arrive_expect_tx(&misc->k_full, DKB * 16384);
#pragma unroll
        for (int kb = 0; kb < DKB; ++kb) tma_load_4d(smem + L::OFF_KA + kb * 16384, &tm_k, &misc->k_full, kb * 64, h, t0, b);
        mbar_arrive_expect_tx(&misc->v_full, DVB * 16384);
#pragma unroll
        for (int vb = 0; vb < DVB; ++vb) tma_load_4d(smem + L::OFF_V + vb * 16384, &tm_v, &misc->v_full, vb * 64, h, t0, b);
        // U_i: read by the previous chunk's P product (which has run: px_ready above)
        mbar_arrive_expect_tx(&misc->u_full, DVB * 16384);
#pragma unroll
        for (int vb = 0; vb < DVB; ++vb)
          tma_load_4d(smem + L::OFF_UR + vb * 16384, &tm_u, &misc->u_full, vb * 64, group * 128, i, lane_id);
        // dY: read by the previous chunk's dV and G products
        if (j > 0 && !(ok = wait_or_abort(&misc->dv_ready, pp, misc))) break;
        mbar_arrive_expect_tx(&misc->dy_full, DVB * 16384);
#pragma unroll
        for (int vb = 0; vb < DVB; ++vb) tma_load_4d(smem + L::OFF_DY + vb * 16384, &tm_dy, &misc->dy_full, vb * 64, h, t0, b);
      }
    }
  } else if (warp == W_MMA) {
    // ======================================= MMA issuer =======================================
    if (lane == 0) {
      // All operands are bf16: tcgen05.mma kind::f16 wants A and B in ONE format (a descriptor that mixes fp16 and
      // bf16 operands is rejected by the hardware as an illegal instruction), and everything that scales with the
      // caller's data (V, dY, U, G, the masked A, R) needs the bf16 range.
      constexpr uint32_t ID_SS = make_idesc_bf16(128, 128, 0, 0);   // K-major x K-major (scores, A, U dY^T, G V^T, R A^T)
      constexpr uint32_t ID_PE = make_idesc_bf16(128, 128, 0, 1);   // E (K-major) x masked A (MN-major)
      constexpr uint32_t ID_WT = make_idesc_bf16(128, 128, 1, 1);   // E (MN-major) x R (MN-major)
      constexpr uint32_t ID_DV1 = make_idesc_bf16(128, DV, 1, 1);   // E (MN-major) x G (MN-major)
      constexpr uint32_t ID_DV2 = make_idesc_bf16(128, DV, 0, 1);   // masked E^T R (TMEM) x dY (MN-major)
      constexpr uint32_t ID_G = make_idesc_bf16(128, DV, 0, 1);     // R (K-major) x dY (MN-major)
      const uint64_t d_k = make_desc_sw128(smem_u32(smem + L::OFF_KA), 16, 1024);        // K tile, K-major
      const uint64_t d_am_k = d_k;                                                        // masked A, K-major (N = tau)
      const uint64_t d_am_mn = make_desc_sw128(smem_u32(smem + L::OFF_KA), 16384, 1024);  // masked A, MN-major (N = t)
      const uint64_t d_v_k = make_desc_sw128(smem_u32(smem + L::OFF_V), 16, 1024);
      const uint64_t d_dy_k = make_desc_sw128(smem_u32(smem + L::OFF_DY), 16, 1024);
      const uint64_t d_dy_mn = make_desc_sw128(smem_u32(smem + L::OFF_DY), 16384, 1024);
      const uint64_t d_u_k = make_desc_sw128(smem_u32(smem + L::OFF_UR), 16, 1024);
      const uint64_t d_g_k = make_desc_sw128(smem_u32(smem + L::OFF_GC), 16, 1024);
      const uint64_t d_g_mn = make_desc_sw128(smem_u32(smem + L::OFF_GC), 16384, 1024);
      const uint64_t d_e_k = make_desc_sw128(smem_u32(smem + L::OFF_E), 16, 1024);
      const uint64_t d_e_mn = make_desc_sw128(smem_u32(smem + L::OFF_E), 16384, 1024);
      const uint64_t d_r_k = make_desc_sw128(smem_u32(smem + L::OFF_R), 16, 1024);
      const uint64_t d_r_mn = make_desc_sw128(smem_u32(smem + L::OFF_R), 16384, 1024);

      ok = wait_or_abort(&misc->q_ready, 0, misc);  // the latent bank is in tensor memory
      tc_fence_after_sync();
      for (int j = 0; ok && j < nch; ++j) {
        const uint32_t par = j & 1, pp = (j - 1) & 1;
        // scores S^T = Q K^T -> T1 (the previous chunk's X has been read)
        if (!(ok = wait_or_abort(&misc->k_full, par, misc))) break;
        if (j > 0 && !(ok = wait_or_abort(&misc->x_done, pp, misc))) break;
        tc_fence_after_sync();
        BT_TRACE(2, j, 0);
#pragma unroll
        for (int s = 0; s < 4 * DKB; ++s) mma_ts(tmem + T1, tmem + TQ + s * 8, kmaj_step(d_k, s), ID_SS, s > 0);
        tc_commit(&misc->s_ready);
        // A = V dY^T -> T0 (the previous chunk's dV has been stored)
        if (!(ok = wait_or_abort(&misc->v_full, par, misc))) break;
        if (!(ok = wait_or_abort(&misc->dy_full, par, misc))) break;
        if (j > 0 && !(ok = wait_or_abort(&misc->dv_free, pp, misc))) break;
        tc_fence_after_sync();
        BT_TRACE(2, j, 1);
#pragma unroll
        for (int s = 0; s < 4 * DVB; ++s) mma_ss(tmem + T0, kmaj_step(d_v_k, s), kmaj_step(d_dy_k, s), ID_SS, s > 0);
        tc_commit(&misc->a_ready);
        // P -> T0, X -> T1, then G += R dY
        if (!(ok = wait_or_abort(&misc->er_done, par, misc))) break;
        if (!(ok = wait_or_abort(&misc->am_done, par, misc))) break;
        if (!(ok = wait_or_abort(&misc->u_full, par, misc))) break;
        if (j > 0 && !(ok = wait_or_abort(&misc->gc_done, pp, misc))) break;
        tc_fence_after_sync();
        BT_TRACE(2, j, 2);
#pragma unroll
        for (int s = 0; s < 4 * DVB; ++s) mma_ss(tmem + T0, kmaj_step(d_u_k, s), kmaj_step(d_dy_k, s), ID_SS, s > 0);
#pragma unroll
        for (int s = 0; s < 8; ++s) mma_ss(tmem + T0, kmaj_step(d_e_k, s), mnmaj_step(d_am_mn, s), ID_PE, 1);
        if (j > 0) {
#pragma unroll
          for (int s = 0; s < 4 * DVB; ++s) mma_ss(tmem + T1, kmaj_step(d_g_k, s), kmaj_step(d_v_k, s), ID_SS, s > 0);
        }
#pragma unroll
        for (int s = 0; s < 8; ++s) mma_ss(tmem + T1, kmaj_step(d_r_k, s), kmaj_step(d_am_k, s), ID_SS, (j > 0 || s > 0) ? 1u : 0u);
        tc_commit(&misc->px_ready);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          mma_ss(tmem + TG, kmaj_step(d_r_k, s), mnmaj_step(d_dy_mn, s), ID_G, (j > 0 || s > 0) ? 1u : 0u);
        tc_commit(&misc->g_ready);
        // W^T = E^T R -> T0 (P has been read)
        if (!(ok = wait_or_abort(&misc->p_free, par, misc))) break;
        tc_fence_after_sync();
        BT_TRACE(2, j, 3);
        for (int s = 0; s < ksm; ++s) mma_ss(tmem + T0, mnmaj_step(d_e_mn, s), mnmaj_step(d_r_mn, s), ID_WT, s > 0);
        tc_commit(&misc->wt_ready);
        // dV = E^T G + (masked W^T) dY -> T0
        if (!(ok = wait_or_abort(&misc->wm_done, par, misc))) break;
        tc_fence_after_sync();
        BT_TRACE(2, j, 4);
        if (j > 0)
          for (int s = 0; s < ksm; ++s) mma_ss(tmem + T0, mnmaj_step(d_e_mn, s), mnmaj_step(d_g_mn, s), ID_DV1, s > 0);
#pragma unroll
        for (int s = 0; s < 8; ++s) mma_ts(tmem + T0, tmem + T2 + s * 8, mnmaj_step(d_dy_mn, s), ID_DV2, (j > 0 || s > 0) ? 1u : 0u);
        tc_commit(&misc->dv_ready);
      }
    }
  } else if (warp < 4 * LW) {
    // ======== latent group: thread = (latent = TMEM lane, quarter of the chunk's tokens); 4 warps per lane quarter ========
    const int tq = warp >> 2, q = warp & 3;
    const uint32_t tl = tmem + ((uint32_t)(q * 32) << 16);
    const int m = q * 32 + lane;
    const int mg = group * 128 + m;
    const bool live = mg < p.M;
    const float sc2 = p.scale * kLog2e;
    const int tok0 = tq * TOK;
    // this thread's 32 tokens are 16-byte chunks ch0 .. ch0 + 3 of row m in t-block tq / 2 of the [2][128][64] buffers
    const int ch0 = (tq & 1) * 4;
    uint8_t* const e_row = smem + L::OFF_E + (tq >> 1) * 16384;
    uint8_t* const r_row = smem + L::OFF_R + (tq >> 1) * 16384;
    {
      // latent bank row -> tensor memory as packed bf16 (element k in column k / 2); each warp of the quarter writes
      // 32 elements of the row (Dk = 64: the first two warps)
      if (tq * 32 < DKB * 64) {
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)h * p.q_stride_h +
                                                          (int64_t)(live ? mg : 0) * p.q_stride_m + tq * 32);
        uint32_t r[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 x = live ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
          r[4 * i] = x.x; r[4 * i + 1] = x.y; r[4 * i + 2] = x.z; r[4 * i + 3] = x.w;
        }
        tmem_st16(tl + TQ + tq * 16, r);
        tmem_wait_st();
      }
      tc_fence_before_sync();
      warp_arrive(&misc->q_ready, lane);
    }
    float cc_carry = 0.f;  // Cc: sum over later chunks of R p, in the current chunk's frame
    const int64_t stat0 = (int64_t)lane_id * nch * p.M + mg;
    // dS rows of this lane: element (token t, part, latent) at (t * 2 + part) * M + latent; a warp's 32 latents are
    // contiguous, so every store instruction of a warp writes one 64-byte segment
    __nv_bfloat16* const ds_col = reinterpret_cast<__nv_bfloat16*>(p.ds) + (int64_t)lane_id * p.npad * 2 * p.M + (live ? mg : 0);
    // value columns of G this warp rescales and repacks: a quarter of them
    constexpr int GCOLS = DVB * 16;
    const int gcol = tq * GCOLS;
    uint8_t* const g_dst = smem + L::OFF_GC + (gcol >> 6) * 16384;
    const int gch0 = (gcol & 63) >> 3;

    if (!__any_sync(0xffffffffu, live)) {
      // A warp whose 32 latents all lie beyond M (M <= 96, or the ragged last group): its operand rows are zero for
      // the whole kernel and it only keeps the barrier phases in step with the working warps.
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        *reinterpret_cast<uint4*>(e_row + swz_chunk_off(m, ch0 + ch)) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(r_row + swz_chunk_off(m, ch0 + ch)) = make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int ch = 0; ch < GCOLS / 8; ++ch)
        *reinterpret_cast<uint4*>(g_dst + swz_chunk_off(m, gch0 + ch)) = make_uint4(0, 0, 0, 0);
      fence_proxy_async_smem();
      for (int j = 0; ok && j < nch; ++j) {
        const uint32_t par = j & 1, pp = (j - 1) & 1;
        if (j > 0 && !(ok = wait_or_abort(&misc->dv_ready, pp, misc))) break;
        if (!(ok = wait_or_abort(&misc->s_ready, par, misc))) break;
        warp_arrive(&misc->er_done, lane);
        if (!(ok = wait_or_abort(&misc->px_ready, par, misc))) break;
        warp_arrive(&misc->p_free, lane);
        warp_arrive(&misc->x_done, lane);
        if (j + 1 < nch) {
          if (!(ok = wait_or_abort(&misc->dv_ready, par, misc))) break;
          warp_arrive(&misc->gc_done, lane);
        }
      }
    } else {
      // Per-chunk statistics of this thread's latent and per-token statistics of this warp's 32 tokens (lane l keeps
      // token tok0 + l; the loops broadcast them with shuffles), all fetched one chunk ahead so that the global-memory
      // latency never sits between two phases.
      const float* const l2_row = p.tok_l2 + (int64_t)lane_id * p.npad + tok0 + lane;
      const float* const dl_row = p.tok_delta + (int64_t)lane_id * p.npad + tok0 + lane;
      float c_cur = (live && !STABLE) ? __ldg(p.chunk_c + stat0 + (int64_t)(nch - 1) * p.M) : 0.f;
      float d_cur = live ? __ldg(p.chunk_d + stat0 + (int64_t)(nch - 1) * p.M) : 1.f;
      float c_nxt = (live && !STABLE && nch > 1) ? __ldg(p.chunk_c + stat0 + (int64_t)(nch - 2) * p.M) : c_cur;
      float l2_cur = __ldg(l2_row + (int64_t)(nch - 1) * C), dl_cur = __ldg(dl_row + (int64_t)(nch - 1) * C);

      for (int j = 0; ok && j < nch; ++j) {
        const int i = nch - 1 - j, t0 = i * C;
        const uint32_t par = j & 1, pp = (j - 1) & 1;
        const int nvalid = min(C, p.N - t0);
        const int lim = live ? nvalid - tok0 : 0;  // tokens of this thread's quarter that exist (may be <= 0)
        const bool fast = __all_sync(0xffffffffu, lim >= TOK);
        const float c_i = c_cur, d_i = d_cur;
        const float c_prev = i > 0 ? c_nxt : c_i;
        const float l2_mine = l2_cur, dl_mine = dl_cur;
        // the next chunk's (i - 1) values, used one iteration from now
        if (tid == 0) BT_TRACE(3, j, 0);
        const float d_pre = (live && i > 0) ? ldg_pinned(p.chunk_d + stat0 + (int64_t)(i - 1) * p.M) : 1.f;
        const float c_pre = (live && !STABLE && i > 1) ? ldg_pinned(p.chunk_c + stat0 + (int64_t)(i - 2) * p.M) : c_nxt;
        const float l2_pre = i > 0 ? ldg_pinned(l2_row + (int64_t)(i - 1) * C) : 0.f;
        const float dl_pre = i > 0 ? ldg_pinned(dl_row + (int64_t)(i - 1) * C) : 0.f;
        // E / R buffers: the previous chunk's products have read them
        if (j > 0 && !(ok = wait_or_abort(&misc->dv_ready, pp, misc))) break;
        if (!(ok = wait_or_abort(&misc->s_ready, par, misc))) break;
        tc_fence_after_sync();
        if (tid == 0) BT_TRACE(0, j, 0);
        uint32_t rs[32];  // the 32 raw scores of this thread
        tmem_ld32(tl + T1 + tok0, rs);
        tmem_wait_ld();
        tmem_fence_regs(rs);
        if (tid == 0) BT_TRACE(3, j, 1);
        // ---- phase 1a: E rows (bf16) and their sums
        float g16[2] = {0.f, 0.f};  // sums of the rounded E per 16 tokens
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          float e[8];
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const int k = ch * 8 + jj;
            const float sv = __uint_as_float(rs[k]);
            float x = STABLE ? sigma_fast(sv * p.scale, p.power) : ex2_approx(fmaf(sv, sc2, -c_i));
            if (!fast) x = k < lim ? x : 0.f;
            e[jj] = x;
          }
          uint4 v;
          v.x = pack_bf16(e[0], e[1]); v.y = pack_bf16(e[2], e[3]); v.z = pack_bf16(e[4], e[5]); v.w = pack_bf16(e[6], e[7]);
          g16[ch >> 1] += (bf16_lo(v.x) + bf16_hi(v.x)) + (bf16_lo(v.y) + bf16_hi(v.y)) + (bf16_lo(v.z) + bf16_hi(v.z)) +
                          (bf16_lo(v.w) + bf16_hi(v.w));
          *reinterpret_cast<uint4*>(e_row + swz_chunk_off(m, ch0 + ch)) = v;
        }
        misc->xch[tq][m] = g16[0] + g16[1];
        warp_arrive(&misc->psum[q], lane);
        if (tid == 0) BT_TRACE(3, j, 2);
        if (!(ok = wait_partner(&misc->psum[q], par, misc))) break;
        if (tid == 0) BT_TRACE(3, j, 3);
        // denominator before this thread's first token
        float base_run = d_i;
#pragma unroll
        for (int t = 0; t < LW - 1; ++t) base_run += t < tq ? misc->xch[t][m] : 0.f;
        float dend[2], invg[2];  // block-causal: denominator at the end of the block of each 16-token group
        if constexpr (BLOCK) {
          const int bs = p.block;
          const float p0 = base_run + g16[0], p1 = p0 + g16[1];
          if (bs == 16) { dend[0] = p0; dend[1] = p1; }
          else if (bs == 32) { dend[0] = dend[1] = p1; }
          else {
            // blocks of 64 or 128 tokens end in a later quarter: add the quarters up to the block's last one
            const int last = bs == 64 ? (tq | 1) : LW - 1;
            float tot = p1;
#pragma unroll
            for (int t = 1; t < LW; ++t) tot += (t > tq && t <= last) ? misc->xch[t][m] : 0.f;
            dend[0] = dend[1] = tot;
          }
          invg[0] = rcp_approx(dend[0]);
          invg[1] = rcp_approx(dend[1]);
        }
        // ---- phase 1b: R = g / D rows (bf16)
        {
          float run = base_run;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            const uint4 ev = *reinterpret_cast<const uint4*>(e_row + swz_chunk_off(m, ch0 + ch));
            float r[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const int k = ch * 8 + jj;
              const float l2 = __shfl_sync(0xffffffffu, l2_mine, k);
              const float g = ex2_approx(fmaf(__uint_as_float(rs[k]), sc2, -l2));
              float inv;
              if constexpr (BLOCK) {
                inv = invg[ch >> 1];
              } else {
                run += unpack8(ev, jj);
                inv = rcp_approx(run);
              }
              float x = g * inv;
              if (!fast) x = k < lim ? x : 0.f;
              r[jj] = x;
            }
            *reinterpret_cast<uint4*>(r_row + swz_chunk_off(m, ch0 + ch)) =
                make_uint4(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]), pack_bf16(r[4], r[5]), pack_bf16(r[6], r[7]));
          }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        warp_arrive(&misc->er_done, lane);
        if (tid == 0) BT_TRACE(0, j, 1);

        // ---- phase 2a (ascending): p = P / D, R p, decode part of dS - everything stays in registers
        if (!(ok = wait_or_abort(&misc->px_ready, par, misc))) break;
        tc_fence_after_sync();
        if (tid == 0) BT_TRACE(0, j, 2);
        uint32_t pd[32];   // P accumulators of the 32 tokens, replaced in place by the decode-side dS (fp32)
        uint32_t rpk[16];  // R p, packed bf16 pairs
        float rg16[2] = {0.f, 0.f};  // sums of the rounded R p per 16 tokens
        tmem_ld32(tl + T0 + tok0, pd);
        tmem_wait_ld();
        tmem_fence_regs(pd);
        tc_fence_before_sync();
        warp_arrive(&misc->p_free, lane);  // T0 may take E^T R
        {
          float run = base_run;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            const uint4 ev = *reinterpret_cast<const uint4*>(e_row + swz_chunk_off(m, ch0 + ch));
            const uint4 rv = *reinterpret_cast<const uint4*>(r_row + swz_chunk_off(m, ch0 + ch));
            float rp[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const int k = ch * 8 + jj;
              const float pacc = __uint_as_float(pd[k]);
              const float rbv = unpack8(rv, jj);
              const float dl = __shfl_sync(0xffffffffu, dl_mine, k);
              float dcur, inv;
              if constexpr (BLOCK) {
                dcur = dend[ch >> 1];
                inv = invg[ch >> 1];
              } else {
                run += unpack8(ev, jj);
                dcur = run;
                inv = rcp_approx(run);
              }
              rp[jj] = rbv * (pacc * inv);
              pd[k] = __float_as_uint(rbv * fmaf(-dcur, dl, pacc));
            }
#pragma unroll
            for (int jj = 0; jj < 8; jj += 2) {
              const uint32_t w = pack_bf16(rp[jj], rp[jj + 1]);
              rpk[ch * 4 + (jj >> 1)] = w;
              rg16[ch >> 1] += bf16_lo(w) + bf16_hi(w);
            }
          }
        }
        if (tid == 0) BT_TRACE(0, j, 3);
        const float rp_mine = rg16[0] + rg16[1];
        misc->xch[tq][m] = rp_mine;
        warp_arrive(&misc->prp[q], lane);
        if (!(ok = wait_partner(&misc->prp[q], par, misc))) break;
        if (tid == 0) BT_TRACE(3, j, 4);
        float rp_later = 0.f, rp_all = 0.f;  // R p of the quarters after this one, and of the whole chunk
#pragma unroll
        for (int t = 0; t < LW; ++t) {
          const float x = misc->xch[t][m];
          rp_all += x;
          rp_later += t > tq ? x : 0.f;
        }

        // ---- phase 2b (descending): encoder part, dS rows to global memory as a hi + lo pair
        {
          float ccg[2];  // block-causal: Cc + sum of R p from the start of the group's block on
          float cc = cc_carry + rp_later;
          if constexpr (BLOCK) {
            const int bs = p.block;
            if (bs == 16) { ccg[1] = cc + rg16[1]; ccg[0] = ccg[1] + rg16[0]; }
            else if (bs == 32) { ccg[0] = ccg[1] = cc + rp_mine; }
            else {
              // the block starts in an earlier (or this) quarter: add the quarters from its first one on
              const int first = bs == 64 ? (tq & ~1) : 0;
              float tot = cc + rp_mine;
#pragma unroll
              for (int t = 0; t < LW - 1; ++t) tot += (t >= first && t < tq) ? misc->xch[t][m] : 0.f;
              ccg[0] = ccg[1] = tot;
            }
          }
          __nv_bfloat16* const dst = ds_col + (int64_t)(t0 + tok0) * 2 * p.M;
          const int64_t tstride = 2 * (int64_t)p.M;
#pragma unroll
          for (int blk = 1; blk >= 0; --blk) {
            uint32_t xr[16];
            tmem_ld16(tl + T1 + tok0 + blk * 16, xr);
            tmem_wait_ld();
            tmem_fence_regs16(xr);
#pragma unroll
            for (int c2 = 1; c2 >= 0; --c2) {
              const int ch = blk * 2 + c2;
              const uint4 ev = *reinterpret_cast<const uint4*>(e_row + swz_chunk_off(m, ch0 + ch));
              float ds[8];
#pragma unroll
              for (int jj = 7; jj >= 0; --jj) {
                const int k = ch * 8 + jj;
                const float x = __uint_as_float(xr[c2 * 8 + jj]);
                const float eb = unpack8(ev, jj);
                float csub;
                if constexpr (BLOCK) {
                  csub = ccg[ch >> 1];
                } else {
                  const uint32_t w = rpk[k >> 1];
                  cc += (k & 1) ? bf16_hi(w) : bf16_lo(w);
                  csub = cc;
                }
                float enc = eb * (x - csub);
                if constexpr (STABLE) enc *= slope_from_sigma(eb, p.power);
                ds[jj] = __uint_as_float(pd[k]) + ((STABLE && eb == 0.f) ? 0.f : enc);
              }
              // dS = hi + lo, two bf16 values: the dK / dQ products then see it with 16 mantissa bits
              if (live) {
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                  const __nv_bfloat16 hi = __float2bfloat16_rn(ds[jj]);
                  const __nv_bfloat16 lo = __float2bfloat16_rn(ds[jj] - __bfloat162float(hi));
                  __nv_bfloat16* d = dst + (int64_t)(ch * 8 + jj) * tstride;
                  d[0] = hi;
                  d[p.M] = lo;
                }
              }
            }
          }
        }
        if (tid == 0) BT_TRACE(3, j, 5);
        tc_fence_before_sync();
        warp_arrive(&misc->x_done, lane);
        if (tid == 0) BT_TRACE(0, j, 4);
        // carries into the previous chunk's frame
        const float phi = STABLE ? 1.0f : ex2_approx(c_prev - c_i);
        cc_carry = (cc_carry + rp_all) * phi;
        if (!(fabsf(cc_carry) < INFINITY)) {
          // an overflow or 0 / 0 upstream (score spreads beyond what these frames hold) has reached the carries: the
          // results of this call are invalid; the exact kernels standing by behind this pass redo it
          atomicOr(p.err, 2);
          if (p.gate != nullptr) p.gate[0] = 1;
        }
        if (i > 0) {
          // G has taken this chunk's R dY: rescale this warp's value columns in tensor memory and pack them as bf16.
          // The shared-memory copy is still read by this chunk's dV product, so the packed rows wait in registers
          // until that product has run.
          if (!(ok = wait_or_abort(&misc->g_ready, par, misc))) break;
          tc_fence_after_sync();
          if (tid == 0) BT_TRACE(0, j, 5);
          const bool need = __any_sync(0xffffffffu, phi != 1.0f);
          uint4 gv[GCOLS / 8];
          if constexpr (DVB == 2) {
            uint32_t r[32];
            tmem_ld32(tl + TG + gcol, r);
            tmem_wait_ld();
            tmem_fence_regs(r);
            if (need) {
#pragma unroll
              for (int k = 0; k < 32; ++k) r[k] = __float_as_uint(__uint_as_float(r[k]) * phi);
              tmem_st32(tl + TG + gcol, r);
            }
#pragma unroll
            for (int ch = 0; ch < 4; ++ch)
              gv[ch] = make_uint4(pack_bf16(__uint_as_float(r[ch * 8 + 0]), __uint_as_float(r[ch * 8 + 1])),
                                  pack_bf16(__uint_as_float(r[ch * 8 + 2]), __uint_as_float(r[ch * 8 + 3])),
                                  pack_bf16(__uint_as_float(r[ch * 8 + 4]), __uint_as_float(r[ch * 8 + 5])),
                                  pack_bf16(__uint_as_float(r[ch * 8 + 6]), __uint_as_float(r[ch * 8 + 7])));
          } else {
            uint32_t r[16];
            tmem_ld16(tl + TG + gcol, r);
            tmem_wait_ld();
            tmem_fence_regs16(r);
            if (need) {
#pragma unroll
              for (int k = 0; k < 16; ++k) r[k] = __float_as_uint(__uint_as_float(r[k]) * phi);
              tmem_st16(tl + TG + gcol, r);
            }
#pragma unroll
            for (int ch = 0; ch < 2; ++ch)
              gv[ch] = make_uint4(pack_bf16(__uint_as_float(r[ch * 8 + 0]), __uint_as_float(r[ch * 8 + 1])),
                                  pack_bf16(__uint_as_float(r[ch * 8 + 2]), __uint_as_float(r[ch * 8 + 3])),
                                  pack_bf16(__uint_as_float(r[ch * 8 + 4]), __uint_as_float(r[ch * 8 + 5])),
                                  pack_bf16(__uint_as_float(r[ch * 8 + 6]), __uint_as_float(r[ch * 8 + 7])));
          }
          if (need) tmem_wait_st();
          if (tid == 0) BT_TRACE(3, j, 6);
          if (!(ok = wait_or_abort(&misc->dv_ready, par, misc))) break;
          if (tid == 0) BT_TRACE(0, j, 6);
#pragma unroll
          for (int ch = 0; ch < GCOLS / 8; ++ch) *reinterpret_cast<uint4*>(g_dst + swz_chunk_off(m, gch0 + ch)) = gv[ch];
          fence_proxy_async_smem();
          tc_fence_before_sync();
          warp_arrive(&misc->gc_done, lane);
          if (tid == 0) BT_TRACE(0, j, 7);
        }
        c_cur = c_prev;
        d_cur = d_pre;
        c_nxt = c_pre;
        l2_cur = l2_pre;
        dl_cur = dl_pre;
      }
    }  // working warp
  } else {
    // ============================ token group: thread = token of the chunk = TMEM lane ============================
    const int wq = warp - W_TOKEN;
    const uint32_t tl = tmem + ((uint32_t)(wq * 32) << 16);
    const int tt = wq * 32 + lane;
    const int lo = BLOCK ? (tt & ~(p.block - 1)) : tt;  // first column (token) this row keeps
    __nv_bfloat16* dv_base;
    int64_t dv_stride_n;
    {
      const int64_t group_off = p.groups > 1 ? (int64_t)group * ((int64_t)(gridDim.x / p.H) * p.N * p.H * DV) : 0;
      dv_base = reinterpret_cast<__nv_bfloat16*>(p.dv) + group_off + ((int64_t)b * p.N * p.H + h) * DV;
      dv_stride_n = (int64_t)p.H * DV;
    }
    for (int j = 0; ok && j < nch; ++j) {
      const int i = nch - 1 - j, t0 = i * C;
      const uint32_t par = j & 1;
      const int nvalid = min(C, p.N - t0);
      // masked A (bf16) into the K tile's buffer
      if (!(ok = wait_or_abort(&misc->a_ready, par, misc))) break;
      tc_fence_after_sync();
      if (tid == W_TOKEN * 32) BT_TRACE(1, j, 0);
#pragma unroll 1
      for (int jb = 0; jb < 4; ++jb) {
        uint32_t wp[16];
        if (jb * 32 + 31 >= lo) {
          uint32_t r[32];
          tmem_ld32(tl + T0 + jb * 32, r);
          tmem_wait_ld();
          tmem_fence_regs(r);
          if (jb * 32 >= lo) {
#pragma unroll
            for (int k = 0; k < 32; k += 2) wp[k >> 1] = pack_bf16(__uint_as_float(r[k]), __uint_as_float(r[k + 1]));
          } else {
#pragma unroll
            for (int k = 0; k < 32; k += 2)
              wp[k >> 1] = pack_bf16(jb * 32 + k >= lo ? __uint_as_float(r[k]) : 0.f,
                                     jb * 32 + k + 1 >= lo ? __uint_as_float(r[k + 1]) : 0.f);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 16; ++k) wp[k] = 0u;
        }
        uint8_t* blk = smem + L::OFF_KA + (jb >> 1) * 16384;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          *reinterpret_cast<uint4*>(blk + swz_chunk_off(tt, (jb & 1) * 4 + ch)) =
              make_uint4(wp[ch * 4], wp[ch * 4 + 1], wp[ch * 4 + 2], wp[ch * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      warp_arrive(&misc->am_done, lane);
      if (tid == W_TOKEN * 32) BT_TRACE(1, j, 1);
      // masked E^T R (bf16) into tensor memory
      if (!(ok = wait_or_abort(&misc->wt_ready, par, misc))) break;
      tc_fence_after_sync();
      if (tid == W_TOKEN * 32) BT_TRACE(1, j, 2);
#pragma unroll 1
      for (int jb = 0; jb < 4; ++jb) {
        uint32_t wp[16];
        if (jb * 32 + 31 >= lo) {
          uint32_t r[32];
          tmem_ld32(tl + T0 + jb * 32, r);
          tmem_wait_ld();
          tmem_fence_regs(r);
          if (jb * 32 >= lo) {
#pragma unroll
            for (int k = 0; k < 32; k += 2) wp[k >> 1] = pack_bf16(__uint_as_float(r[k]), __uint_as_float(r[k + 1]));
          } else {
#pragma unroll
            for (int k = 0; k < 32; k += 2)
              wp[k >> 1] = pack_bf16(jb * 32 + k >= lo ? __uint_as_float(r[k]) : 0.f,
                                     jb * 32 + k + 1 >= lo ? __uint_as_float(r[k + 1]) : 0.f);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 16; ++k) wp[k] = 0u;
        }
        tmem_st16(tl + T2 + jb * 16, wp);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      warp_arrive(&misc->wm_done, lane);
      if (tid == W_TOKEN * 32) BT_TRACE(1, j, 3);
      // dV rows
      if (!(ok = wait_or_abort(&misc->dv_ready, par, misc))) break;
      tc_fence_after_sync();
      if (tid == W_TOKEN * 32) BT_TRACE(1, j, 4);
#pragma unroll
      for (int half = 0; half < DV / 32; ++half) {
        uint32_t r[32];
        tmem_ld32(tl + T0 + half * 32, r);
        tmem_wait_ld();
        tmem_fence_regs(r);
        if (tt < nvalid) {
          uint4* dst = reinterpret_cast<uint4*>(dv_base + (int64_t)(t0 + tt) * dv_stride_n + half * 32);
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[ch * 8 + 0]), __uint_as_float(r[ch * 8 + 1]));
            v.y = pack_bf16(__uint_as_float(r[ch * 8 + 2]), __uint_as_float(r[ch * 8 + 3]));
            v.z = pack_bf16(__uint_as_float(r[ch * 8 + 4]), __uint_as_float(r[ch * 8 + 5]));
            v.w = pack_bf16(__uint_as_float(r[ch * 8 + 6]), __uint_as_float(r[ch * 8 + 7]));
            dst[ch] = v;
          }
        }
      }
      tc_fence_before_sync();
      warp_arrive(&misc->dv_free, lane);
      if (tid == W_TOKEN * 32) BT_TRACE(1, j, 5);
    }
  }
  if (!ok) {
    misc->abort_flag = 1;
    atomicOr(p.err, 1);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == W_MMA) tmem_dealloc(tmem, TM_COLS);
}

namespace {

template <int DKB, int DVB, int MODE>
int launch_main(const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdy, const CUtensorMap& tu,
                const BwdTcParams& p, dim3 grid, cudaStream_t stream) {
  auto kern = bwd_tc_kernel<DKB, DVB, MODE>;
  FLARE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BL<DVB>::SMEM_BYTES));
  LaunchTimer timer("bwd_tc_kernel", stream);
  kern<<<grid, NT_MAIN, BL<DVB>::SMEM_BYTES, stream>>>(tk, tv, tdy, tu, p);
  FLARE_CUDA_CHECK(cudaGetLastError());
  return FLARE_OK;
}

}  // namespace

template <>
int launch_bwd_tc_unit<FLARE_BT_UNIT>(int mode, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdy,
                                      const CUtensorMap& tu, const BwdTcParams& p, dim3 grid, cudaStream_t stream) {
  // units 0..2: (Dk, Dv) = (64, 64), (128, 128), (64, 128)
  constexpr int DKB = FLARE_BT_UNIT == 1 ? 2 : 1;
  constexpr int DVB = FLARE_BT_UNIT == 0 ? 1 : 2;
  if (mode == 1) return launch_main<DKB, DVB, 1>(tk, tv, tdy, tu, p, grid, stream);
  if (mode == 2) return launch_main<DKB, DVB, 2>(tk, tv, tdy, tu, p, grid, stream);
  return launch_main<DKB, DVB, 0>(tk, tv, tdy, tu, p, grid, stream);
}

#else  // host side, the dK / dQ kernel and the small helper kernels

template <> int launch_bwd_tc_unit<0>(int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const BwdTcParams&, dim3, cudaStream_t);
template <> int launch_bwd_tc_unit<1>(int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const BwdTcParams&, dim3, cudaStream_t);
template <> int launch_bwd_tc_unit<2>(int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const BwdTcParams&, dim3, cudaStream_t);

namespace {

// -------------------------------------------------------------------------------------------------
// per-token statistics: delta_t = <dY_t, y_t> and the decode log-sum-exp in log2 units, rows padded to whole chunks
// (delta = 0, log-sum-exp = +inf there, which makes every decode weight of a padding token exactly zero)
// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bwd_tc_token_stats_kernel(const __nv_bfloat16* __restrict__ dy, int64_t dy_sb,
                                                                  int64_t dy_sn, int64_t dy_sh,
                                                                  const __nv_bfloat16* __restrict__ y, int64_t y_sb,
                                                                  int64_t y_sn, int64_t y_sh, const float* __restrict__ lse,
                                                                  int B, int N, int H, int Dv, int npad, float* tok_l2,
                                                                  float* tok_delta) {
  // Dv / 8 threads per (b, n, h) row (8 or 16, a divisor of the warp size), one 16-byte load of dY and of y each
  const int tpr = Dv >> 3;
  const int64_t row = (int64_t)blockIdx.x * (256 / tpr) + threadIdx.x / tpr;  // (b, n, h), h fastest
  const int sub = threadIdx.x % tpr;
  const bool in_range = row < (int64_t)B * npad * H;
  const int h = in_range ? (int)(row % H) : 0;
  const int64_t bn = in_range ? row / H : 0;
  const int n = (int)(bn % npad);
  const int b = (int)(bn / npad);
  float acc = 0.f;
  if (in_range && n < N) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(dy + b * dy_sb + (int64_t)n * dy_sn + h * dy_sh + sub * 8));
    const uint4 c = __ldg(reinterpret_cast<const uint4*>(y + b * y_sb + (int64_t)n * y_sn + h * y_sh + sub * 8));
    acc = (bf16_lo(a.x) * bf16_lo(c.x) + bf16_hi(a.x) * bf16_hi(c.x)) + (bf16_lo(a.y) * bf16_lo(c.y) + bf16_hi(a.y) * bf16_hi(c.y)) +
          (bf16_lo(a.z) * bf16_lo(c.z) + bf16_hi(a.z) * bf16_hi(c.z)) + (bf16_lo(a.w) * bf16_lo(c.w) + bf16_hi(a.w) * bf16_hi(c.w));
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1)
    if (o < tpr) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (in_range && sub == 0) {
    const int64_t o = ((int64_t)b * H + h) * npad + n;
    tok_delta[o] = n < N ? acc : 0.f;
    tok_l2[o] = n < N ? lse[((int64_t)b * H + h) * N + n] * kLog2e : INFINITY;
  }
}

// sum of the latent groups' dV partials (bf16) in fp32
__global__ void __launch_bounds__(256) bwd_tc_sum_groups_kernel(const __nv_bfloat16* __restrict__ part, int groups, int64_t n8,
                                                                 __nv_bfloat16* out) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n8) return;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int g = 0; g < groups; ++g) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(part + (int64_t)g * n8 * 8) + idx);
    acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
    acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
  }
  reinterpret_cast<uint4*>(out)[idx] = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]),
                                                  pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
}

// dq[i] = sum over the (batch, split) partials in fixed order
__global__ void __launch_bounds__(256) bwd_tc_sum_dq_kernel(const float* __restrict__ part, int count, int64_t n4, float* out) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n4) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < count; ++s) {
    const float4 v = __ldcs(reinterpret_cast<const float4*>(part + (int64_t)s * n4 * 4) + idx);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  reinterpret_cast<float4*>(out)[idx] = acc;
}

// -------------------------------------------------------------------------------------------------
// dK = scale dS^T Q per chunk, dQ = scale sum_t dS K per (lane, split of the chunks).
// One CTA per (lane, split), 6 warps: 0 TMA producer, 1 MMA issuer, 2-5 epilogue (thread = TMEM lane).
// -------------------------------------------------------------------------------------------------
constexpr int NT_GRAD = 192;
constexpr int GRAD_MAXG = 4;

template <int DKB>
struct GL {
  static constexpr int OFF_DS = 0;                         // 2 stages x [2 m-blocks][128 t][64 m]
  static constexpr int OFF_K = 65536;                      // 2 stages x [DKB][128 t][64]
  static constexpr int OFF_Q = OFF_K + 2 * DKB * 16384;    // groups x [DKB][128 m][64]
  static constexpr int off_misc(int groups) { return OFF_Q + groups * DKB * 16384; }
  static constexpr int smem_bytes(int groups) { return off_misc(groups) + 256 + 1024; }
  static constexpr uint32_t TM_DK = 0;                     // 2 buffers x Dk columns
  static constexpr uint32_t TM_DQ = 2 * DKB * 64;          // groups x Dk columns
};

struct GradMisc {
  uint64_t q_full, ds_full[2], ds_empty[2], k_full[2], k_empty[2], dk_ready[2], dk_free[2], dq_ready;
  uint32_t tmem_base;
  volatile int abort_flag;
};

template <int DKB>
__global__ void __launch_bounds__(NT_GRAD, 1)
bwd_tc_grads_kernel(const __grid_constant__ CUtensorMap tm_ds, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_q, const GradTcParams p) {
  using L = GL<DKB>;
  constexpr int DK = DKB * 64;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  const int G = p.groups;
  GradMisc* misc = reinterpret_cast<GradMisc*>(smem + L::off_misc(G));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lane_id = blockIdx.x, split = blockIdx.y;
  const int b = lane_id / p.H, h = lane_id % p.H;
  const int c_begin = split * p.chunks_per_split, c_end = min(p.nch, c_begin + p.chunks_per_split);
  const int ncs = max(0, c_end - c_begin);
  const uint32_t tm_cols = (2 + G) * DK <= 256 ? 256u : 512u;

  if (tid == 0) {
    mbar_init(&misc->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&misc->ds_full[i], 1);
      mbar_init(&misc->ds_empty[i], 1);
      mbar_init(&misc->k_full[i], 1);
      mbar_init(&misc->k_empty[i], 1);
      mbar_init(&misc->dk_ready[i], 1);
      mbar_init(&misc->dk_free[i], 4);
    }
    mbar_init(&misc->dq_ready, 1);
    misc->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&misc->tmem_base, tm_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = misc->tmem_base;
  bool ok = true;
  auto wait = [&](uint64_t* bar, uint32_t parity) { return tc::wait_or_abort(bar, parity, &misc->abort_flag, 1); };

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&tm_ds);
      prefetch_tensormap(&tm_k);
      mbar_arrive_expect_tx(&misc->q_full, G * DKB * 16384);
      for (int g = 0; g < G; ++g)
        for (int kb = 0; kb < DKB; ++kb)
          tma_load_3d(smem + L::OFF_Q + (g * DKB + kb) * 16384, &tm_q, &misc->q_full, kb * 64, g * 128, h);
      int it = 0;
      for (int cc = 0; ok && cc < ncs; ++cc) {
        const int t0 = (c_begin + cc) * C;
        const int ks = cc & 1;
        if (cc >= 2 && !(ok = wait(&misc->k_empty[ks], ((cc - 2) >> 1) & 1))) break;
        mbar_arrive_expect_tx(&misc->k_full[ks], DKB * 16384);
        for (int kb = 0; kb < DKB; ++kb)
          tma_load_4d(smem + L::OFF_K + (ks * DKB + kb) * 16384, &tm_k, &misc->k_full[ks], kb * 64, h, t0, b);
        for (int gp = 0; ok && gp < 2 * G; ++gp, ++it) {  // (group, hi | lo plane)
          const int g = gp >> 1, part = gp & 1;
          const int s = it & 1;
          if (it >= 2 && !(ok = wait(&misc->ds_empty[s], ((it - 2) >> 1) & 1))) break;
          mbar_arrive_expect_tx(&misc->ds_full[s], 32768);
          for (int mb = 0; mb < 2; ++mb)
            tma_load_4d(smem + L::OFF_DS + s * 32768 + mb * 16384, &tm_ds, &misc->ds_full[s], g * 128 + mb * 64, part, t0,
                        lane_id);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t ID_DK = make_idesc_bf16(128, DK, 0, 1);  // dS (K-major: rows = tokens, latents contiguous) x Q (MN-major)
      constexpr uint32_t ID_DQ = make_idesc_bf16(128, DK, 1, 1);  // dS (MN-major) x K tile (MN-major)
      ok = wait(&misc->q_full, 0);
      int it = 0;
      for (int cc = 0; ok && cc < ncs; ++cc) {
        const int ks = cc & 1, kb = cc & 1;
        if (!(ok = wait(&misc->k_full[ks], (cc >> 1) & 1))) break;
        if (cc >= 2 && !(ok = wait(&misc->dk_free[kb], ((cc - 2) >> 1) & 1))) break;
        tc_fence_after_sync();
        const uint64_t d_k_mn = make_desc_sw128(smem_u32(smem + L::OFF_K + ks * DKB * 16384), 16384, 1024);
        for (int gp = 0; ok && gp < 2 * G; ++gp, ++it) {  // (group, hi | lo plane): lo accumulates on top of hi
          const int g = gp >> 1;
          const int s = it & 1;
          if (!(ok = wait(&misc->ds_full[s], (it >> 1) & 1))) break;
          tc_fence_after_sync();
          const uint32_t ds_addr = smem_u32(smem + L::OFF_DS + s * 32768);
          const uint64_t d_ds_mn = make_desc_sw128(ds_addr, 16384, 1024), d_ds_k = make_desc_sw128(ds_addr, 16, 1024);
          const uint64_t d_q_mn = make_desc_sw128(smem_u32(smem + L::OFF_Q + g * DKB * 16384), 16384, 1024);
          const int rows = min(128, p.M - g * 128);
          const int ksm = (rows + 15) >> 4;
          for (int st = 0; st < ksm; ++st)  // contraction over the latents of the group
            mma_ss(tmem + L::TM_DK + kb * DK, kmaj_step(d_ds_k, st), mnmaj_step(d_q_mn, st), ID_DK, (gp > 0 || st > 0) ? 1u : 0u);
#pragma unroll
          for (int st = 0; st < 8; ++st)  // contraction over the tokens of the chunk
            mma_ss(tmem + L::TM_DQ + g * DK, mnmaj_step(d_ds_mn, st), mnmaj_step(d_k_mn, st), ID_DQ,
                   (cc > 0 || (gp & 1) || st > 0) ? 1u : 0u);
          tc_commit(&misc->ds_empty[s]);
        }
        if (!ok) break;
        tc_commit(&misc->dk_ready[kb]);
        tc_commit(&misc->k_empty[ks]);
      }
      if (ok) tc_commit(&misc->dq_ready);
    }
  } else {
    const int wq = warp & 3;  // TMEM lane quarter of this warp
    const uint32_t tl = tmem + ((uint32_t)(wq * 32) << 16);
    const int tt = wq * 32 + lane;
    __nv_bfloat16* dk_base = reinterpret_cast<__nv_bfloat16*>(p.dk) + ((int64_t)b * p.N * p.H + h) * DK;
    for (int cc = 0; ok && cc < ncs; ++cc) {
      const int kb = cc & 1;
      const int t = (c_begin + cc) * C + tt;
      if (!(ok = wait(&misc->dk_ready[kb], (cc >> 1) & 1))) break;
      tc_fence_after_sync();
#pragma unroll
      for (int half = 0; half < DK / 32; ++half) {
        uint32_t r[32];
        tmem_ld32(tl + L::TM_DK + kb * DK + half * 32, r);
        tmem_wait_ld();
        tmem_fence_regs(r);
        if (t < p.N) {
          uint4* dst = reinterpret_cast<uint4*>(dk_base + (int64_t)t * p.H * DK + half * 32);
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[ch * 8 + 0]) * p.scale, __uint_as_float(r[ch * 8 + 1]) * p.scale);
            v.y = pack_bf16(__uint_as_float(r[ch * 8 + 2]) * p.scale, __uint_as_float(r[ch * 8 + 3]) * p.scale);
            v.z = pack_bf16(__uint_as_float(r[ch * 8 + 4]) * p.scale, __uint_as_float(r[ch * 8 + 5]) * p.scale);
            v.w = pack_bf16(__uint_as_float(r[ch * 8 + 6]) * p.scale, __uint_as_float(r[ch * 8 + 7]) * p.scale);
            dst[ch] = v;
          }
        }
      }
      tc_fence_before_sync();
      warp_arrive(&misc->dk_free[kb], lane);
    }
    // this split's part of dQ
    float* part = p.dq_part + (((int64_t)(b * p.nsplit + split) * p.H + h) * p.M) * DK;
    if (ncs > 0) ok = ok && wait(&misc->dq_ready, 0);
    tc_fence_after_sync();
    for (int g = 0; g < G; ++g) {
      const int mg = g * 128 + tt;
#pragma unroll
      for (int half = 0; half < DK / 32; ++half) {
        uint32_t r[32];
        if (ncs > 0 && ok) {
          tmem_ld32(tl + L::TM_DQ + g * DK + half * 32, r);
          tmem_wait_ld();
          tmem_fence_regs(r);
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) r[k] = 0u;
        }
        if (mg < p.M) {
          float4* dst = reinterpret_cast<float4*>(part + (int64_t)mg * DK + half * 32);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            dst[k] = make_float4(__uint_as_float(r[4 * k]) * p.scale, __uint_as_float(r[4 * k + 1]) * p.scale,
                                 __uint_as_float(r[4 * k + 2]) * p.scale, __uint_as_float(r[4 * k + 3]) * p.scale);
        }
      }
    }
  }
  if (!ok) {
    misc->abort_flag = 1;
    atomicOr(p.err, 1);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, tm_cols);
}

template <int DKB>
int launch_grads(const CUtensorMap& tds, const CUtensorMap& tk, const CUtensorMap& tq, const GradTcParams& p, dim3 grid,
                 cudaStream_t stream) {
  auto kern = bwd_tc_grads_kernel<DKB>;
  const int smem = GL<DKB>::smem_bytes(p.groups);
  FLARE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  LaunchTimer timer("bwd_tc_grads_kernel", stream);
  kern<<<grid, NT_GRAD, smem, stream>>>(tds, tk, tq, p);
  FLARE_CUDA_CHECK(cudaGetLastError());
  return FLARE_OK;
}

// -------------------------------------------------------------------------------------------------
// host: plan, workspace, launch sequence
// -------------------------------------------------------------------------------------------------
bool have_saved(const flare_bwd_args_t& a);  // defined below, with the keep-buffer layout

struct TcBwdPlan {
  int nch, npad, groups, nsplit, chunks_per_split;
  size_t gate_bytes;  // per-call gate words come first
  size_t exact_bytes;  // path AUTO: scratch of the exact pass standing by (shares the space behind the gate words)
  size_t fwd_ws;  // then the forward's own scratch
  size_t off_y, off_lse, off_l2, off_delta, off_cu, off_cc, off_cd, off_ds, off_dqp, off_dvp, total;
};

TcBwdPlan plan_tc(const flare_bwd_args_t& a) {
  const flare_fwd_args_t& f = a.fwd;
  TcBwdPlan pl;
  memset(&pl, 0, sizeof(pl));
  pl.nch = (f.N + C - 1) / C;
  pl.npad = pl.nch * C;
  pl.groups = (f.M + 127) / 128;
  const int64_t lanes = (int64_t)f.B * f.H;
  int nsplit = (int)(sm_count() / (lanes > 0 ? lanes : 1));
  if (nsplit < 1) nsplit = 1;
  if (nsplit > pl.nch) nsplit = pl.nch;
  pl.chunks_per_split = (pl.nch + nsplit - 1) / nsplit;
  pl.nsplit = (pl.nch + pl.chunks_per_split - 1) / pl.chunks_per_split;
  flare_fwd_args_t probe = f;
  probe.y = const_cast<void*>(a.dy);  // any non-null pointer: "an output is wanted"
  probe.y_stride_b = a.dy_stride_b; probe.y_stride_n = a.dy_stride_n; probe.y_stride_h = a.dy_stride_h;
  probe.mask = nullptr; probe.lengths = nullptr;
  probe.lse_dec = nullptr; probe.lse_enc = nullptr;
  memset(&probe.state_in, 0, sizeof(probe.state_in));
  memset(&probe.state_out, 0, sizeof(probe.state_out));
  probe.path = FLARE_PATH_TENSOR;
  probe.keep = nullptr; probe.keep_bytes = 0;
  const bool saved = have_saved(a);
  pl.fwd_ws = saved ? 0 : align_up(flare_forward_workspace_bytes(&probe), 256);
  pl.gate_bytes = align_up((size_t)(1 + lanes) * sizeof(int), 256);
  size_t off = pl.gate_bytes + pl.fwd_ws;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off += align_up(bytes, 256);
    return o;
  };
  pl.off_y = saved ? 0 : take((size_t)f.B * f.N * f.H * f.Dv * 2);
  pl.off_lse = saved ? 0 : take((size_t)lanes * f.N * 4);
  pl.off_l2 = take((size_t)lanes * pl.npad * 4);
  pl.off_delta = take((size_t)lanes * pl.npad * 4);
  pl.off_cu = saved ? 0 : take((size_t)lanes * pl.nch * f.M * f.Dv * 2);
  pl.off_cc = saved ? 0 : take((size_t)lanes * pl.nch * f.M * 4);
  pl.off_cd = saved ? 0 : take((size_t)lanes * pl.nch * f.M * 4);
  pl.off_ds = take((size_t)2 * lanes * f.M * pl.npad * 2);  // a hi and a lo row per token
  pl.off_dqp = take((size_t)f.B * pl.nsplit * f.H * f.M * f.Dk * 4);
  pl.off_dvp = pl.groups > 1 ? take((size_t)pl.groups * f.B * f.N * f.H * f.Dv * 2) : 0;
  pl.total = off;
  if (f.path == FLARE_PATH_AUTO) {
    flare_bwd_args_t ex = a;
    ex.fwd.path = FLARE_PATH_EXACT;
    pl.exact_bytes = bwd_exact_workspace_bytes(ex);
    if (pl.gate_bytes + pl.exact_bytes > pl.total) pl.total = pl.gate_bytes + pl.exact_bytes;
  }
  return pl;
}

}  // namespace

// the forward problems whose backward runs on the tensor kernels (everything but the gradient-side conditions)
static bool tc_trainable(const flare_fwd_args_t& f) {
  if (f.path == FLARE_PATH_EXACT || f.B <= 0 || f.N <= 0 || f.state_in.u != nullptr) return false;
  flare_fwd_args_t probe = f;
  if (probe.y == nullptr) probe.y = const_cast<void*>(f.k);  // any aligned non-null pointer: "an output is wanted"
  probe.mask = nullptr; probe.lengths = nullptr; probe.lse_dec = nullptr; probe.lse_enc = nullptr;
  memset(&probe.state_in, 0, sizeof(probe.state_in));
  memset(&probe.state_out, 0, sizeof(probe.state_out));
  probe.path = FLARE_PATH_TENSOR;
  if (f.mask != nullptr || f.lengths != nullptr || !prefill_tc_supported(&probe)) return false;
  const int groups = (f.M + 127) / 128;
  return (2 + groups) * f.Dk <= 512;  // tensor-memory columns of the dK / dQ kernel
}

KeepLayout keep_layout(const flare_fwd_args_t& f) {
  KeepLayout k;
  memset(&k, 0, sizeof(k));
  if (!tc_trainable(f)) return k;
  const size_t lanes = (size_t)f.B * f.H;
  k.nch = (f.N + C - 1) / C;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off += align_up(bytes, 256);
    return o;
  };
  k.off_gate = take((1 + lanes) * sizeof(int));
  k.off_u = take(lanes * k.nch * f.M * f.Dv * 2);
  k.off_c = take(lanes * k.nch * f.M * 4);
  k.off_d = take(lanes * k.nch * f.M * 4);
  k.total = off;
  return k;
}

// true when the caller handed over what a forward with `keep` left behind
namespace {
bool have_saved(const flare_bwd_args_t& a) {
  if (a.y == nullptr || a.lse_dec == nullptr || a.fwd.keep == nullptr) return false;
  const KeepLayout k = keep_layout(a.fwd);
  return k.total > 0 && a.fwd.keep_bytes >= k.total && (reinterpret_cast<uintptr_t>(a.fwd.keep) & 255u) == 0 &&
         (reinterpret_cast<uintptr_t>(a.y) & 15u) == 0 && (a.y_stride_b % 8) == 0 && (a.y_stride_n % 8) == 0 &&
         (a.y_stride_h % 8) == 0;
}
}  // namespace

bool bwd_tc_supported(const flare_bwd_args_t& a) {
  const flare_fwd_args_t& f = a.fwd;
  if (a.carry_b || a.carry_c || a.carry_rho || a.span_b0 || a.span_c0 || a.span_gam || a.span_rho_first || a.phase != 0)
    return false;  // spans of a longer sequence run on the exact kernels
  if (!tc_trainable(f)) return false;
  if ((reinterpret_cast<uintptr_t>(a.dy) & 15u) || (a.dy_stride_b % 8) || (a.dy_stride_n % 8) || (a.dy_stride_h % 8)) return false;
  return true;
}

size_t bwd_tc_workspace_bytes(const flare_bwd_args_t& a) { return plan_tc(a).total; }

int bwd_tc(const flare_bwd_args_t& a, cudaStream_t stream) {
  const flare_fwd_args_t& f = a.fwd;
  const TcBwdPlan pl = plan_tc(a);
  if (f.workspace == nullptr || f.workspace_bytes < pl.total || (reinterpret_cast<uintptr_t>(f.workspace) & 255u))
    return FLARE_ERR_WORKSPACE;
  char* ws = reinterpret_cast<char*>(f.workspace);
  const int64_t lanes = (int64_t)f.B * f.H;
  int* gate = reinterpret_cast<int*>(ws);
  const bool saved = have_saved(a);
  const void* y = nullptr;
  int64_t y_sb, y_sn, y_sh;
  const float* lse = nullptr;
  ChunkStates keep{nullptr, nullptr, nullptr, pl.nch};
  if (saved) {
    // (1') the training forward kept everything: its output, its log-sum-exp, the chunk states, its gate words
    const KeepLayout kl = keep_layout(f);
    char* kb = reinterpret_cast<char*>(f.keep);
    FLARE_CUDA_CHECK(cudaMemcpyAsync(gate, kb + kl.off_gate, (size_t)(1 + lanes) * sizeof(int), cudaMemcpyDeviceToDevice, stream));
    keep.u = kb + kl.off_u;
    keep.c = reinterpret_cast<float*>(kb + kl.off_c);
    keep.d = reinterpret_cast<float*>(kb + kl.off_d);
    y = a.y; y_sb = a.y_stride_b; y_sn = a.y_stride_n; y_sh = a.y_stride_h;
    lse = a.lse_dec;
  } else {
    // (1) forward on the tensor path: y, the decode log-sum-exp and the per-chunk prefix states
    FLARE_CUDA_CHECK(cudaMemsetAsync(gate, 0, pl.gate_bytes, stream));
    keep.u = ws + pl.off_cu;
    keep.c = reinterpret_cast<float*>(ws + pl.off_cc);
    keep.d = reinterpret_cast<float*>(ws + pl.off_cd);
    flare_fwd_args_t fw = f;
    fw.y = ws + pl.off_y;
    fw.y_stride_b = (int64_t)f.N * f.H * f.Dv; fw.y_stride_n = (int64_t)f.H * f.Dv; fw.y_stride_h = f.Dv;
    fw.mask = nullptr; fw.lengths = nullptr;
    fw.lse_dec = reinterpret_cast<float*>(ws + pl.off_lse); fw.lse_enc = nullptr;
    fw.keep = nullptr; fw.keep_bytes = 0;
    memset(&fw.state_in, 0, sizeof(fw.state_in));
    memset(&fw.state_out, 0, sizeof(fw.state_out));
    fw.workspace = ws + pl.gate_bytes; fw.workspace_bytes = pl.fwd_ws;
    fw.path = FLARE_PATH_TENSOR;
    const int rc = forward_keep_states(&fw, keep, gate, stream);
    if (rc != FLARE_OK) return rc;
    y = fw.y; y_sb = fw.y_stride_b; y_sn = fw.y_stride_n; y_sh = fw.y_stride_h;
    lse = fw.lse_dec;
  }
  float* tok_l2 = reinterpret_cast<float*>(ws + pl.off_l2);
  float* tok_delta = reinterpret_cast<float*>(ws + pl.off_delta);
  // (2) per-token statistics
  {
    const int64_t rows = (int64_t)f.B * pl.npad * f.H;
    const int rows_per_block = 256 / (f.Dv / 8);
    LaunchTimer timer("bwd_tc_token_stats_kernel", stream);
    bwd_tc_token_stats_kernel<<<(unsigned)((rows + rows_per_block - 1) / rows_per_block), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(a.dy), a.dy_stride_b, a.dy_stride_n, a.dy_stride_h,
        reinterpret_cast<const __nv_bfloat16*>(y), y_sb, y_sn, y_sh, lse, f.B, f.N,
        f.H, f.Dv, pl.npad, tok_l2, tok_delta);
    FLARE_CUDA_CHECK(cudaGetLastError());
    count_launches(1);
  }
  int* err = nullptr;
  {
    const int rc = tc_error_word(&err);
    if (rc != FLARE_OK) return rc;
  }
  // (3) reverse chunk sweep: dV and the dS plane
  CUtensorMap tk, tv, tdy, tu, tds, tq;
  {
    const uint64_t dimk[4] = {(uint64_t)f.Dk, (uint64_t)f.H, (uint64_t)f.N, (uint64_t)f.B};
    const uint64_t dimv[4] = {(uint64_t)f.Dv, (uint64_t)f.H, (uint64_t)f.N, (uint64_t)f.B};
    const uint32_t box[4] = {64, 1, 128, 1};
    const int64_t strk[3] = {f.k_stride_h, f.k_stride_n, f.k_stride_b};
    const int64_t strv[3] = {f.v_stride_h, f.v_stride_n, f.v_stride_b};
    const int64_t strd[3] = {a.dy_stride_h, a.dy_stride_n, a.dy_stride_b};
    const uint64_t dimu[4] = {(uint64_t)f.Dv, (uint64_t)f.M, (uint64_t)pl.nch, (uint64_t)lanes};
    const int64_t stru[3] = {f.Dv, (int64_t)f.M * f.Dv, (int64_t)pl.nch * f.M * f.Dv};
    const uint32_t boxu[4] = {64, 128, 1, 1};
    const uint64_t dims[4] = {(uint64_t)f.M, 2, (uint64_t)pl.npad, (uint64_t)lanes};
    const int64_t strs[3] = {f.M, 2 * (int64_t)f.M, 2 * (int64_t)f.M * pl.npad};
    const uint32_t boxs[4] = {64, 1, 128, 1};
    const uint64_t dimq[3] = {(uint64_t)f.Dk, (uint64_t)f.M, (uint64_t)f.H};
    const int64_t strq[2] = {f.q_stride_m, f.q_stride_h};
    const uint32_t boxq[3] = {64, 128, 1};
    if (!tc::make_map_bf16(&tk, f.k, 4, dimk, strk, box) || !tc::make_map_bf16(&tv, f.v, 4, dimv, strv, box) ||
        !tc::make_map_bf16(&tdy, a.dy, 4, dimv, strd, box) || !tc::make_map_bf16(&tu, keep.u, 4, dimu, stru, boxu) ||
        !tc::make_map_bf16(&tds, ws + pl.off_ds, 4, dims, strs, boxs) || !tc::make_map_bf16(&tq, f.q, 3, dimq, strq, boxq)) {
      set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled (backward operands)");
      return FLARE_ERR_CUDA;
    }
  }
  {
    BwdTcParams p;
    memset(&p, 0, sizeof(p));
    p.q = f.q; p.q_stride_h = f.q_stride_h; p.q_stride_m = f.q_stride_m;
    p.N = f.N; p.H = f.H; p.M = f.M; p.nch = pl.nch; p.npad = pl.npad; p.block = f.block_size;
    p.scale = f.scale; p.power = f.power;
    p.chunk_c = keep.c; p.chunk_d = keep.d; p.tok_l2 = tok_l2; p.tok_delta = tok_delta;
    p.ds = ws + pl.off_ds;
    p.groups = pl.groups;
    p.dv = pl.groups > 1 ? static_cast<void*>(ws + pl.off_dvp) : a.dv;
    p.err = err;
    p.gate = gate;
    p.trace = trace_buffer();
    const int mode = f.variant == FLARE_STABLEMAX ? 2 : (f.block_size > 1 ? 1 : 0);
    const dim3 grid((unsigned)lanes, pl.groups, 1);
    int rc;
    if (f.Dk == 128) rc = launch_bwd_tc_unit<1>(mode, tk, tv, tdy, tu, p, grid, stream);
    else if (f.Dv == 128) rc = launch_bwd_tc_unit<2>(mode, tk, tv, tdy, tu, p, grid, stream);
    else rc = launch_bwd_tc_unit<0>(mode, tk, tv, tdy, tu, p, grid, stream);
    if (rc != FLARE_OK) return rc;
    count_launches(1);
    if (pl.groups > 1) {
      const int64_t n8 = (int64_t)f.B * f.N * f.H * f.Dv / 8;
      LaunchTimer timer("bwd_tc_sum_groups_kernel", stream);
      bwd_tc_sum_groups_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(
          reinterpret_cast<const __nv_bfloat16*>(ws + pl.off_dvp), pl.groups, n8, reinterpret_cast<__nv_bfloat16*>(a.dv));
      FLARE_CUDA_CHECK(cudaGetLastError());
      count_launches(1);
    }
  }
  // (4) dK and dQ from the dS plane
  {
    GradTcParams g;
    memset(&g, 0, sizeof(g));
    g.N = f.N; g.H = f.H; g.M = f.M; g.B = f.B; g.nch = pl.nch; g.npad = pl.npad; g.groups = pl.groups;
    g.nsplit = pl.nsplit; g.chunks_per_split = pl.chunks_per_split; g.scale = f.scale;
    g.dk = a.dk; g.dq_part = reinterpret_cast<float*>(ws + pl.off_dqp);
    g.err = err;
    const dim3 grid((unsigned)lanes, pl.nsplit, 1);
    const int rc = f.Dk == 128 ? launch_grads<2>(tds, tk, tq, g, grid, stream) : launch_grads<1>(tds, tk, tq, g, grid, stream);
    if (rc != FLARE_OK) return rc;
    const int64_t n4 = (int64_t)f.H * f.M * f.Dk / 4;
    LaunchTimer timer("bwd_tc_sum_dq_kernel", stream);
    bwd_tc_sum_dq_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>(g.dq_part, f.B * pl.nsplit, n4, a.dq);
    FLARE_CUDA_CHECK(cudaGetLastError());
    count_launches(2);
  }
  // (5) path AUTO: the exact pass stands by.  Each of its kernels looks at the gate word and returns at once unless the
  // tensor kernels above found the inputs outside their numeric domain, in which case it rewrites dq, dk, dv.
  if (f.path == FLARE_PATH_AUTO) {
    flare_bwd_args_t ex = a;
    ex.fwd.path = FLARE_PATH_EXACT;
    ex.fwd.workspace = ws + pl.gate_bytes;
    ex.fwd.workspace_bytes = pl.total - pl.gate_bytes;
    const int rc = bwd_exact(ex, stream, gate);
    if (rc != FLARE_OK) return rc;
  }
  return FLARE_OK;
}

#endif  // FLARE_BT_UNIT

}  // namespace flare
