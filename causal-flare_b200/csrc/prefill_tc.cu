// Tensor-core (tcgen05 + TMEM + TMA) chunked causal prefill, bf16 operands, fp32 accumulation and statistics.
// Shape class: M <= 512 latents (multiple of 16, in groups of 128 rows, the last one padded), (Dk, Dv) = (64, 64),
// (128, 128) or (64, 128), shared decode weights; softmax encoder token- or block-causal, stablemax encoder
// token-causal; optional per-row lengths (right padding).
//
// One CTA owns a (batch, head, sequence segment, slice of 64 value columns, group of 128 latents) and walks its chunks
// of C = 128 tokens in order ((128, 128) heads on a grid that would not fit the SMs at once: one CTA for all 128
// value columns, the "wide" instance below).  With more than one latent group every CTA emits a partial read-out
// (normalised over its own latents, fp16) and the log2 of its weight mass per token; a small kernel merges the
// groups.  Read-out rows leave the CTA as tiled bulk stores of 32 x 32 tiles staged in shared memory.  The CTA carries the
// latent state on chip: U [128 latents x 64] fp32 in tensor memory, the latent bank Q in shared memory (Dk = 64) or
// as packed bf16 in tensor memory (Dk = 128; A operand of the score MMA), running max c and denominator d per latent
// in registers of the thread that owns the latent (TMEM lane = thread).  Per chunk, with the frame c_m = running
// max after the chunk and kappa = max_m c_m:
//
//   S^T = Q K_c^T                          MMA1  (128 x 128, k = 64)      latents on lanes, tokens on columns
//   E[m,t]   = exp(s[m,t] - c_m)           one exp per element, thread m scans its row
//   D[m,t]   = d_m + cumsum_t E[m,t]       (d_m already rescaled into the new frame)
//   R[m,t]   = E[m,t] exp(c_m - kappa) / D[m,t]        = softmax-numerator / encoder denominator
//   [W | Y | Den0] = R^T [E | U_bf16 | d]   MMA2  ONE product of width 208 (256 with two value blocks, Den0 separate):
//                                                  W = R^T E (tokens x tokens), Y = R^T U_bf16, Den0 = R^T d
//   W -> causal mask + bf16, written back to TMEM (token group)
//   U   += E V_c                           MMA3
//   Y   += tril(W) V_c                     MMA4  (A operand from TMEM)
//   y_t  = Y[t,:] / (Den0[t] + rowsum tril(W)[t,:])
//
// Operands E, R (written by the latent threads row-wise) feed MMAs both K-major and MN-major from the same
// 128-byte-swizzled buffers, so no transposition pass exists.  E, the bf16 copy of the state and the block whose
// column 0 is d lie behind one another in shared memory, so that they form ONE MN-major B operand and R is read once
// for all three products (28 MMA instructions per chunk at Dk = 64 instead of 44: every instruction costs 100-190
// cycles from issue to issue in this kernel whatever its width, 49-130 cycles alone).
//
// Warp roles (14 warps): 0-7 "latent group" (two warps per lane quarter, each half of the chunk's tokens): scores ->
// E, R, state rescale (chunk i+1);  8-11 "token group": causal mask of W, normalisation and store of Y (chunk i);
// 12: MMA issuer (one thread);  13: TMA producer (one thread).  The three stages work on consecutive chunks
// concurrently.  E and R have one buffer each (every product that reads them is issued when the latent group has
// finished the chunk; the latent group waits for the state update of the previous chunk before it writes E), the
// accumulators [W | Y | Den0] are single and go back to the MMA issuer as soon as the token group has them in
// registers, K is single-buffered (free as soon as its score MMA has run), V has two stages.
#include "prefill_tc.cuh"

#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "sm100_ptx.cuh"
#include "tc_device.cuh"

// polling rounds of every wait of the prefill kernel before it suspends (see tc::wait_or_abort)
#ifndef FLARE_TC_FWD_POLLS
#define FLARE_TC_FWD_POLLS 24
#endif

namespace flare {

using namespace sm100;

namespace {

constexpr int C = 128;    // tokens per chunk
constexpr int M = 128;    // latents
constexpr int D = 64;     // value columns per CTA, and width of one 128-byte operand block
constexpr int NTHREADS = 448;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// shared memory map (bytes, every operand buffer 1024-aligned for the 128B swizzle)
// DKB = Dk / 64 = number of 64-wide key blocks
// WIDE: one CTA handles both 64-column value blocks of Dv = 128 (Dk = 128 only), see the kernel's comment
template <int DKB, bool WIDE = false>
struct Lay {
  static_assert(!WIDE || DKB == 2, "the wide instance is the (128, 128) head shape");
  // Dk = 64: the latent bank stays in shared memory (TMA-loaded); Dk = 128 has no room for it there and keeps it in
  // tensor memory as the A operand of the score MMA
  static constexpr bool Q_SMEM = DKB == 1;
  // Every product that reads R (W, Y0, Den0) is ONE tcgen05.mma sequence over a B operand of adjacent 64-wide
  // MN-major blocks [E t-block 0 | E t-block 1 | U_bf16 ... | d], issued when the latent group has finished a chunk:
  // R is read once, and E and R need one buffer each (free long before the next chunk writes them).
  static constexpr int VB = WIDE ? 2 : 1;                  // 64-column value blocks per CTA
  static constexpr int OFF_Q = 0;                          // [128 m][64] bf16, K-major                 16 KB or 0
  static constexpr int OFF_K = Q_SMEM ? 16384 : 0;         // DKB x [128 t][64] bf16                    16 KB each
  static constexpr int OFF_V = OFF_K + DKB * 16384;        // 2 stages x [VB value blocks][128 t][64]   16 KB each
  static constexpr int OFF_E = OFF_V + 2 * VB * 16384;     // [2 t-blocks][128 m][64 t] bf16            32 KB
  // merged product: the bf16 state operand follows E directly; with one value block the denominator follows as a
  // fourth MN-major block [128 m][64] of which column 0 holds d (product width 128 + 64 + 16 = 208); with two value
  // blocks the width is 256 already and Den0 stays a product of its own over the small K-major d tile
  static constexpr int OFF_U = OFF_E + 32768;              // [VB][128 m][64 dv] bf16                    16 KB each
  static constexpr int OFF_B16 = OFF_U + VB * 16384;       // d: MN-major block 16 KB, or (wide) the K-major tile
                                                           // [2 m-blocks][16 n][64 m] 4 KB
  static constexpr int D_BYTES = WIDE ? 4096 : 16384;
  static constexpr int OFF_R = OFF_B16 + D_BYTES;          // [2 t-blocks][128 m][64 t] bf16              32 KB
  static constexpr int OFF_MISC = OFF_R + 32768;           // barriers, tmem slot, reductions          4608 B
  static constexpr int OFF_STAGE = OFF_MISC + 4608;        // 4 token warps x [32 t][32 columns] 16-bit: source of the
                                                           // read-out's bulk stores (64-byte swizzle)     8 KB
  // wide, two latent groups merged on chip: the partner CTA's normalised partial rows of the value block this CTA
  // finalises, [128 t][64] fp16 (16-byte pieces swizzled by row), and the log2 weight mass per row
  static constexpr int OFF_XCH = OFF_STAGE + 8192;         //                                          16 KB + 512 B
  static constexpr int SMEM_BYTES = OFF_XCH + (WIDE ? 16384 + 512 : 0) + 1024;  // + slack for manual 1024-byte alignment
  static_assert(SMEM_BYTES <= 232448, "shared memory");
  // tensor-memory columns.  [W | Y | Den] are adjacent (one product writes them); single accumulators, handed back by
  // the token group as soon as it has them in registers.  Wide: W shares the columns of S (the latent group has the
  // next chunk's scores in registers before W of this chunk is written) and U takes 128 columns.
  static constexpr uint32_t TM_S = 0, TM_W = WIDE ? 0 : 128, TM_Y = TM_W + 128, TM_DEN = WIDE ? 384 : TM_Y + 64,
                            TM_U = WIDE ? 256 : TM_DEN + 16, TM_Q = WIDE ? 400 : TM_U + 64 /* packed bf16 (Dk = 128 only) */;
  static_assert(TM_Q + (Q_SMEM ? 0 : DKB * 32) <= 512, "tensor memory columns");
};
constexpr uint32_t TM_COLS = 512;

struct Misc {
  uint64_t q_full, k_full, k_empty, v_full[2], v_empty[2];
  uint64_t s_ready, s_free, kap_done, p1_done, u_done, w_ready, p2_done, y_ready, y_free;
  uint64_t pmax[4], psum[4];  // pair barriers of the two latent half-groups, one per lane quarter
  uint64_t xfull[4], xfree[4];  // on-chip merge of two latent groups, per token warp: the partner's rows have arrived /
                                // the partner has read the rows this CTA sent
  uint32_t tmem_base;
  volatile int abort_flag;
  float wmax[2][4];
  float kap[4];  // decode frame of chunk i in slot i % 4, for the token group (log-sum-exp, weight mass of a latent group)
  float xmax[2][2][128], xsum[2][2][128];  // [chunk parity][half][latent]
};


// optional cycle trace of CTA (0, 0): [role][chunk < 16][slot < 8] clock64 stamps (diagnostic hook, null in normal use)
#define TC_TRACE(role, chunk, slot)                                                                   \
  do {                                                                                                \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (chunk) < 16)                   \
      p.trace[((role) * 16 + (chunk)) * 8 + (slot)] = clock64();                                      \
  } while (0)

using tc::swz_chunk_off;
using tc::warp_arrive;
using tc::sigma_fast;

// bounded wait that also gives up as soon as another role of the CTA has given up
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, Misc* misc) {
  return tc::wait_or_abort(bar, parity, &misc->abort_flag, FLARE_TC_FWD_POLLS);
}

// grid.z = latent group * DKB + value slice.  First value column of this CTA's slice (a compile-time zero when there
// is one slice) and first latent of its group (zero without the latent split).
template <int DVB, bool SPLIT>
__device__ __forceinline__ int value_col0() {
  return DVB == 1 ? 0 : (SPLIT ? (int)blockIdx.z % DVB : (int)blockIdx.z) * D;
}
template <int DVB, bool SPLIT>
__device__ __forceinline__ int latent0() {
  return SPLIT ? ((int)blockIdx.z / DVB) * M : 0;
}

}  // namespace

// The kernel instances are compiled in separate translation units (FLARE_TC_UNIT = 0..5: head widths (64, 64) / (128, 128) / (64, 128), without /
// with the latent-group split) to keep build times short; the unit without FLARE_TC_UNIT holds the host side.
template <int UNIT>
int launch_prefill_tc_unit(bool padded, int mode, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const CUtensorMap& ty, const TcParams& p, dim3 grid, cudaStream_t stream);

#ifdef FLARE_TC_UNIT


// PADDED: fewer than 128 latents (rows padded); the full-width instance carries none of the padding predicates
// SPLIT: more than 128 latents, partial read-outs
// BLOCK: block-causal (semi-autoregressive) read-out with blocks of 16, 32, 64 or 128 tokens: a token reads the state
//        at the end of its block, so the denominator of a block's tokens is the one at the block's end and the mask
//        of W is "column <= end of the row's block"
// MODE 2 (STABLE): stablemax encoder weights sigma(s) = (1+s)^p | (1-s)^-p.  The encoder side then has no frames
//        (E = sigma(s), D = plain running sum, the state is never rescaled); the decode weights stay a softmax over
//        the latents, whose numerator exp2(s - c) a_m is formed with the same running-max machinery as before.
// DVB = Dv / 64 = number of value slices (grid.z); Dv may differ from Dk (Dk = 64 with Dv = 128)
// KEEP: training forward that leaves the per-chunk prefix states for the backward pass (a separate instance: the
//       extra live values cost the register-capped latent group about 5 % when the code is merely present)
// WIDE: (Dk, Dv) = (128, 128) with ONE CTA per (lane, latent group) that carries all 128 value columns, instead of two
//       CTAs that each repeat the score / E / R work for 64 of them.  Used when the two-slice grid would not fit the
//       SMs in one wave.  Differences: U and Y are 128 columns wide; W and Y0 = R^T U_bf16 come out of ONE product of
//       width 256 ([E | U_bf16] as one B operand, [W | Y] adjacent in tensor memory), so R is read once for both; W
//       shares the columns of S; E and R are single-buffered.
template <bool PADDED, int DKB, int DVB, bool SPLIT, int MODE, bool KEEP, bool WIDE>
__global__ void __launch_bounds__(NTHREADS, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_y, const TcParams p) {
  using L = Lay<DKB, WIDE>;
  static_assert(!WIDE || (DVB == 2 && !PADDED), "wide instance");
  constexpr int ZS = WIDE ? 1 : DVB;  // value slices on grid.z
  constexpr bool BLOCK = MODE == 1, STABLE = MODE == 2;
  constexpr int OFF_K = L::OFF_K, OFF_V = L::OFF_V, OFF_E = L::OFF_E, OFF_R = L::OFF_R, OFF_U = L::OFF_U,
                OFF_B16 = L::OFF_B16, OFF_Q = L::OFF_Q, OFF_MISC = L::OFF_MISC, VB = L::VB, D_BYTES = L::D_BYTES;
  constexpr bool Q_SMEM = L::Q_SMEM;
  constexpr uint32_t TM_S = L::TM_S, TM_W = L::TM_W, TM_U = L::TM_U, TM_Y = L::TM_Y, TM_DEN = L::TM_DEN, TM_Q = L::TM_Q;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + OFF_MISC);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lane_id = blockIdx.x, seg = blockIdx.y;
  // This CTA's slice of the value columns starts at blockIdx.z * D (a compile-time zero when Dv = 64); the
  // roles read it where they need it instead of keeping it in a register across their chunk loops, because the
  // latent group runs at the register cap and an extra live value there cost 4 % of the kernel's time.
  constexpr int DV = DVB * D;
  const int b = lane_id / p.H, h = lane_id % p.H;
  const int seg_begin = seg * p.seg_len;
  // rows beyond the batch row's own length are right padding: they are not walked
  const int n_row = p.lens != nullptr ? min(p.N, max(0, p.lens[b])) : p.N;
  const int seg_end = max(seg_begin, min(n_row, seg_begin + p.seg_len));
  const int nchunks = (seg_end - seg_begin + C - 1) / C;

  if (tid == 0) {
    mbar_init(&misc->q_full, Q_SMEM ? 1 : 8);
    mbar_init(&misc->k_full, 1);
    mbar_init(&misc->k_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&misc->v_full[i], 1);
      mbar_init(&misc->v_empty[i], 1);
    }
    mbar_init(&misc->s_ready, 1);
    mbar_init(&misc->s_free, 8);
    mbar_init(&misc->kap_done, 4);
    mbar_init(&misc->p1_done, 8);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&misc->pmax[i], 2);
      mbar_init(&misc->psum[i], 2);
    }
    mbar_init(&misc->u_done, 1);
    mbar_init(&misc->w_ready, 1);
    mbar_init(&misc->p2_done, 4);
    mbar_init(&misc->y_ready, 1);
    mbar_init(&misc->y_free, 4);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&misc->xfull[i], 1);
      mbar_init(&misc->xfree[i], 32);
    }
    misc->abort_flag = 0;
    fence_barrier_init();
  }
  // zero the denominator operand tile once (rows 1..15 stay zero for the whole kernel)
  for (int i = tid; i < D_BYTES / 16; i += NTHREADS) reinterpret_cast<uint4*>(smem + OFF_B16)[i] = make_uint4(0, 0, 0, 0);

  if (warp == 12) {
    tmem_alloc(&misc->tmem_base, TM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // on-chip merge: the partner CTA arrives on this CTA's barriers, which must be initialised first
  const bool xmerge = WIDE && SPLIT && p.cluster_merge != 0;
  if (xmerge) cluster_sync_all();
  const uint32_t tmem = misc->tmem_base;
  bool ok = true;
  // No read-out wanted (segment states for a scan, prefix states): only E and U += E V are computed; R, W, the
  // read-out MMAs and the token group are skipped.
  const bool state_only = p.y == nullptr;

  if (warp == 13) {
    // ======================================= TMA producer =======================================
    if (lane == 0) {
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      if (Q_SMEM) {
        mbar_arrive_expect_tx(&misc->q_full, 16384);
        tma_load_3d(smem + OFF_Q, &tm_q, &misc->q_full, 0, latent0<ZS, SPLIT>(), h);  // rows beyond M read as zero
      }
      const int vc0 = value_col0<ZS, SPLIT>();
      for (int i = 0; ok && i < nchunks; ++i) {
        const int t0 = seg_begin + i * C;
        // K tile: free once the score MMA of the previous chunk has run
        if (i > 0 && !(ok = wait_or_abort(&misc->k_empty, (i - 1) & 1, misc))) break;
        mbar_arrive_expect_tx(&misc->k_full, DKB * 16384);
#pragma unroll
        for (int kb = 0; kb < DKB; ++kb) tma_load_4d(smem + OFF_K + kb * 16384, &tm_k, &misc->k_full, kb * 64, h, t0, b);
        // V tile: stage i & 1, free once chunk i - 2 has been folded into Y
        const int st = i & 1;
        if (i >= 2 && !(ok = wait_or_abort(&misc->v_empty[st], ((i - 2) >> 1) & 1, misc))) break;
        mbar_arrive_expect_tx(&misc->v_full[st], VB * 16384);
#pragma unroll
        for (int vb = 0; vb < VB; ++vb)
          tma_load_4d(smem + OFF_V + (st * VB + vb) * 16384, &tm_v, &misc->v_full[st], vc0 + vb * 64, h, t0, b);
      }
    }
  } else if (warp == 12) {
    // ======================================= MMA issuer =======================================
    if (lane == 0) {
      const uint32_t k_addr = smem_u32(smem + OFF_K);
      const uint32_t b16_addr = smem_u32(smem + OFF_B16);
      constexpr uint32_t ID_S = make_idesc_bf16(128, 128, 0, 0);   // Q (TMEM) x K_c (K-major)
      constexpr uint32_t ID_U = make_idesc_bf16(128, WIDE ? 128 : 64, 0, 1);  // E (K-major) x V (MN-major)
      constexpr uint32_t ID_DEN = make_idesc_bf16(128, 16, 1, 0);  // R (MN-major) x d tile (K-major)
      constexpr uint32_t ID_Y1 = make_idesc_bf16(128, WIDE ? 128 : 64, 0, 1);  // tril(W) (TMEM) x V (MN-major)
      // merged: R (MN-major) x [E | U_bf16 (| d)] (MN-major), width 256 with two value blocks, 208 with one
      constexpr uint32_t ID_WY = make_idesc_bf16(128, WIDE ? 256 : 208, 1, 1);

      // descriptors are built once; inside the loops only the start-address field (units of 16 bytes) advances
      const uint64_t dk = make_desc_sw128(k_addr, 16, 1024);
      const uint64_t dq = make_desc_sw128(smem_u32(smem + OFF_Q), 16, 1024);
      const uint64_t db16 = make_desc_sw128(b16_addr, 16, 1024);
      // second buffer of a double-buffered operand = first + its byte distance (in 16-byte units)
      const uint64_t de_k0 = make_desc_sw128(smem_u32(smem + OFF_E), 16, 1024);
      const uint64_t de_mn0 = make_desc_sw128(smem_u32(smem + OFF_E), 16384, 1024);
      const uint64_t dr_mn0 = make_desc_sw128(smem_u32(smem + OFF_R), 16384, 1024);
      // (wide: the two 64-column value blocks are 16384 bytes apart, the leading-dimension stride of the N = 128 operand)
      const uint64_t dv_mn0 = make_desc_sw128(smem_u32(smem + OFF_V), WIDE ? 16384 : 1024, 1024);
      constexpr int V_STAGE = VB * 16384;

      auto issue_scores = [&](int i) -> bool {  // S^T of chunk i; K tile and the S columns must be free
        if (!wait_or_abort(&misc->k_full, i & 1, misc)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 4 * DKB; ++j) {
          const uint64_t dkj = dk + (((j >> 2) * 16384 + (j & 3) * 32) >> 4);
          if (Q_SMEM) mma_ss(tmem + TM_S, dq + (j * 32 >> 4), dkj, ID_S, j > 0);
          else mma_ts(tmem + TM_S, tmem + TM_Q + j * 8, dkj, ID_S, j > 0);
        }
        tc_commit(&misc->s_ready);
        tc_commit(&misc->k_empty);
        return true;
      };
      auto issue_tail = [&](int i) -> bool {  // Y += tril(W) V of chunk i, after the token group masked W
        if (!wait_or_abort(&misc->p2_done, i & 1, misc)) return false;
        tc_fence_after_sync();
        const uint64_t dv = dv_mn0 + (uint64_t)((i & 1) * (V_STAGE >> 4));
#pragma unroll
        for (int j = 0; j < 8; ++j)
          mma_ts(tmem + TM_Y, tmem + TM_W + j * 8, dv + (j * 2048 >> 4), ID_Y1, 1);
        tc_commit(&misc->y_ready);
        tc_commit(&misc->v_empty[i & 1]);
        return true;
      };

      ok = wait_or_abort(&misc->q_full, 0, misc);  // the latent bank is in place
      tc_fence_after_sync();
      if (ok && nchunks > 0) ok = issue_scores(0);
      for (int i = 0; ok && i < nchunks; ++i) {
        const uint32_t par = i & 1;
        TC_TRACE(2, i, 0);
        // Next chunk's scores first: the latent group took S of chunk i long ago, while the token group is still
        // masking W of chunk i - 1, which the read-out product below waits for.  (Wide: the scores go into the columns
        // that hold the packed W of chunk i - 1 until that product has read them, so they come second there.)
        if (!WIDE && i + 1 < nchunks) {
          if (!(ok = wait_or_abort(&misc->s_free, par, misc))) break;
          if (!(ok = issue_scores(i + 1))) break;
        }
        TC_TRACE(2, i, 2);
        if (!state_only && i >= 1 && !(ok = issue_tail(i - 1))) break;
        TC_TRACE(2, i, 1);
        if (WIDE && i + 1 < nchunks) {
          // the latent group has read S of chunk i: the columns can take the next chunk's scores
          if (!(ok = wait_or_abort(&misc->s_free, par, misc))) break;
          if (!(ok = issue_scores(i + 1))) break;
        }
        if (!(ok = wait_or_abort(&misc->p1_done, par, misc))) break;
        if (!(ok = wait_or_abort(&misc->v_full[i & 1], (i >> 1) & 1, misc))) break;
        tc_fence_after_sync();
        TC_TRACE(2, i, 3);
        const uint64_t dek = de_k0, dem = de_mn0, drm = dr_mn0;
        const uint64_t dv = dv_mn0 + (uint64_t)((i & 1) * (V_STAGE >> 4));
        if (!state_only) {
          // Single-buffered accumulators: the token group must have taken Y of chunk i - 1.
          if (i >= 1) {
            if (!(ok = wait_or_abort(&misc->y_free, (i - 1) & 1, misc))) break;
            tc_fence_after_sync();
          }
          {
            // wide: W shares the columns of S: the latent group must have taken the next chunk's scores
            if (WIDE && i + 1 < nchunks) {
              if (!(ok = wait_or_abort(&misc->s_free, (i + 1) & 1, misc))) break;
              tc_fence_after_sync();
            }
            // [W | Y0 (| Den0)] = R^T [E | U_bf16 (| d)]: one product (k = latents); the B operand's four 64-wide blocks
            // lie 16384 bytes apart: the E t-blocks, then the two value blocks of the bf16 state, or its one value
            // block and the block whose column 0 is d
#pragma unroll
            for (int j = 0; j < 8; ++j) mma_ss(tmem + TM_W, drm + (j * 2048 >> 4), dem + (j * 2048 >> 4), ID_WY, j > 0);
            tc_commit(&misc->w_ready);
            TC_TRACE(2, i, 5);
            if constexpr (WIDE) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                mma_ss(tmem + TM_DEN, drm + (j * 2048 >> 4), db16 + (((j >> 2) * 2048 + (j & 3) * 32) >> 4), ID_DEN, j > 0);
            }
          }
          TC_TRACE(2, i, 6);
        }
        // U += E V_c  (k = tokens of the chunk)
#pragma unroll
        for (int j = 0; j < 8; ++j)
          mma_ss(tmem + TM_U, dek + (((j >> 2) * 16384 + (j & 3) * 32) >> 4), dv + (j * 2048 >> 4), ID_U, 1);
        tc_commit(&misc->u_done);
        if (state_only) tc_commit(&misc->v_empty[i & 1]);  // no read-out MMA will read this V stage
        TC_TRACE(2, i, 4);
      }
      if (!state_only && ok && nchunks > 0) ok = issue_tail(nchunks - 1);
    }
  } else if (warp < 8) {
    // ===================== latent group: 8 warps, thread = (latent = TMEM lane, half of the chunk's tokens) =====================
    // Warps q and q + 4 own the same 32 latents and split the 128 tokens of a chunk in halves, so that two warps
    // per scheduler overlap the special-function, ALU and FMA pipes.  The halves exchange the row maximum and the
    // row sum of E through shared memory.
    const int hf = warp >> 2, q = warp & 3;
    const uint32_t tl = tmem + ((uint32_t)(q * 32) << 16);
    const int m = q * 32 + lane;
    const float sc2 = p.scale * kLog2e;
    const int64_t st_idx = (int64_t)lane_id * p.in_lane_stride + (int64_t)seg * p.in_seg_stride;
    // Fewer than 128 latents: the missing rows are padding (zero rows of Q).  A padding latent gets the frame +inf,
    // so its E = exp2(0 - inf) is exactly zero without any predicate in the element loops, and a denominator of 1.
    const bool live = !PADDED || latent0<ZS, SPLIT>() + m < p.M;
    float c2 = -INFINITY, dsum = 0.f;  // running max (log2 units) and the denominator in that frame
    if (!live) {
      c2 = 0.f;
      dsum = 1.f;
    } else if (p.in_m != nullptr) {
      // (stablemax: the carried m is a constant zero and not a frame; the decode frame starts empty)
      if (!STABLE) c2 = p.in_m[st_idx * p.M + latent0<ZS, SPLIT>() + m] * kLog2e;
      dsum = p.in_d[st_idx * p.M + latent0<ZS, SPLIT>() + m];
    }
    float d_prev = 0.f;                                  // denominator before the chunk in flight, in its frame
    if constexpr (!Q_SMEM) {
      // latent bank row m -> tensor memory as packed bf16 (element k in column k / 2); each half-group thread
      // writes half of the row.  Rows beyond M are zero.
      uint32_t r[DKB * 16];
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.q) +
                                                        (int64_t)h * p.q_stride_h +
                                                        (int64_t)(live ? latent0<ZS, SPLIT>() + m : 0) * p.q_stride_m +
                                                        hf * (DKB * 32));
#pragma unroll
      for (int i = 0; i < DKB * 4; ++i) {
        const uint4 x = live ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
        r[4 * i] = x.x; r[4 * i + 1] = x.y; r[4 * i + 2] = x.z; r[4 * i + 3] = x.w;
      }
      static_assert(Q_SMEM || DKB == 2, "store width");
      tmem_st32(tl + TM_Q + hf * 32, r);
      tmem_wait_st();
      tc_fence_before_sync();
      warp_arrive(&misc->q_full, lane);
    }
    // columns of the numerator each half-group thread looks after: 32 of the CTA's 64, or (wide) 64 of its 128
    constexpr int UW = WIDE ? 64 : 32;
#pragma unroll
    for (int c0 = 0; c0 < UW; c0 += 32) {
      // carry-in numerator -> tensor memory
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i)
        r[i] = (p.in_u && live) ? __float_as_uint(p.in_u[(st_idx * p.M + latent0<ZS, SPLIT>() + m) * DV +
                                                         value_col0<ZS, SPLIT>() + hf * UW + c0 + i])
                                : 0u;
      tmem_st32(tl + TM_U + hf * UW + c0, r);
      tmem_wait_st();
    }

    for (int i = 0; ok && i < nchunks; ++i) {
      const uint32_t par = i & 1;
      const int nvalid = min(C, seg_end - (seg_begin + i * C));
      const int tok0 = hf * 64;
      uint8_t* e_row = smem + OFF_E + hf * 16384;  // t-block hf of the operand buffers
      uint8_t* r_row = smem + OFF_R + hf * 16384;
      if (!(ok = wait_or_abort(&misc->s_ready, par, misc))) break;
      tc_fence_after_sync();
      if (tid == 0) TC_TRACE(0, i, 0);
      // the 64 scores of this thread stay in registers for the whole chunk
      uint32_t ra[32], rb[32];
      tmem_ld32(tl + TM_S + tok0, ra);
      tmem_ld32(tl + TM_S + tok0 + 32, rb);
      // Frame of this chunk.  Chunk 0 exchanges the two halves' maxima synchronously (the carried frame may be
      // empty).  Later chunks use the running max through the PREVIOUS chunk, known without waiting (this bookkeeping
      // runs while the scores are on their way out of tensor memory); E may then exceed 1 by the growth of the max
      // inside one chunk, which fp32 / bf16 hold easily.  This chunk's own row maximum is taken along with the E pass
      // and enters the next chunk's frame.  The state is put into the exact running-max frame when it is written out.
      float c_new = c2;
      if (i > 0) {
        // bookkeeping of chunk i - 1: both halves' sums and maxima are published once its psum phase completed
        if (!(ok = wait_or_abort(&misc->psum[q], (i - 1) & 1, misc))) break;
        dsum = d_prev + (misc->xsum[par ^ 1][0][m] + misc->xsum[par ^ 1][1][m]);
        c_new = fmaxf(c2, fmaxf(misc->xmax[par ^ 1][0][m], misc->xmax[par ^ 1][1][m]));
      }
      tmem_wait_ld();
      tmem_fence_regs(ra);
      tmem_fence_regs(rb);
      tc_fence_before_sync();
      warp_arrive(&misc->s_free, lane);  // the S columns may take the next chunk's scores
      if (i == 0) {
        // row maximum over the valid tokens of this half, exchanged with the other half
        float cm0 = -INFINITY, cm2 = -INFINITY;
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          if (tok0 + k < nvalid) cm0 = fmaxf(cm0, __uint_as_float(ra[k]) * sc2);
          if (tok0 + 32 + k < nvalid) cm2 = fmaxf(cm2, __uint_as_float(rb[k]) * sc2);
        }
        misc->xmax[0][hf][m] = live ? fmaxf(cm0, cm2) : -INFINITY;
        warp_arrive(&misc->pmax[q], lane);
        if (!(ok = wait_or_abort(&misc->pmax[q], 0, misc))) break;
        c_new = fmaxf(c2, fmaxf(misc->xmax[0][0][m], misc->xmax[0][1][m]));
      }
      float alpha = STABLE ? 1.0f : ex2_approx(c2 - c_new);  // 0 when the old state is empty
      // kappa: common frame of the decode weights = max over latents of the running max.  Chunk 0 synchronises;
      // later chunks use the value published during the previous chunk (one chunk stale, which only changes a
      // per-token scale that cancels in y).  (Publishing behind the E pass and reading the value of two chunks before,
      // to take the warp reduction off the start of the chunk, measured 3 % slower: the E pass grew by more.)
      if (hf == 0) {  // (both half-groups hold the same frames: one of them publishes)
        float wm = live ? c_new : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
        // (Two slots suffice: the slot written now is read by the other warps at the top of the NEXT chunk and
        // rewritten at the top of the one after; a warp gets that far only after every warp has finished this chunk -
        // the state update it waits for follows the product that waits for all of them - and has 3 000 cycles of passes
        // of its own in between, while a reader needs a few hundred from the end of this chunk to its read.  Four
        // slots indexed by chunk % 4 measured 4 % slower: one more live value in a register-capped loop.)
        if (lane == 0) misc->wmax[par][q] = wm;
      }
      if (i == 0) {
        if (hf == 0 && lane == 0) mbar_arrive(&misc->kap_done);
        if (!(ok = wait_or_abort(&misc->kap_done, 0, misc))) break;
      }
      const float* wsrc = misc->wmax[i == 0 ? 0 : ((i - 1) & 1)];
      const float kappa = fmaxf(fmaxf(wsrc[0], wsrc[1]), fmaxf(wsrc[2], wsrc[3]));
      // ordered before the token group's read by the barrier chain
      if ((SPLIT || BLOCK || p.lse_dec != nullptr) && tid == 0) misc->kap[i & 3] = kappa;
      if (tid == 0) TC_TRACE(0, i, 1);
      float a_m = ex2_approx(c_new - kappa);
      float d_carry = dsum * alpha;  // denominator of the carried state in the new frame
      if (PADDED && !live) {
        c_new = INFINITY;
        alpha = 1.0f;
        a_m = 0.f;
        d_carry = 1.0f;
      }
      c2 = c_new;
      // phase a: E for the 64 tokens of this half (in place of the scores), their sum, E operand rows
      float tot0 = 0.f, tot1 = 0.f;
      float g16[4] = {0.f, 0.f, 0.f, 0.f};  // BLOCK: sums of the four groups of 16 tokens of this half
      // this half's row maximum of s - c_new (log2 units), taken along with the pass
      float cma = -INFINITY, cmb = -INFINITY;
      // single E / R buffers: the products that read the previous chunk's E and R (they are all issued together and
      // the state update comes last) must have run
      if (STABLE && i > 0) {
        if (!(ok = wait_or_abort(&misc->u_done, (i - 1) & 1, misc))) break;
        tc_fence_after_sync();
      }
      if constexpr (STABLE) {
        // encoder weights sigma(s): packed and stored 8 tokens at a time; the raw scores stay in ra / rb for phase b
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float sg[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float raw = __uint_as_float(ch < 4 ? ra[ch * 8 + j] : rb[(ch - 4) * 8 + j]);
            if (tok0 + ch * 8 + j < nvalid) cma = fmaxf(cma, raw * sc2 - c_new);
            sg[j] = (tok0 + ch * 8 + j < nvalid) ? sigma_fast(raw * p.scale, p.power) : 0.f;
            tot0 += sg[j];
          }
          *reinterpret_cast<uint4*>(e_row + swz_chunk_off(m, ch)) =
              make_uint4(pack_bf16(sg[0], sg[1]), pack_bf16(sg[2], sg[3]), pack_bf16(sg[4], sg[5]), pack_bf16(sg[6], sg[7]));
        }
      } else if (nvalid == C) {
        // two tokens per FMA / add instruction (packed fp32 pairs): the passes are bound by instruction issue
        const uint64_t sc2p = f2_pack(sc2, sc2), cnp = f2_pack(-c_new, -c_new);
        uint64_t sa[2] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)}, sb[2] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};
#pragma unroll
        for (int k = 0; k < 32; k += 2) {
          float xa0, xa1, xb0, xb1;
          f2_unpack(f2_fma(f2_pack(__uint_as_float(ra[k]), __uint_as_float(ra[k + 1])), sc2p, cnp), xa0, xa1);
          f2_unpack(f2_fma(f2_pack(__uint_as_float(rb[k]), __uint_as_float(rb[k + 1])), sc2p, cnp), xb0, xb1);
          cma = fmax3(cma, xa0, xa1);
          cmb = fmax3(cmb, xb0, xb1);
          const float ea0 = ex2_approx(xa0), ea1 = ex2_approx(xa1), eb0 = ex2_approx(xb0), eb1 = ex2_approx(xb1);
          ra[k] = __float_as_uint(ea0);
          ra[k + 1] = __float_as_uint(ea1);
          rb[k] = __float_as_uint(eb0);
          rb[k + 1] = __float_as_uint(eb1);
          sa[BLOCK ? (k >> 4) : 0] = f2_add(sa[BLOCK ? (k >> 4) : 0], f2_pack(ea0, ea1));
          sb[BLOCK ? (k >> 4) : 0] = f2_add(sb[BLOCK ? (k >> 4) : 0], f2_pack(eb0, eb1));
        }
        float lo, hi;
        if (BLOCK) {
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            f2_unpack(sa[g], lo, hi);
            g16[g] = lo + hi;
            f2_unpack(sb[g], lo, hi);
            g16[2 + g] = lo + hi;
          }
        } else {
          f2_unpack(sa[0], lo, hi);
          tot0 = lo + hi;
          f2_unpack(sb[0], lo, hi);
          tot1 = lo + hi;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          const float x0 = __uint_as_float(ra[k]) * sc2 - c_new, x1 = __uint_as_float(rb[k]) * sc2 - c_new;
          if (tok0 + k < nvalid) cma = fmaxf(cma, x0);
          if (tok0 + 32 + k < nvalid) cmb = fmaxf(cmb, x1);
          const float e0 = (tok0 + k < nvalid) ? ex2_approx(x0) : 0.f;
          const float e1 = (tok0 + 32 + k < nvalid) ? ex2_approx(x1) : 0.f;
          ra[k] = __float_as_uint(e0);
          rb[k] = __float_as_uint(e1);
          if (BLOCK) {
            g16[k >> 4] += e0;
            g16[2 + (k >> 4)] += e1;
          } else {
            tot0 += e0;
            tot1 += e1;
          }
        }
      }
      if (BLOCK) {
        tot0 = g16[0] + g16[1];
        tot1 = g16[2] + g16[3];
      }
      misc->xsum[par][hf][m] = tot0 + tot1;
      // (chunk 0 published its maximum before the pass; an empty half stays at -inf)
      if (i > 0) misc->xmax[par][hf][m] = live ? fmaxf(cma, cmb) + c_new : -INFINITY;
      if (!(tot0 + tot1 < 1.15e18f)) {
        // the running max grew by more than 60 powers of two inside one chunk (the frame is the max through the
        // previous chunk): the denominators of this row leave the range in which the read-out weights are safe, see
        // the token group's check; an overflow (or a NaN) lands here as well.  Outside the numeric domain of this path.
        atomicOr(p.err, 2);
        if (p.gate != nullptr) {
          p.gate[0] = 1;
          p.gate[1 + lane_id] = 1;
        }
      }
      warp_arrive(&misc->psum[q], lane);
      // E has one buffer: the products that read the previous chunk's E and R (issued together, the state update last)
      // must have run.  (Storing inside the pass would need this wait before it, where it is not yet satisfied.)
      if (!STABLE && i > 0) {
        if (!(ok = wait_or_abort(&misc->u_done, (i - 1) & 1, misc))) break;
        tc_fence_after_sync();
      }
      if constexpr (!STABLE)
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        *reinterpret_cast<uint4*>(e_row + swz_chunk_off(m, ch)) =
            make_uint4(pack_bf16(__uint_as_float(ra[ch * 8 + 0]), __uint_as_float(ra[ch * 8 + 1])),
                       pack_bf16(__uint_as_float(ra[ch * 8 + 2]), __uint_as_float(ra[ch * 8 + 3])),
                       pack_bf16(__uint_as_float(ra[ch * 8 + 4]), __uint_as_float(ra[ch * 8 + 5])),
                       pack_bf16(__uint_as_float(ra[ch * 8 + 6]), __uint_as_float(ra[ch * 8 + 7])));
        *reinterpret_cast<uint4*>(e_row + swz_chunk_off(m, 4 + ch)) =
            make_uint4(pack_bf16(__uint_as_float(rb[ch * 8 + 0]), __uint_as_float(rb[ch * 8 + 1])),
                       pack_bf16(__uint_as_float(rb[ch * 8 + 2]), __uint_as_float(rb[ch * 8 + 3])),
                       pack_bf16(__uint_as_float(rb[ch * 8 + 4]), __uint_as_float(rb[ch * 8 + 5])),
                       pack_bf16(__uint_as_float(rb[ch * 8 + 6]), __uint_as_float(rb[ch * 8 + 7])));
      }
      d_prev = d_carry;
      // the upper half continues the lower half's running denominator; the lower half needs nothing from its partner
      // (except for blocks of 128 tokens, whose end lies in the upper half)
      float run = d_carry;
      if (!state_only && (hf || (BLOCK && p.block == 128))) {
        if (!(ok = wait_or_abort(&misc->psum[q], par, misc))) break;
        run += misc->xsum[par][0][m];
        if (BLOCK && p.block == 128 && hf == 0) run = d_carry;  // lower half: only the wait was needed
      }
      if (tid == 0) TC_TRACE(0, i, 2);
      if (state_only) {
        // no read-out: R is not needed
      } else if constexpr (STABLE) {
        // phase b, stablemax: D = running sum of sigma (recomputed), decode numerator exp2(s - c) a_m, R = numerator / D
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          uint32_t rp[16];
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            const float s0 = __uint_as_float(blk ? rb[k] : ra[k]), s1 = __uint_as_float(blk ? rb[k + 1] : ra[k + 1]);
            const int tk = tok0 + blk * 32 + k;
            run += (tk < nvalid) ? sigma_fast(s0 * p.scale, p.power) : 0.f;
            const float r0 = ex2_approx(s0 * sc2 - c_new) * (a_m * rcp_approx(run));
            run += (tk + 1 < nvalid) ? sigma_fast(s1 * p.scale, p.power) : 0.f;
            const float r1 = ex2_approx(s1 * sc2 - c_new) * (a_m * rcp_approx(run));
            rp[k >> 1] = pack_bf16(r0, r1);
          }
#pragma unroll
          for (int ch = 0; ch < 4; ++ch)
            *reinterpret_cast<uint4*>(r_row + swz_chunk_off(m, blk * 4 + ch)) =
                make_uint4(rp[ch * 4], rp[ch * 4 + 1], rp[ch * 4 + 2], rp[ch * 4 + 3]);
        }
      } else if constexpr (!BLOCK) {
        // phase b: D = running denominator, R = E a_m / D, R operand rows.  Reciprocals run on the special-function
        // unit (25-35 % busy); a Newton reciprocal on the FMA pipe for every other element cost 1-9 % of the kernel
        // depending on the box, and carrying the denominator pre-divided by a_m (one FMA + reciprocal + multiply per
        // element) measured 1.5 % slower than this form.
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          uint32_t rp[16];
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            const float e0 = __uint_as_float(blk ? rb[k] : ra[k]);
            const float e1 = __uint_as_float(blk ? rb[k + 1] : ra[k + 1]);
            run += e0;
            const float i0 = rcp_approx(run);
            run += e1;
            const float i1 = rcp_approx(run);
            float r0, r1;  // e * (a_m / D), two tokens per multiply
            f2_unpack(f2_mul(f2_pack(e0, e1), f2_mul(f2_pack(i0, i1), f2_pack(a_m, a_m))), r0, r1);
            rp[k >> 1] = pack_bf16(r0, r1);
          }
#pragma unroll
          for (int ch = 0; ch < 4; ++ch)
            *reinterpret_cast<uint4*>(r_row + swz_chunk_off(m, blk * 4 + ch)) =
                make_uint4(rp[ch * 4], rp[ch * 4 + 1], rp[ch * 4 + 2], rp[ch * 4 + 3]);
        }
      } else {
        // phase b, block-causal: the denominator of a token is the one at the end of its block.  dend[g] is that
        // value for the g-th group of 16 tokens of this half (`run` = denominator before this half).
        const int bs = p.block;
        float dend[4];
        {
          const float p0 = run + g16[0], p1 = p0 + g16[1], p2 = p1 + g16[2], p3 = p2 + g16[3];
          if (bs == 16) {
            dend[0] = p0; dend[1] = p1; dend[2] = p2; dend[3] = p3;
          } else if (bs == 32) {
            dend[0] = dend[1] = p1; dend[2] = dend[3] = p3;
          } else if (bs == 64) {
            dend[0] = dend[1] = dend[2] = dend[3] = p3;
          } else {
            // one block per chunk: both halves use the chunk's end
            const float whole = d_carry + (misc->xsum[par][0][m] + misc->xsum[par][1][m]);
            dend[0] = dend[1] = dend[2] = dend[3] = whole;
          }
        }
        // log normaliser after each block that ends in this half (natural log, exact-frame independent)
        if (p.lse_enc != nullptr && live && value_col0<ZS, SPLIT>() == 0) {
          const int t_half = seg_begin + i * C + tok0;  // first token of this half in the sequence
          float* dst = p.lse_enc + ((int64_t)lane_id * (p.N / bs)) * p.M + latent0<ZS, SPLIT>() + m;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int t_end = t_half + g * 16 + 15;            // last token of the group
            const bool ends = ((t_end + 1) % bs) == 0;         // a block ends with this group
            if (ends && tok0 + g * 16 < nvalid) dst[(int64_t)(t_end / bs) * p.M] = (c_new + __log2f(dend[g])) * kLn2;
          }
        }
        float inv[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) inv[g] = a_m * rcp_approx(dend[g]);
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          uint32_t rp[16];
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            const float w = inv[blk * 2 + (k >> 4)];
            float r0, r1;
            f2_unpack(f2_mul(f2_pack(__uint_as_float(blk ? rb[k] : ra[k]), __uint_as_float(blk ? rb[k + 1] : ra[k + 1])),
                             f2_pack(w, w)), r0, r1);
            rp[k >> 1] = pack_bf16(r0, r1);
          }
#pragma unroll
          for (int ch = 0; ch < 4; ++ch)
            *reinterpret_cast<uint4*>(r_row + swz_chunk_off(m, blk * 4 + ch)) =
                make_uint4(rp[ch * 4], rp[ch * 4 + 1], rp[ch * 4 + 2], rp[ch * 4 + 3]);
        }
      }
      if (tid == 0) TC_TRACE(0, i, 3);
      // state part: needs the numerator update of the previous chunk to have landed (waited for before the E rows
      // were written)
      if (tid == 0) TC_TRACE(0, i, 4);
      if (hf == 0 && !state_only) {
        // d of the carried state: column 0 of row m of the MN-major block (merged product with one value block), or
        // element m of row 0 of the small K-major tile
        if (!WIDE)
          *reinterpret_cast<__nv_bfloat16*>(smem + OFF_B16 + swz_chunk_off(m, 0)) = __float2bfloat16_rn(d_carry);
        else
          *reinterpret_cast<__nv_bfloat16*>(smem + OFF_B16 + (m >> 6) * 2048 + ((m & 63) >> 3) * 16 + (m & 7) * 2) =
              __float2bfloat16_rn(d_carry);
      }
      const bool need = __any_sync(0xffffffffu, alpha != 1.0f);
      if constexpr (WIDE) {
        // 64 value columns per thread = value block hf of the bf16 state operand (free: the products that read it
        // were issued before the state update this thread has just waited for)
        if (!state_only || need) {
#pragma unroll
          for (int c0 = 0; c0 < 64; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tl + TM_U + hf * 64 + c0, r);
            tmem_wait_ld();
            tmem_fence_regs(r);
            if (need) {
#pragma unroll
              for (int k = 0; k < 32; k += 2) {
                float u0, u1;
                f2_unpack(f2_mul(f2_pack(__uint_as_float(r[k]), __uint_as_float(r[k + 1])), f2_pack(alpha, alpha)), u0, u1);
                r[k] = __float_as_uint(u0);
                r[k + 1] = __float_as_uint(u1);
              }
              tmem_st32(tl + TM_U + hf * 64 + c0, r);
            }
            if (!state_only) {
#pragma unroll
              for (int ch = 0; ch < 4; ++ch) {
                uint4 v;
                v.x = pack_bf16(__uint_as_float(r[ch * 8 + 0]), __uint_as_float(r[ch * 8 + 1]));
                v.y = pack_bf16(__uint_as_float(r[ch * 8 + 2]), __uint_as_float(r[ch * 8 + 3]));
                v.z = pack_bf16(__uint_as_float(r[ch * 8 + 4]), __uint_as_float(r[ch * 8 + 5]));
                v.w = pack_bf16(__uint_as_float(r[ch * 8 + 6]), __uint_as_float(r[ch * 8 + 7]));
                *reinterpret_cast<uint4*>(smem + OFF_U + hf * 16384 + swz_chunk_off(m, (c0 >> 3) + ch)) = v;
              }
              if constexpr (KEEP) {
                // training: the state before this chunk in the exact running-max frame through it (see below)
                if (c0 == 0 && !(ok = wait_or_abort(&misc->psum[q], par, misc))) break;
                float fin = 1.0f, c_true = c2;
                if (!STABLE) {
                  c_true = fmaxf(c2, fmaxf(misc->xmax[par][0][m], misc->xmax[par][1][m]));
                  fin = ex2_approx(c2 - c_true);
                }
                const int64_t o = ((int64_t)lane_id * p.dump_nch + (seg_begin / C + i)) * p.M + latent0<ZS, SPLIT>() + m;
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.dump_u) + o * DV + hf * 64 + c0);
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                  uint4 v;
                  v.x = pack_bf16(__uint_as_float(r[ch * 8 + 0]) * fin, __uint_as_float(r[ch * 8 + 1]) * fin);
                  v.y = pack_bf16(__uint_as_float(r[ch * 8 + 2]) * fin, __uint_as_float(r[ch * 8 + 3]) * fin);
                  v.z = pack_bf16(__uint_as_float(r[ch * 8 + 4]) * fin, __uint_as_float(r[ch * 8 + 5]) * fin);
                  v.w = pack_bf16(__uint_as_float(r[ch * 8 + 6]) * fin, __uint_as_float(r[ch * 8 + 7]) * fin);
                  dst[ch] = v;
                }
                if (hf == 0 && c0 == 0) {
                  p.dump_c[o] = c_true;
                  p.dump_d[o] = d_carry * fin;
                }
              }
            }
          }
          if (!ok) break;
          if (need) tmem_wait_st();
        }
      } else
      if (!state_only || need) {
        uint32_t r[32];
        tmem_ld32(tl + TM_U + hf * 32, r);
        tmem_wait_ld();
        tmem_fence_regs(r);
        if (need) {
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            float u0, u1;
            f2_unpack(f2_mul(f2_pack(__uint_as_float(r[k]), __uint_as_float(r[k + 1])), f2_pack(alpha, alpha)), u0, u1);
            r[k] = __float_as_uint(u0);
            r[k + 1] = __float_as_uint(u1);
          }
          tmem_st32(tl + TM_U + hf * 32, r);
        }
        if (!state_only) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[ch * 8 + 0]), __uint_as_float(r[ch * 8 + 1]));
            v.y = pack_bf16(__uint_as_float(r[ch * 8 + 2]), __uint_as_float(r[ch * 8 + 3]));
            v.z = pack_bf16(__uint_as_float(r[ch * 8 + 4]), __uint_as_float(r[ch * 8 + 5]));
            v.w = pack_bf16(__uint_as_float(r[ch * 8 + 6]), __uint_as_float(r[ch * 8 + 7]));
            *reinterpret_cast<uint4*>(smem + OFF_U + swz_chunk_off(m, hf * 4 + ch)) = v;
          }
          if constexpr (KEEP) {
            // Training: the state before this chunk is kept for the backward pass, in the EXACT running-max frame
            // through this chunk (= the frame the next chunk will use), so that the backward's encoder weights of
            // the chunk never exceed 1.  Both halves' maxima of this chunk are published once its psum phase completed.
            if (!(ok = wait_or_abort(&misc->psum[q], par, misc))) break;
            float fin = 1.0f, c_true = c2;
            if (!STABLE) {
              c_true = fmaxf(c2, fmaxf(misc->xmax[par][0][m], misc->xmax[par][1][m]));
              fin = ex2_approx(c2 - c_true);
            }
            if (live) {
              const int64_t o = ((int64_t)lane_id * p.dump_nch + (seg_begin / C + i)) * p.M + latent0<ZS, SPLIT>() + m;
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.dump_u) + o * DV +
                                                    value_col0<ZS, SPLIT>() + hf * 32);
#pragma unroll
              for (int ch = 0; ch < 4; ++ch) {
                uint4 v;
                v.x = pack_bf16(__uint_as_float(r[ch * 8 + 0]) * fin, __uint_as_float(r[ch * 8 + 1]) * fin);
                v.y = pack_bf16(__uint_as_float(r[ch * 8 + 2]) * fin, __uint_as_float(r[ch * 8 + 3]) * fin);
                v.z = pack_bf16(__uint_as_float(r[ch * 8 + 4]) * fin, __uint_as_float(r[ch * 8 + 5]) * fin);
                v.w = pack_bf16(__uint_as_float(r[ch * 8 + 6]) * fin, __uint_as_float(r[ch * 8 + 7]) * fin);
                dst[ch] = v;
              }
              if (hf == 0 && value_col0<ZS, SPLIT>() == 0) {
                p.dump_c[o] = c_true;          // log2 units (unused for the stablemax encoder)
                p.dump_d[o] = d_carry * fin;   // denominator before the chunk in that frame
              }
            }
          }
        }
        if (need) tmem_wait_st();
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      warp_arrive(&misc->p1_done, lane);
      if (tid == 0) TC_TRACE(0, i, 5);
    }
    // carry-out state
    if (ok && p.out_u != nullptr && (p.out_mode == 1 || (p.out_mode == 2 && seg == p.nseg_total - 1))) {
      float fin = 1.0f;  // factor from the last chunk's frame to the exact running-max frame
      if (nchunks > 0) {
        const int lp = (nchunks - 1) & 1;
        ok = wait_or_abort(&misc->u_done, lp, misc) && wait_or_abort(&misc->psum[q], lp, misc);
        if (ok) {
          dsum = d_prev + (misc->xsum[lp][0][m] + misc->xsum[lp][1][m]);
          if (!STABLE) {
            const float c_true = fmaxf(c2, fmaxf(misc->xmax[lp][0][m], misc->xmax[lp][1][m]));
            fin = ex2_approx(c2 - c_true);
            c2 = c_true;
          }
        }
      }
      tc_fence_after_sync();
      if (ok) {
        const int64_t so = (int64_t)lane_id * p.out_lane_stride + (int64_t)seg * p.out_seg_stride;
        const int mg = latent0<ZS, SPLIT>() + m;  // latent index in the whole bank
        if (hf == 0 && live && value_col0<ZS, SPLIT>() == 0) {
          p.out_m[so * p.M + mg] = STABLE ? 0.f : c2 * kLn2;
          p.out_d[so * p.M + mg] = dsum * fin;
        }
#pragma unroll
        for (int c0 = 0; c0 < UW; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(tl + TM_U + hf * UW + c0, r);
          tmem_wait_ld();
          tmem_fence_regs(r);
          float4* dst = reinterpret_cast<float4*>(p.out_u + (so * p.M + (live ? mg : 0)) * DV +
                                                  value_col0<ZS, SPLIT>() + hf * UW + c0);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            if (live) dst[k] = make_float4(__uint_as_float(r[4 * k]) * fin, __uint_as_float(r[4 * k + 1]) * fin,
                                 __uint_as_float(r[4 * k + 2]) * fin, __uint_as_float(r[4 * k + 3]) * fin);
        }
      }
    }
  } else {
    // ============================ token group: thread = token of the chunk = TMEM lane ============================
    const int wq = warp - 8;  // lane quarter
    const uint32_t tl = tmem + ((uint32_t)(wq * 32) << 16);
    const int tt = wq * 32 + lane;  // token index inside the chunk
    uint8_t* const stage = smem + L::OFF_STAGE + wq * 2048;
    // latent-group split: dense fp16 partials [group][B][N][H][DV] and log2 weight masses [group][B][N][H]
    const int64_t part_row0 = SPLIT ? (((int64_t)(blockIdx.z / ZS) * (gridDim.x / p.H) + b) * p.N) : 0;
    for (int i = 0; !state_only && ok && i < nchunks; ++i) {
      const uint32_t par = i & 1;
      const int t0 = seg_begin + i * C;
      const int nvalid = min(C, seg_end - t0);
      // causal mask of W, bf16 pack, row sums
      if (!(ok = wait_or_abort(&misc->w_ready, par, misc))) break;
      tc_fence_after_sync();
      // This chunk's decode frame, taken now: the latent group is one to two chunks ahead and reuses the slot four
      // chunks on (read late, in the epilogue, from a two-slot array, a slow token group saw a later chunk's frame:
      // wrong weight masses for the merge of latent groups)
      const float kap_i = misc->kap[i & 3];
      if (tid == 256) TC_TRACE(1, i, 0);
      uint64_t rs2 = f2_pack(0.f, 0.f);  // row sum of the bf16-rounded masked W (the values the read-out MMA multiplies), as a pair of partial sums
      // last column (token of the chunk) this row may see: itself, or the end of its block
      const int be = BLOCK ? (tt | (p.block - 1)) : tt;
#pragma unroll 1
      for (int j = 0; j < 4; ++j) {
        uint32_t wp[16];
        if (BLOCK ? (j * 32 <= be) : (j <= wq)) {
          uint32_t r[32];
          tmem_ld32(tl + TM_W + j * 32, r);
          tmem_wait_ld();
          if (BLOCK ? (j * 32 + 31 <= be) : (j < wq)) {
            // the whole 32-column block is visible to every row of this warp
#pragma unroll
            for (int k = 0; k < 32; k += 2) {
              const uint32_t pk = pack_bf16(__uint_as_float(r[k]), __uint_as_float(r[k + 1]));
              wp[k >> 1] = pk;
              rs2 = f2_add(rs2, f2_pack(__uint_as_float(pk << 16), __uint_as_float(pk & 0xffff0000u)));
            }
          } else {
#pragma unroll
            for (int k = 0; k < 32; k += 2) {
              const float w0 = (BLOCK ? (j * 32 + k <= be) : (k <= lane)) ? __uint_as_float(r[k]) : 0.f;
              const float w1 = (BLOCK ? (j * 32 + k + 1 <= be) : (k + 1 <= lane)) ? __uint_as_float(r[k + 1]) : 0.f;
              const uint32_t pk = pack_bf16(w0, w1);
              wp[k >> 1] = pk;
              rs2 = f2_add(rs2, f2_pack(__uint_as_float(pk << 16), __uint_as_float(pk & 0xffff0000u)));
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < 16; ++k) wp[k] = 0u;
        }
        tmem_st16(tl + TM_W + j * 16, wp);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      warp_arrive(&misc->p2_done, lane);
      if (tid == 256) TC_TRACE(1, i, 1);

      // normalise and store (wide: the first of the two value blocks; two accumulator phases per chunk)
      if (!(ok = wait_or_abort(&misc->y_ready, par, misc))) break;
      tc_fence_after_sync();
      if (tid == 256) TC_TRACE(1, i, 2);
      uint32_t den0;
      tmem_ld1(tl + TM_DEN, den0);
      tmem_wait_ld();
      float rs_lo, rs_hi;
      f2_unpack(rs2, rs_lo, rs_hi);
      const float den = __uint_as_float(den0) + (rs_lo + rs_hi);
      // Numeric domain of this path.  The read-out weight of (token, latent) is R = E a_m / D: it is flushed to zero
      // below 2^-126, while what it stands for, R D = the token's decode weight in the frame kappa, may still matter
      // when the whole token's weight mass is small.  With the row denominators held below 2^60 (checked by the latent
      // group) a flushed weight is below 2^-66, so a token whose mass is at least 2^-40 loses nothing it can see in
      // bf16; below that, or with a mass that overflowed or is not a number, the token is flagged and the exact path,
      // which has no such limit, redoes its lane.  With several latent groups each group's own mass is held to this
      // (the frames differ between groups, so a group that looks empty in its own frame may carry the token).
      const bool den_ok = den >= 9.1e-13f && den < INFINITY;
      if (tt < nvalid && !den_ok) {
        atomicOr(p.err, 2);
        if (p.gate != nullptr) {
          p.gate[0] = 1;
          p.gate[1 + lane_id] = 1;
        }
      }
      const float inv = (SPLIT && !den_ok) ? 0.f : rcp_approx(den);  // (a true division compiles to a call here)
      if (SPLIT && !xmerge && p.part_y != nullptr && tt < nvalid && value_col0<ZS, SPLIT>() == 0)
        p.part_lw[(part_row0 + t0 + tt) * p.H + h] = den_ok ? kap_i + __log2f(den) : -INFINITY;
      // log-sum-exp of the token's decode scores = log of the decode weights' mass in the frame kappa
      if (!SPLIT && p.lse_dec != nullptr && tt < nvalid && value_col0<ZS, SPLIT>() == 0)
        p.lse_dec[(int64_t)lane_id * p.N + t0 + tt] = (kap_i + __log2f(den)) * kLn2;
      if constexpr (WIDE && SPLIT) {
        if (xmerge) {
          // Two latent groups = two CTAs of a cluster.  CTA r finalises value block r: it sends its normalised
          // partial of the OTHER block (fp16) and the log2 of its weight mass into the partner's shared memory,
          // takes the partner's rows for its own block, and stores y = sum_g w_g y_g / sum_g w_g.
          const uint32_t rank = cluster_ctarank(), peer = rank ^ 1u;
          const float lw_own = den_ok ? kap_i + __log2f(den) : -INFINITY;
          uint32_t ra[32], rb[32], pk[32];
          // The exchange tile was the source of the previous chunk's bulk stores: once they have read it the partner
          // may send this chunk's rows (32 rows x 128 bytes and 32 weight masses per warp), which the barrier counts.
          if (lane == 0) {
            bulk_wait_group_read0();
            mbar_arrive_expect_tx(&misc->xfull[wq], 4096 + 128);
          }
          __syncwarp();
          if (i > 0) mbar_arrive_cluster_relaxed(mapa_shared(smem_u32(&misc->xfree[wq]), peer));
          // the partner's block, normalised, as fp16 pairs; then this CTA's block; the accumulator is free again
          tmem_ld32(tl + TM_Y + peer * 64, ra);
          tmem_ld32(tl + TM_Y + peer * 64 + 32, rb);
          tmem_wait_ld();
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const uint64_t inv2 = f2_pack(inv, inv);
            float a0, a1, b0, b1;
            f2_unpack(f2_mul(f2_pack(__uint_as_float(ra[2 * k]), __uint_as_float(ra[2 * k + 1])), inv2), a0, a1);
            f2_unpack(f2_mul(f2_pack(__uint_as_float(rb[2 * k]), __uint_as_float(rb[2 * k + 1])), inv2), b0, b1);
            pk[k] = pack_f16(a0, a1);
            pk[16 + k] = pack_f16(b0, b1);
          }
          tmem_ld32(tl + TM_Y + rank * 64, ra);
          tmem_ld32(tl + TM_Y + rank * 64 + 32, rb);
          tmem_wait_ld();
          tc_fence_before_sync();
          warp_arrive(&misc->y_free, lane);
          // (1) send: the rows sent for chunk i - 1 must have been read by the partner.  The stores are asynchronous and
          // count their bytes on the partner's barrier: plain remote stores followed by a releasing arrive cost 1600
          // cycles per chunk here.  Every thread sends the eight 16-byte pieces of its row, in the tile's layout.
          if (i > 0 && !(ok = tc::wait_or_abort_cluster(&misc->xfree[wq], (i - 1) & 1, &misc->abort_flag))) break;
          {
            const uint32_t xw = mapa_shared(smem_u32(smem + L::OFF_XCH + wq * 4096), peer);
            const uint32_t xbar = mapa_shared(smem_u32(&misc->xfull[wq]), peer);
#pragma unroll
            for (int half = 0; half < 2; ++half)
#pragma unroll
              for (int ch = 0; ch < 4; ++ch)
                st_async_v4(xw + half * 2048 + lane * 64 + ((ch ^ ((lane >> 1) & 3)) << 4),
                            make_uint4(pk[half * 16 + ch * 4], pk[half * 16 + ch * 4 + 1], pk[half * 16 + ch * 4 + 2],
                                       pk[half * 16 + ch * 4 + 3]), xbar);
            st_async_b32(mapa_shared(smem_u32(smem + L::OFF_XCH + 16384 + tt * 4), peer), __float_as_uint(lw_own), xbar);
          }
          if (tid == 256) TC_TRACE(1, i, 4);
          // (2) receive the partner's rows of this CTA's block
          if (!(ok = tc::wait_or_abort_cluster(&misc->xfull[wq], par, &misc->abort_flag))) break;
          if (tid == 256) TC_TRACE(1, i, 5);
          const float lw_p = *reinterpret_cast<const float*>(smem + L::OFF_XCH + 16384 + tt * 4);
          uint4 xp[8];
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)  // [warp][32-column half][32 rows x 64 bytes, 16-byte pieces swizzled as in the staging tile]
            xp[ch] = *reinterpret_cast<const uint4*>(smem + L::OFF_XCH + wq * 4096 + (ch >> 2) * 2048 + lane * 64 +
                                                     (((ch & 3) ^ ((lane >> 1) & 3)) << 4));
          const float mx = fmaxf(lw_own, lw_p);
          float ca = 0.f, cb = 0.f;  // coefficients of the raw accumulator values and of the partner's normalised rows
          if (mx == -INFINITY) {
            // every group's weights underflowed: outside the numeric domain of this path
            if (rank == 0 && tt < nvalid) {
              atomicOr(p.err, 2);
              if (p.gate != nullptr) {
                p.gate[0] = 1;
                p.gate[1 + lane_id] = 1;
              }
            }
          } else {
            const float wa = ex2_approx(lw_own - mx), wb = ex2_approx(lw_p - mx);
            const float iw = rcp_approx(wa + wb);
            ca = wa * iw * inv;
            cb = wb * iw;
            if (rank == 0 && p.lse_dec != nullptr && tt < nvalid)
              p.lse_dec[(int64_t)lane_id * p.N + t0 + tt] = (mx + __log2f(wa + wb)) * kLn2;
          }
          // The merged rows go out from the exchange tile itself (its layout is the bulk store's 64-byte swizzle and
          // the partner's rows are in registers by now): both 32-column tiles are stored without waiting on each other.
          uint8_t* const xt = smem + L::OFF_XCH + wq * 4096;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const uint32_t(&r)[32] = half ? rb : ra;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              const uint4 x = xp[half * 4 + ch];
              const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
              uint32_t o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xw[j]));
                float y0, y1;  // own raw values * ca + partner's normalised values * cb, two columns per instruction
                f2_unpack(f2_fma(f2_pack(__uint_as_float(r[ch * 8 + 2 * j]), __uint_as_float(r[ch * 8 + 2 * j + 1])),
                                 f2_pack(ca, ca), f2_mul(f2_pack(f.x, f.y), f2_pack(cb, cb))), y0, y1);
                o[j] = pack_bf16(y0, y1);
              }
              *reinterpret_cast<uint4*>(xt + half * 2048 + lane * 64 + ((ch ^ ((lane >> 1) & 3)) << 4)) =
                  make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_4d(&tm_y, xt, (int)rank * 64, h, t0 + wq * 32, b);
            tma_store_4d(&tm_y, xt + 2048, (int)rank * 64 + 32, h, t0 + wq * 32, b);
            bulk_commit_group();
          }
          // (the partner learns that the tile is free when the next chunk's epilogue begins, see above: by then the
          // stores have long read it; it does not send before its own next epilogue anyway)
          if (tid == 256) TC_TRACE(1, i, 3);
          continue;
        }
      }
      // The accumulator goes back to the MMA issuer as soon as its columns are in registers (single-buffered
      // instances); scaling and the stores follow.  Wide: two value blocks of 64 columns, handed back after the second.
#pragma unroll
      for (int vb = 0; vb < VB; ++vb) {
        uint32_t ra[32], rb[32];
        tmem_ld32(tl + TM_Y + vb * 64, ra);
        tmem_ld32(tl + TM_Y + vb * 64 + 32, rb);
        tmem_wait_ld();
        if (vb == VB - 1) {
          tc_fence_before_sync();
          warp_arrive(&misc->y_free, lane);
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint32_t(&r)[32] = half ? rb : ra;
          const int col = value_col0<ZS, SPLIT>() + vb * 64 + half * 32;
          // 32 columns of this thread's row as 16-bit values: bf16 of y, or fp16 of a latent group's partial
          uint4 v[4];
          const uint64_t inv2 = f2_pack(inv, inv);
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float y0, y1;  // two columns per multiply
              f2_unpack(f2_mul(f2_pack(__uint_as_float(r[ch * 8 + 2 * j]), __uint_as_float(r[ch * 8 + 2 * j + 1])), inv2), y0, y1);
              o[j] = SPLIT ? pack_f16(y0, y1) : pack_bf16(y0, y1);
            }
            v[ch] = make_uint4(o[0], o[1], o[2], o[3]);
          }
          if (p.y_tma) {
            // One tiled bulk store per warp and 32 x 32 tile.  A thread storing its own row straight to global
            // memory costs 32 separate 16-byte transactions per instruction; the latent warps' operand stores to
            // shared memory queued behind those and the whole kernel ran 12 % slower.  Rows beyond the sequence end
            // are clipped by the copy.
            if (lane == 0) bulk_wait_group_read0();  // the previous tile has left the staging buffer
            __syncwarp();
#pragma unroll
            for (int ch = 0; ch < 4; ++ch)  // 64-byte swizzle: 16-byte piece index ^ (row / 2) % 4
              *reinterpret_cast<uint4*>(stage + lane * 64 + ((ch ^ ((lane >> 1) & 3)) << 4)) = v[ch];
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_4d(&tm_y, stage, col, h, t0 + wq * 32, SPLIT ? (int)(blockIdx.z / ZS) * (int)(gridDim.x / p.H) + b : b);
              bulk_commit_group();
            }
          } else if (SPLIT) {
            if (p.part_y != nullptr && tt < nvalid) {
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.part_y) +
                                                    ((part_row0 + t0 + tt) * p.H + h) * DV + col);
#pragma unroll
              for (int ch = 0; ch < 4; ++ch) dst[ch] = v[ch];
            }
          } else if (p.y != nullptr && tt < nvalid) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.y) + (int64_t)b * p.y_stride_b +
                                                  (int64_t)h * p.y_stride_h + (int64_t)(t0 + tt) * p.y_stride_n + col);
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) dst[ch] = v[ch];
          }
        }
      }
      if (!ok) break;
      if (tid == 256) TC_TRACE(1, i, 3);
    }
    if (lane == 0) bulk_wait_group0();  // the bulk stores of this warp are complete
  }
  if (!ok) {
    misc->abort_flag = 1;
    atomicOr(p.err, 1);
  }
  tc_fence_before_sync();
  __syncthreads();
  // the partner may still write to this CTA's shared memory or arrive on its barriers until it is done as well
  if (xmerge) cluster_sync_all();
  if (warp == 12) tmem_dealloc(tmem, TM_COLS);
}



namespace {

template <bool PADDED, int DKB, int DVB, bool SPLIT, int MODE, bool KEEP, bool WIDE = false>
int launch_keep(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& ty,
                const TcParams& p, dim3 grid, cudaStream_t stream) {
  auto kern = prefill_tc_kernel<PADDED, DKB, DVB, SPLIT, MODE, KEEP, WIDE>;
  FLARE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay<DKB, WIDE>::SMEM_BYTES));
  LaunchTimer timer(p.y == nullptr ? "prefill_tc_kernel (state only)" : (WIDE ? "prefill_tc_kernel (wide)" : "prefill_tc_kernel"),
                    stream);
  if (WIDE && SPLIT && p.cluster_merge) {
    // the two latent-group CTAs of a lane (adjacent in grid.z) as one thread-block cluster
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = Lay<DKB, WIDE>::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 1;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 2;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    FLARE_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tq, tk, tv, ty, p));
  } else {
    kern<<<grid, NTHREADS, Lay<DKB, WIDE>::SMEM_BYTES, stream>>>(tq, tk, tv, ty, p);
  }
  FLARE_CUDA_CHECK(cudaGetLastError());
  return FLARE_OK;
}

template <bool PADDED, int DKB, int DVB, bool SPLIT, int MODE>
int launch_instance(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& ty,
                    const TcParams& p, dim3 grid, cudaStream_t stream) {
  return p.dump_u != nullptr ? launch_keep<PADDED, DKB, DVB, SPLIT, MODE, true>(tq, tk, tv, ty, p, grid, stream)
                             : launch_keep<PADDED, DKB, DVB, SPLIT, MODE, false>(tq, tk, tv, ty, p, grid, stream);
}

}  // namespace

template <>
int launch_prefill_tc_unit<FLARE_TC_UNIT>(bool padded, int mode, const CUtensorMap& tq, const CUtensorMap& tk,
                                          const CUtensorMap& tv, const CUtensorMap& ty, const TcParams& p, dim3 grid,
                                          cudaStream_t stream) {
  // units 0..2: (Dk, Dv) = (64, 64), (128, 128), (64, 128); units 3..5: the same with the latent-group split;
  // units 6, 7: the wide (128, 128) instance (one CTA for both value blocks) without / with the latent-group split
#if FLARE_TC_UNIT >= 6
  constexpr bool WSPLIT = FLARE_TC_UNIT == 7;
  (void)padded;
  if (p.dump_u != nullptr) {  // training forward that keeps its per-chunk states
    if (mode == 1) return launch_keep<false, 2, 2, WSPLIT, 1, true, true>(tq, tk, tv, ty, p, grid, stream);
    if (mode == 2) return launch_keep<false, 2, 2, WSPLIT, 2, true, true>(tq, tk, tv, ty, p, grid, stream);
    return launch_keep<false, 2, 2, WSPLIT, 0, true, true>(tq, tk, tv, ty, p, grid, stream);
  }
  if (mode == 1) return launch_keep<false, 2, 2, WSPLIT, 1, false, true>(tq, tk, tv, ty, p, grid, stream);
  if (mode == 2) return launch_keep<false, 2, 2, WSPLIT, 2, false, true>(tq, tk, tv, ty, p, grid, stream);
  return launch_keep<false, 2, 2, WSPLIT, 0, false, true>(tq, tk, tv, ty, p, grid, stream);
#else
  constexpr int COMBO = FLARE_TC_UNIT % 3;
  constexpr int DKB = COMBO == 1 ? 2 : 1;
  constexpr int DVB = COMBO == 0 ? 1 : 2;
  constexpr bool SPLIT = FLARE_TC_UNIT >= 3;
  if (mode == 1)
    return padded ? launch_instance<true, DKB, DVB, SPLIT, 1>(tq, tk, tv, ty, p, grid, stream)
                  : launch_instance<false, DKB, DVB, SPLIT, 1>(tq, tk, tv, ty, p, grid, stream);
  if (mode == 2)
    return padded ? launch_instance<true, DKB, DVB, SPLIT, 2>(tq, tk, tv, ty, p, grid, stream)
                  : launch_instance<false, DKB, DVB, SPLIT, 2>(tq, tk, tv, ty, p, grid, stream);
  return padded ? launch_instance<true, DKB, DVB, SPLIT, 0>(tq, tk, tv, ty, p, grid, stream)
                : launch_instance<false, DKB, DVB, SPLIT, 0>(tq, tk, tv, ty, p, grid, stream);
#endif
}

#else  // host side and the merge kernel

__device__ int g_tc_error = 0;

template <> int launch_prefill_tc_unit<0>(bool, int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const TcParams&, dim3, cudaStream_t);
template <> int launch_prefill_tc_unit<1>(bool, int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const TcParams&, dim3, cudaStream_t);
template <> int launch_prefill_tc_unit<2>(bool, int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const TcParams&, dim3, cudaStream_t);
template <> int launch_prefill_tc_unit<3>(bool, int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const TcParams&, dim3, cudaStream_t);
template <> int launch_prefill_tc_unit<4>(bool, int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const TcParams&, dim3, cudaStream_t);
template <> int launch_prefill_tc_unit<5>(bool, int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const TcParams&, dim3, cudaStream_t);
template <> int launch_prefill_tc_unit<6>(bool, int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const TcParams&, dim3, cudaStream_t);
template <> int launch_prefill_tc_unit<7>(bool, int, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const TcParams&, dim3, cudaStream_t);

// -------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------
namespace {

bool make_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const int64_t* strides_elems,
              const uint32_t* box) {
  return tc::make_map_bf16(map, base, rank, dims, strides_elems, box);
}

}  // namespace

bool prefill_tc_supported(const flare_fwd_args_t* a) {
  const int bs = a->block_size;
  const bool block_ok = bs == 1 || ((bs == 16 || bs == 32 || bs == 64 || bs == 128) && a->N % bs == 0);
  // the per-block encoder normalisers exist in block-causal mode only; the decode log-sum-exp in every mode
  const bool lse_ok = a->lse_enc == nullptr || bs > 1;
  if (a->lengths != nullptr && bs > 1) return false;  // per-row lengths: token-causal only
  // stablemax encoder weights: token-causal only
  const bool variant_ok = a->variant == FLARE_SOFTMAX || (a->variant == FLARE_STABLEMAX && bs == 1 && a->power > 0.f);
  // the tiled copies need positive strides whose byte size is a multiple of 16 and stays below 2^40; anything else
  // (a tensor expanded over heads with stride 0, say) is served by the exact kernels
  const int64_t strides[] = {a->k_stride_b, a->k_stride_n, a->k_stride_h, a->v_stride_b, a->v_stride_n, a->v_stride_h,
                             a->q_stride_h, a->q_stride_m};
  for (int64_t st : strides)
    if (st <= 0 || (st % 8) != 0 || st >= (int64_t(1) << 39)) return false;
  return a->dtype == FLARE_BF16 && variant_ok && block_ok && lse_ok && a->M <= 4 * M && a->M >= 16 &&
         (a->M % 16) == 0 && ((a->Dk == 64 && (a->Dv == 64 || a->Dv == 128)) || (a->Dk == 128 && a->Dv == 128)) && a->q_dec == nullptr &&
         a->k_dec == nullptr && a->mask == nullptr && a->N >= 1;
}

// Merge of the latent groups' partial read-outs: y = sum_g w_g y_g / sum_g w_g with w_g = exp2(lw_g - max lw).
// One thread per (token, head, 8 value columns).
__global__ void __launch_bounds__(256) tc_merge_groups_kernel(const __half* __restrict__ part_y, const float* __restrict__ part_lw,
                                                               int groups, int64_t rows /* B*N*H */, int N, int H, int dv,
                                                               __nv_bfloat16* y, int64_t y_stride_b, int64_t y_stride_n,
                                                               int64_t y_stride_h, float* lse_dec /* [B, H, N] or null */,
                                                               const int32_t* lens /* [B] or null */, int* gate) {
  const int cols8 = dv >> 3;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * cols8) return;
  const int64_t row = idx / cols8;
  const int c8 = (int)(idx % cols8);
  if (lens != nullptr && (int)((row / H) % N) >= lens[row / ((int64_t)H * N)]) return;  // right padding: nothing emitted
  float lw[4], mx = -INFINITY;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    lw[g] = g < groups ? part_lw[g * rows + row] : -INFINITY;
    mx = fmaxf(mx, lw[g]);
  }
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, wsum = 0.f;
  if (mx == -INFINITY) {
    if (c8 == 0) {  // every group's weights underflowed: outside the numeric domain
      atomicOr(&g_tc_error, 2);
      if (gate != nullptr) {
        gate[0] = 1;
        gate[1 + (row / ((int64_t)H * N)) * H + (row % H)] = 1;
      }
    }
  } else {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g >= groups) break;
      const float w = exp2f(lw[g] - mx);
      wsum += w;
      const uint4 raw = *reinterpret_cast<const uint4*>(part_y + (g * rows + row) * dv + c8 * 8);
      const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&rw[j]));
        acc[2 * j] += w * f.x;
        acc[2 * j + 1] += w * f.y;
      }
    }
  }
  const float inv = wsum > 0.f ? 1.0f / wsum : 0.f;
  const int h = (int)(row % H);
  const int64_t bn = row / H;
  const int n = (int)(bn % N);
  const int64_t b = bn / N;
  if (lse_dec != nullptr && c8 == 0) lse_dec[(b * H + h) * N + n] = (mx + log2f(wsum)) * kLn2;
  uint4 v;
  v.x = pack_bf16(acc[0] * inv, acc[1] * inv);
  v.y = pack_bf16(acc[2] * inv, acc[3] * inv);
  v.z = pack_bf16(acc[4] * inv, acc[5] * inv);
  v.w = pack_bf16(acc[6] * inv, acc[7] * inv);
  *reinterpret_cast<uint4*>(y + b * y_stride_b + (int64_t)n * y_stride_n + (int64_t)h * y_stride_h + c8 * 8) = v;
}


int prefill_tc_latent_groups(const flare_fwd_args_t* a) { return (a->M + M - 1) / M; }

int prefill_tc_ctas_per_lane(const flare_fwd_args_t* a) { return a->Dv / D * prefill_tc_latent_groups(a); }

// fp16 partial read-outs [groups][B][N][H][Dv], then fp32 weight masses [groups][B][N][H]
size_t prefill_tc_partial_lw_offset(const flare_fwd_args_t* a) {
  const int groups = prefill_tc_latent_groups(a);
  return align_up((size_t)groups * a->B * a->N * a->H * a->Dv * sizeof(__half), 256);
}

size_t prefill_tc_partial_bytes(const flare_fwd_args_t* a) {
  const int groups = prefill_tc_latent_groups(a);
  if (groups == 1) return 0;
  return prefill_tc_partial_lw_offset(a) + (size_t)groups * a->B * a->N * a->H * sizeof(float);
}

int launch_prefill_tc(const flare_fwd_args_t* a, const TcParams& p_in, int nseg_grid, cudaStream_t stream) {
  TcParams p = p_in;
  {
    void* err = nullptr;
    FLARE_CUDA_CHECK(cudaGetSymbolAddress(&err, g_tc_error));  // of the current device
    p.err = reinterpret_cast<int*>(err);
  }
  p.block = a->block_size;
  p.power = a->power;
  p.lens = a->lengths;
  p.lse_dec = a->lse_dec;
  p.lse_enc = a->lse_enc;
  if (p.y == nullptr) {  // state-only passes emit nothing else
    p.lse_dec = p.lse_enc = nullptr;
    p.dump_u = nullptr;
  }
  CUtensorMap tq, tk, tv;
  {
    // latent bank (used by the Dk = 64 instances only; any valid map otherwise)
    const uint64_t dims[3] = {(uint64_t)a->Dk, (uint64_t)a->M, (uint64_t)a->H};
    const int64_t str[2] = {a->q_stride_m, a->q_stride_h};
    const uint32_t box[3] = {64, 128, 1};
    if (!make_map(&tq, a->q, 3, dims, str, box)) {
      set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled (latent bank)");
      return FLARE_ERR_CUDA;
    }
  }
  {
    const uint64_t dimk[4] = {(uint64_t)a->Dk, (uint64_t)a->H, (uint64_t)a->N, (uint64_t)a->B};
    const uint64_t dimv[4] = {(uint64_t)a->Dv, (uint64_t)a->H, (uint64_t)a->N, (uint64_t)a->B};
    const uint32_t box[4] = {64, 1, 128, 1};
    const int64_t strk[3] = {a->k_stride_h, a->k_stride_n, a->k_stride_b};
    const int64_t strv[3] = {a->v_stride_h, a->v_stride_n, a->v_stride_b};
    if (!make_map(&tk, a->k, 4, dimk, strk, box) || !make_map(&tv, a->v, 4, dimv, strv, box)) {
      set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled (keys / values)");
      return FLARE_ERR_CUDA;
    }
  }
  const int groups = prefill_tc_latent_groups(a);
  const bool padded = (a->M % M) != 0;
  const int mode = a->variant == FLARE_STABLEMAX ? 2 : (a->block_size > 1 ? 1 : 0);
  // (128, 128) heads: two CTAs per (lane, group), each repeating the score / E / R work for 64 value columns, while
  // they all fit the SMs at once; beyond that the wide instance, one CTA for all 128 columns.  (Not for a padded
  // latent bank.)  FLARE_B200_WIDE=0 / 1 forces the choice.
  bool wide = a->Dk == 128 && a->Dv == 128 && !padded && (int64_t)a->B * a->H * nseg_grid * groups * 2 > sm_count();
  if (const char* env = getenv("FLARE_B200_WIDE")) wide = a->Dk == 128 && a->Dv == 128 && !padded && env[0] == '1';
  // Read-out rows leave through tiled bulk stores of 32 tokens x 32 columns (64-byte swizzle): into y, or with several
  // latent groups into the dense fp16 partials.  Per-row lengths (rows beyond a length stay untouched) and output
  // strides the tiled copy cannot express fall back to per-thread stores.
  CUtensorMap ty = tk;
  p.y_tma = 0;
  p.cluster_merge = 0;
  if (p.y != nullptr && a->lengths == nullptr) {
    const uint32_t box[4] = {32, 1, 32, 1};
    const int64_t str[3] = {p.y_stride_h, p.y_stride_n, p.y_stride_b};
    bool y_ok = (reinterpret_cast<uintptr_t>(p.y) % 16) == 0;
    for (int64_t st : str) y_ok = y_ok && st > 0 && (st % 8) == 0 && st < (int64_t(1) << 39);
    const uint64_t ydims[4] = {(uint64_t)a->Dv, (uint64_t)a->H, (uint64_t)a->N, (uint64_t)a->B};
    // wide instance with exactly two latent groups: the two CTAs of a lane merge on chip (thread-block cluster) and
    // store y themselves.  FLARE_B200_CLUSTER=0 keeps the partials in global memory and the merge kernel.
    bool cluster = wide && groups == 2 && y_ok;
    if (const char* env = getenv("FLARE_B200_CLUSTER"))
      if (env[0] == '0') cluster = false;
    if (cluster && tc::make_map_bf16(&ty, p.y, 4, ydims, str, box, CU_TENSOR_MAP_SWIZZLE_64B)) {
      p.y_tma = 1;
      p.cluster_merge = 1;
    } else if (groups > 1) {
      const uint64_t dims[4] = {(uint64_t)a->Dv, (uint64_t)a->H, (uint64_t)a->N, (uint64_t)groups * a->B};
      const int64_t pstr[3] = {a->Dv, (int64_t)a->H * a->Dv, (int64_t)a->N * a->H * a->Dv};
      p.y_tma = tc::make_map_bf16(&ty, p.part_y, 4, dims, pstr, box, CU_TENSOR_MAP_SWIZZLE_64B) ? 1 : 0;
    } else {
      p.y_tma = y_ok && tc::make_map_bf16(&ty, p.y, 4, ydims, str, box, CU_TENSOR_MAP_SWIZZLE_64B) ? 1 : 0;
    }
  }
  if (const char* env = getenv("FLARE_B200_ROW_STORES"))  // diagnostic: per-thread row stores instead
    if (env[0] == '1' && !p.cluster_merge) p.y_tma = 0;
  const dim3 grid(a->B * a->H, nseg_grid, wide ? groups : a->Dv / D * groups);
  int rc;
  const int combo = a->Dk == 128 ? 1 : (a->Dv == 128 ? 2 : 0);  // (64, 64), (128, 128), (64, 128)
  if (wide)
    rc = groups > 1 ? launch_prefill_tc_unit<7>(padded, mode, tq, tk, tv, ty, p, grid, stream)
                    : launch_prefill_tc_unit<6>(padded, mode, tq, tk, tv, ty, p, grid, stream);
  else if (combo == 0)
    rc = groups > 1 ? launch_prefill_tc_unit<3>(padded, mode, tq, tk, tv, ty, p, grid, stream)
                    : launch_prefill_tc_unit<0>(padded, mode, tq, tk, tv, ty, p, grid, stream);
  else if (combo == 1)
    rc = groups > 1 ? launch_prefill_tc_unit<4>(padded, mode, tq, tk, tv, ty, p, grid, stream)
                    : launch_prefill_tc_unit<1>(padded, mode, tq, tk, tv, ty, p, grid, stream);
  else
    rc = groups > 1 ? launch_prefill_tc_unit<5>(padded, mode, tq, tk, tv, ty, p, grid, stream)
                    : launch_prefill_tc_unit<2>(padded, mode, tq, tk, tv, ty, p, grid, stream);
  if (rc != FLARE_OK || groups == 1 || p.y == nullptr || p.cluster_merge) return rc;
  const int64_t rows = (int64_t)a->B * a->N * a->H;
  const int64_t threads = rows * (a->Dv / 8);
  LaunchTimer timer("tc_merge_groups_kernel", stream);
  tc_merge_groups_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __half*>(p.part_y), p.part_lw, groups, rows, a->N, a->H, a->Dv, reinterpret_cast<__nv_bfloat16*>(p.y), p.y_stride_b,
      p.y_stride_n, p.y_stride_h, p.lse_dec, p.lens, p.gate);
  FLARE_CUDA_CHECK(cudaGetLastError());
  return FLARE_OK;
}

int tc_error_word(int** device_address) {
  void* err = nullptr;
  FLARE_CUDA_CHECK(cudaGetSymbolAddress(&err, g_tc_error));  // of the current device
  *device_address = reinterpret_cast<int*>(err);
  return FLARE_OK;
}

int prefill_tc_error_flag(int* host_value, bool reset) {
  int v = 0;
  FLARE_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)));
  if (reset && v != 0) {
    const int zero = 0;
    FLARE_CUDA_CHECK(cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int)));
  }
  *host_value = v;
  return FLARE_OK;
}

#endif  // FLARE_TC_UNIT

}  // namespace flare
