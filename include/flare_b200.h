/*
 * flare_b200.h — C ABI of libflare_b200.so: Causal FLARE attention kernels for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes, launches on the given CUDA stream and
 * returns an int status (FLARE_OK == 0).  Nothing here allocates device memory unless stated; scratch
 * is passed in by the caller (size from the matching *_workspace_bytes query).  No call synchronises.
 *
 * Tensor layouts are the public ones of the `causal_flare` Python package:
 *   Q      [H, M, Dk]       latent queries, shared over the batch
 *   K      [B, N, H, Dk]    token keys            V [B, N, H, Dv]   token values
 *   Q_dec  [B, N, H, Dk]    optional decode-side queries (NULL: use K)
 *   K_dec  [H, M, Dk]       optional decode-side keys    (NULL: use Q)
 *   Y      [B, N, H, Dv]    output (any (b, n, h) strides, so [B, H, N, Dv] is expressible)
 *   state  m, d [B, H, M] fp32 and u [B, H, M, Dv] fp32 (running max, denominator, numerator)
 * The innermost dimension of every tensor is contiguous; the other strides are given in ELEMENTS.
 * M, Dk and Dv must be multiples of 16.
 */
#ifndef FLARE_B200_H_
#define FLARE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* flare_stream_t; /* same handle type as cudaStream_t */

enum flare_status {
  FLARE_OK = 0,
  FLARE_ERR_BAD_SHAPE = 1,      /* a dimension is zero/negative or not a multiple of 16 */
  FLARE_ERR_UNSUPPORTED = 2,    /* shape outside what the kernels cover (e.g. M > 512) */
  FLARE_ERR_BAD_POINTER = 3,    /* NULL where a tensor is required, or not 16-byte aligned */
  FLARE_ERR_WORKSPACE = 4,      /* workspace missing or smaller than *_workspace_bytes says */
  FLARE_ERR_BAD_DTYPE = 5,
  FLARE_ERR_BAD_CONFIG = 6,     /* block_size does not divide N, bad variant, ... */
  FLARE_ERR_CUDA = 7,           /* a CUDA runtime call failed; see flare_last_cuda_error() */
  FLARE_ERR_TOO_LARGE = 8       /* request exceeds a fixed capacity of the entry point */
};

enum flare_dtype { FLARE_F32 = 0, FLARE_BF16 = 1, FLARE_F16 = 2 };

/* Encoder weight of a token for a latent: exp(s) (softmax, tracked online with a running max) or
 * the stablemax transform sigma(s) = (1+s)^p for s >= 0, (1-s)^-p for s < 0. */
enum flare_variant { FLARE_SOFTMAX = 0, FLARE_STABLEMAX = 1 };

/* Which implementation a call may use. AUTO picks the tensor-core path when the shape qualifies. */
enum flare_path { FLARE_PATH_AUTO = 0, FLARE_PATH_EXACT = 1, FLARE_PATH_TENSOR = 2 };

typedef struct flare_state {
  float* m; /* [B, H, M]      running max per latent (ignored for stablemax) */
  float* d; /* [B, H, M]      running denominator */
  float* u; /* [B, H, M, Dv]  running un-normalised numerator */
} flare_state_t;

/*
 * Forward problem.  Replaces the kernel launch sequences behind
 *   flare_autoregressive_triton            causal_flare/autoregressive/training.py:4921 (forward :733-905)
 *   flare_autoregressive_prefill_triton    causal_flare/autoregressive/inference.py:624-820
 *   flare_recurrent_triton (forward)       causal_flare/autoregressive/recurrent.py:288-414
 *   flare_autoregressive_stablemax_triton  causal_flare/autoregressive/stablemax_triton.py:1709-1978
 *   flare_semi_autoregressive_trition      causal_flare/semi_autoregressive/training.py:1836-1961
 */
typedef struct flare_fwd_args {
  const void* q;
  const void* k;
  const void* v;
  const void* q_dec; /* NULL: weight sharing with k */
  const void* k_dec; /* NULL: weight sharing with q */
  void* y;           /* same dtype as the inputs; may be NULL when only the final state is wanted */
  const int32_t* mask;      /* [B, N] int32, 0 = token leaves the state untouched and emits y = 0; may be NULL */
  const int32_t* lengths;   /* [B] int32 or NULL: batch row b has lengths[b] tokens, the rest of its N rows is right
                               padding (state untouched, those rows of y are NOT written).  Tensor-core path only, not
                               together with mask; FLARE_ERR_UNSUPPORTED when the call resolves to the exact path. */
  flare_state_t state_in;   /* all NULL: start from the empty state (m=-inf, d=0, u=0) */
  flare_state_t state_out;  /* all NULL: final state not written */
  float* lse_dec;           /* [B, H, N] log-sum-exp of the decode scores; may be NULL */
  float* lse_enc;           /* [B, H, N/block_size, M] log normaliser after each block; semi-AR only; may be NULL */
  void* workspace;
  size_t workspace_bytes;
  int32_t B, N, H, M, Dk, Dv;
  int64_t q_stride_h, q_stride_m;
  int64_t k_stride_b, k_stride_n, k_stride_h;
  int64_t v_stride_b, v_stride_n, v_stride_h;
  int64_t qd_stride_b, qd_stride_n, qd_stride_h;
  int64_t kd_stride_h, kd_stride_m;
  int64_t y_stride_b, y_stride_n, y_stride_h;
  float scale;
  float power;        /* stablemax exponent p */
  int32_t dtype;      /* flare_dtype of q, k, v, q_dec, k_dec, y */
  int32_t variant;    /* flare_variant */
  int32_t block_size; /* 1: token-causal (autoregressive); > 1: block-causal (semi-autoregressive) */
  int32_t path;       /* flare_path */
  /* Training (optional, NULL / 0 otherwise): a buffer of flare_forward_keep_bytes(args) bytes in which the tensor-core
   * forward leaves what flare_backward needs to skip its own replay of the forward: the state before every chunk of
   * 128 tokens (bf16 numerator, fp32 frame and denominator per latent) and the call's numeric-domain gate words.
   * Needs y and lse_dec as well; FLARE_ERR_BAD_CONFIG when given for a problem whose keep size is 0. */
  void* keep;
  size_t keep_bytes;
} flare_fwd_args_t;

size_t flare_forward_workspace_bytes(const flare_fwd_args_t* args);
int flare_forward(const flare_fwd_args_t* args, flare_stream_t stream);
/* Size of flare_fwd_args_t::keep for this problem: 0 unless the call takes the tensor-core path with shared decode
 * weights, no mask / lengths / carry-in state (the problems flare_backward_uses_tensor_path accepts). */
size_t flare_forward_keep_bytes(const flare_fwd_args_t* args);

/*
 * flare_forward for callers that cannot allocate device memory (no counterpart in the reference, whose wrappers
 * always allocate their workspaces with torch).  Same arguments and results as flare_forward, except that
 * args->workspace / workspace_bytes are ignored: the scratch for the segment-state scan lives in a fixed array
 * inside the library, flare_noalloc_scratch_capacity() bytes (8 MiB) per GPU, held from library load to exit.
 * Returns FLARE_ERR_TOO_LARGE, without launching anything, when the problem needs more scratch than that
 * (flare_forward_workspace_bytes tells how much).  The call performs no cudaMalloc / cudaFree and calls no
 * allocating library routine.  The first call on each device resolves the array's device address
 * (cudaGetSymbolAddress); make that first call outside any stream capture.  All calls share the one array:
 * two calls whose kernels may overlap on the GPU (different streams, or different host threads) race on it,
 * so serialise them.  Nothing in the array needs clearing between calls.
 */
int flare_forward_noalloc(const flare_fwd_args_t* args, flare_stream_t stream);
size_t flare_noalloc_scratch_capacity(void);

/*
 * Backward problem: gradients of <Y, dY>.  Replaces
 *   _chunked_flare_lse_backward_impl       causal_flare/autoregressive/training.py:4369-4918
 *   _recurrent_flare_backward_impl         causal_flare/autoregressive/recurrent.py:749-935
 *   FLAREAutoregressiveStablemaxTriton.backward   causal_flare/autoregressive/stablemax_triton.py:1981-2420
 *   _semi_autoregressive_backward_impl     causal_flare/semi_autoregressive/training.py:3768-3987
 * Nothing but the inputs is needed from the forward: intermediates are recomputed.  Two implementations: the
 * tensor-core one (bwd_tc.cu: a forward that keeps per-chunk states, then a reverse chunk sweep on tcgen05 and a
 * tensor-core dK / dQ product) for the shapes flare_backward_uses_tensor_path accepts, and the exact fp32 one
 * (bwd_exact.cu) for everything else; fwd.path = FLARE_PATH_EXACT forces the latter.
 * dq / dk_dec are fp32 [H, M, Dk] (summed over the batch); dk, dv, dq_dec have the input dtype and the
 * input's shape, densely packed.  With weight sharing (q_dec/k_dec NULL) the decode-side gradients are
 * folded into dk / dq and dq_dec / dk_dec must be NULL.
 */
typedef struct flare_bwd_args {
  flare_fwd_args_t fwd; /* y, mask, lengths, state_out, lse_* are ignored; state_in only in span mode (below) */
  const void* dy;       /* [B, N, H, Dv], input dtype */
  int64_t dy_stride_b, dy_stride_n, dy_stride_h;
  float* dq;            /* [H, M, Dk] fp32 */
  void* dk;             /* [B, N, H, Dk] contiguous */
  void* dv;             /* [B, N, H, Dv] contiguous */
  void* dq_dec;         /* [B, N, H, Dk] contiguous or NULL */
  float* dk_dec;        /* [H, M, Dk] fp32 or NULL */
  /*
   * Spans of a longer sequence (sequence parallelism over GPUs; no counterpart in the reference).  All NULL / 0 for a
   * whole sequence.  The span's tokens are fwd.k / fwd.v / dy; fwd.state_in (else ignored) is the forward state of the
   * tokens before the span.  phase 1 replays the span and writes its summary - (b, c) at its first token for a zero
   * carry-in from the right, the product of its decays, the decay of its first token (block) - into span_*; the
   * caller combines the summaries of the spans to its right into carry_* and calls phase 2 with the SAME workspace,
   * which writes dk, dv and this span's part of dq (to be summed over the spans).  phase 0 does both at once
   * (carry_* may then be given directly).
   */
  const float* carry_b;   /* [B, H, M, Dv]  b at the first token after the span */
  const float* carry_c;   /* [B, H, M] */
  const float* carry_rho; /* [B, H, M]      decay (1 - e) of the first token (block) after the span */
  float* span_b0;         /* [B, H, M, Dv] */
  float* span_c0;         /* [B, H, M] */
  float* span_gam;        /* [B, H, M] */
  float* span_rho_first;  /* [B, H, M] */
  int32_t phase;          /* 0, 1 or 2 */
  /* Optional, from a forward of the same problem that was given fwd.keep: its output y (strides in elements), its
   * lse_dec [B, H, N], and the keep buffer in fwd.keep / fwd.keep_bytes.  With all three the tensor-core backward
   * skips its replay of the forward (and asks for a smaller workspace); otherwise they are ignored. */
  const void* y;
  int64_t y_stride_b, y_stride_n, y_stride_h;
  const float* lse_dec;
} flare_bwd_args_t;

size_t flare_backward_workspace_bytes(const flare_bwd_args_t* args);
int flare_backward(const flare_bwd_args_t* args, flare_stream_t stream);

/*
 * One decode token per (batch, head): updates (m, d, u) IN PLACE and writes y [B, H, Dv].
 * Replaces flare_recurrent_step_kernel and its wrapper flare_autoregressive_decode_triton,
 * causal_flare/autoregressive/inference.py:359-489, :492-621.
 */
typedef struct flare_decode_args {
  const void* q;      /* [H, M, Dk] */
  const void* k;      /* [B, H, Dk] */
  const void* v;      /* [B, H, Dv] */
  const void* q_dec;  /* [B, H, Dk] or NULL */
  const void* k_dec;  /* [H, M, Dk] or NULL */
  void* y;            /* [B, H, Dv], input dtype, contiguous */
  const int32_t* mask; /* [B] or NULL */
  flare_state_t state; /* updated in place; contiguous */
  int32_t B, H, M, Dk, Dv;
  int64_t q_stride_h, q_stride_m;
  int64_t k_stride_b, k_stride_h;
  int64_t v_stride_b, v_stride_h;
  int64_t qd_stride_b, qd_stride_h;
  int64_t kd_stride_h, kd_stride_m;
  float scale;
  int32_t dtype;
} flare_decode_args_t;

int flare_decode_step(const flare_decode_args_t* args, flare_stream_t stream);

/*
 * out = merge(a, b): the associative combination of two online-softmax states over `lanes` = B*H
 * independent (batch, head) lanes; `out` may alias `a` or `b`.  Replaces _merge_flare_stats,
 * causal_flare/autoregressive/inference.py:194-228.  With `count` > 1, `b` holds `count` states
 * back to back (state j at offset j*lanes) which are folded in order into `a`.
 */
int flare_state_merge(const flare_state_t* a, const flare_state_t* b, const flare_state_t* out,
                      int64_t lanes, int32_t M, int32_t Dv, int32_t count, flare_stream_t stream);

const char* flare_status_string(int status);
const char* flare_last_cuda_error(void);
int flare_abi_version(void);

/* Measurement hooks (no counterpart in the reference; used by the benchmark).
 * flare_set_kernel_events: two cudaEvent_t handles (or NULL, NULL to clear) that later flare_forward /
 * flare_backward calls of this thread record immediately before and after their dominant kernel, on the
 * stream they launch on.  flare_last_launch_count: kernels launched by this thread's last forward/backward. */
void flare_set_kernel_events(void* begin_event, void* end_event);
int flare_last_launch_count(void);
/* Per-kernel timings (the reference's profile=True returns one entry per kernel launch,
 * causal_flare/autoregressive/training.py:4-50).  flare_profile_enable(1) clears this thread's records and makes every
 * later launch of this thread record a pair of CUDA events around its kernel; flare_profile_enable(0) stops recording.
 * flare_profile_entry(i, &name, &ms) synchronises on record i (0 <= i < flare_profile_count()) and returns its kernel
 * name and device time. */
void flare_profile_enable(int on);
int flare_profile_count(void);
int flare_profile_entry(int i, const char** name, float* ms);
/* Diagnostic: device buffer of 3 x 16 x 8 int64 that the tensor-core prefill kernel fills with clock64 stamps of
 * the phases of its first CTA (roles: latent group, token group, MMA issuer; first 16 chunks).  NULL disables. */
void flare_set_trace_buffer(void* device_buffer);

/* 1 when flare_forward would take the tcgen05 tensor-core path for this problem, else 0.  That is: path AUTO or
 * TENSOR, bf16 (or fp16 without args->keep: q, k, v are rounded to bf16 copies in the workspace, the kernels run on
 * those and y is written back as fp16; flare_forward_workspace_bytes includes the copies), 16 <= M <= 512 (multiple of 16), (Dk, Dv) = (64, 64), (128, 128) or (64, 128), shared decode weights (q_dec = k_dec = NULL),
 * mask = NULL, and either the softmax encoder with block_size 1 / 16 / 32 / 64 / 128 (N a multiple of it) or the
 * stablemax encoder with block_size 1; lse_enc only with block_size > 1; lengths only with block_size 1. */
int flare_forward_uses_tensor_path(const flare_fwd_args_t* args);

/* 1 when flare_backward would take the tcgen05 tensor-core backward for this problem, else 0: the conditions of
 * flare_forward_uses_tensor_path plus M <= 256 at Dk = 128, a whole sequence (no span mode, no fwd.state_in) and
 * dense 16-byte aligned dY rows.  Everything else runs on the exact fp32 kernels. */
int flare_backward_uses_tensor_path(const flare_bwd_args_t* args);

/* Device-side health of the tensor-core kernels: synchronises the device and returns a bit set (0 = healthy), or a
 * negative flare_status on a CUDA error.  Bit 0 (1): a kernel gave up on a bounded wait, its outputs are invalid.
 * Bit 1 (2): some token's decode denominator underflowed or overflowed - the inputs are outside the numeric domain
 * of the tensor path (scores spread over more than ~80 nats); rerun with path = FLARE_PATH_EXACT.
 * reset != 0 clears the flags. */
int flare_device_status(int reset);
/* sizeof(flare_fwd_args_t / flare_bwd_args_t / flare_decode_args_t / flare_state_t) for which = 0..3,
 * so that a foreign-language binding can verify its struct layout at load time. */
size_t flare_abi_sizeof(int which);

#ifdef __cplusplus
}
#endif
#endif /* FLARE_B200_H_ */
