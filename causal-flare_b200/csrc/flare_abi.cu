// extern "C" entry points of libflare_b200.so: argument validation, launch planning, dispatch.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "bwd_exact.cuh"
#include "bwd_tc.cuh"
#include "decode_step.cuh"
#include "flare_common.cuh"
#include "prefill_tc.cuh"
#include "state_ops.cuh"
#include "walk_exact.cuh"

namespace flare {

static thread_local char g_cuda_error[512] = "";

void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
}

int sm_count() {
  constexpr int kMaxDevices = 64;
  static int cached[kMaxDevices] = {};  // per device ordinal; racing first calls write the same value
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 148;  // B200; used only for planning when no device is visible
  }
  if (dev >= 0 && dev < kMaxDevices && cached[dev] > 0) return cached[dev];
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    return 148;
  }
  if (dev >= 0 && dev < kMaxDevices) cached[dev] = n;
  return n;
}

// Optional CUDA events recorded around the dominant kernel of the next forward calls (benchmark hook).
static thread_local cudaEvent_t g_ev_begin = nullptr, g_ev_end = nullptr;
static thread_local int g_last_launches = 0;
static thread_local long long* g_trace = nullptr;
// per-chunk prefix states the next read-out pass of this thread's forward keeps for the backward (u == null: none)
static thread_local ChunkStates g_keep = {nullptr, nullptr, nullptr, 0};
// gate words of the tensor-core forward in flight on this thread (null: none), see FwdPlan::gate_bytes
static thread_local int* g_gate = nullptr;

void count_launches(int n) { g_last_launches += n; }

// ---- per-kernel profile records of this thread -----------------------------------------------------------
namespace {
struct ProfileRecord {
  const char* name;
  cudaEvent_t begin, end;
};
constexpr int kMaxProfileRecords = 256;
thread_local ProfileRecord g_prof[kMaxProfileRecords];
thread_local int g_prof_count = 0;
thread_local bool g_prof_on = false;

void profile_clear() {
  for (int i = 0; i < g_prof_count; ++i) {
    cudaEventDestroy(g_prof[i].begin);
    cudaEventDestroy(g_prof[i].end);
  }
  g_prof_count = 0;
}
}  // namespace

LaunchTimer::LaunchTimer(const char* name, cudaStream_t s) : slot(-1), stream(s) {
  if (!g_prof_on || g_prof_count >= kMaxProfileRecords) return;
  ProfileRecord& r = g_prof[g_prof_count];
  r.name = name;
  if (cudaEventCreate(&r.begin) != cudaSuccess) return;
  if (cudaEventCreate(&r.end) != cudaSuccess) {
    cudaEventDestroy(r.begin);
    return;
  }
  slot = g_prof_count++;
  cudaEventRecord(r.begin, stream);
}
LaunchTimer::~LaunchTimer() {
  if (slot >= 0) cudaEventRecord(g_prof[slot].end, stream);
}
long long* trace_buffer() { return g_trace; }

namespace {

struct DominantKernelTimer {
  cudaStream_t s;
  explicit DominantKernelTimer(cudaStream_t st) : s(st) {
    if (g_ev_begin) cudaEventRecord(g_ev_begin, s);
  }
  ~DominantKernelTimer() {
    if (g_ev_end) cudaEventRecord(g_ev_end, s);
  }
};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool mult8(int64_t x) { return (x % 8) == 0; }

int check_forward(const flare_fwd_args_t* a) {
  if (a == nullptr) return FLARE_ERR_BAD_POINTER;
  if (a->B < 0 || a->N < 0 || a->H <= 0 || a->M <= 0 || a->Dk <= 0 || a->Dv <= 0) return FLARE_ERR_BAD_SHAPE;
  if ((a->M % 16) || (a->Dk % 16) || (a->Dv % 16)) return FLARE_ERR_BAD_SHAPE;
  if (a->dtype != FLARE_F32 && a->dtype != FLARE_BF16 && a->dtype != FLARE_F16) return FLARE_ERR_BAD_DTYPE;
  if (a->variant != FLARE_SOFTMAX && a->variant != FLARE_STABLEMAX) return FLARE_ERR_BAD_CONFIG;
  if (a->block_size < 1) return FLARE_ERR_BAD_CONFIG;
  if (a->block_size > 1 && ((a->block_size % 16) || (a->N % a->block_size) || a->variant != FLARE_SOFTMAX ||
                            a->mask != nullptr))
    return FLARE_ERR_BAD_CONFIG;
  if (a->B == 0 || a->N == 0) return FLARE_OK;
  if (!a->q || !a->k || !a->v) return FLARE_ERR_BAD_POINTER;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->q_dec) || !aligned16(a->k_dec) ||
      !aligned16(a->y))
    return FLARE_ERR_BAD_POINTER;
  if (!mult8(a->q_stride_h) || !mult8(a->q_stride_m) || !mult8(a->k_stride_b) || !mult8(a->k_stride_n) ||
      !mult8(a->k_stride_h) || !mult8(a->v_stride_b) || !mult8(a->v_stride_n) || !mult8(a->v_stride_h))
    return FLARE_ERR_BAD_POINTER;
  if (a->q_dec && (!mult8(a->qd_stride_b) || !mult8(a->qd_stride_n) || !mult8(a->qd_stride_h))) return FLARE_ERR_BAD_POINTER;
  if (a->k_dec && (!mult8(a->kd_stride_h) || !mult8(a->kd_stride_m))) return FLARE_ERR_BAD_POINTER;
  if (a->y && (!mult8(a->y_stride_b) || !mult8(a->y_stride_n) || !mult8(a->y_stride_h))) return FLARE_ERR_BAD_POINTER;
  const bool any_in = a->state_in.m || a->state_in.d || a->state_in.u;
  if (any_in && !(a->state_in.m && a->state_in.d && a->state_in.u)) return FLARE_ERR_BAD_POINTER;
  const bool any_out = a->state_out.m || a->state_out.d || a->state_out.u;
  if (any_out && !(a->state_out.m && a->state_out.d && a->state_out.u)) return FLARE_ERR_BAD_POINTER;
  if (!a->y && !any_out) return FLARE_ERR_BAD_POINTER;
  if (a->lengths != nullptr && a->mask != nullptr) return FLARE_ERR_UNSUPPORTED;
  if (a->M > 512) return FLARE_ERR_UNSUPPORTED;
  return FLARE_OK;
}

struct FwdPlan {
  bool use_tc;
  int nseg;
  int seg_len;
  size_t state_floats;  // floats per state: 2M + M*Dv
  size_t ws_bytes;
  size_t part_off, part_bytes;  // tensor path with more than 128 latents: partial read-outs behind the segment states
  // Path AUTO on the tensor kernels: per-call gate words (1 + lanes ints) that the kernels raise for tokens outside
  // their numeric domain; the exact kernels then run for the flagged lanes only (0 bytes: no guard)
  size_t gate_off, gate_bytes;
};

FwdPlan plan_forward(const flare_fwd_args_t* a) {
  FwdPlan pl{false, 1, a->N > 0 ? a->N : 1, 0, 0, 0, 0, 0, 0};
  if (a->B == 0 || a->N == 0) return pl;
  const int64_t lanes = (int64_t)a->B * a->H;
  pl.state_floats = (size_t)2 * a->M + (size_t)a->M * a->Dv;
  if (a->path != FLARE_PATH_EXACT && prefill_tc_supported(a)) {
    // tensor-core path: one CTA per SM walks a (lane, segment); split the sequence only when lanes are scarce
    pl.use_tc = true;
    int nseg = 1;
    const int sms = sm_count();
    const int64_t ctas = lanes * prefill_tc_ctas_per_lane(a);
    if (ctas * 2 <= sms) {
      // as many segments as still fit the SMs in ONE wave (a second, partly filled wave costs more than it gains:
      // 64 lanes in 3 segments = 192 CTAs measured 0.140 ms for the read-out pass against 0.185 ms unsegmented,
      // plus 0.06 ms for the state-only pass and the fold)
      nseg = (int)(sms / ctas);
      const int max_seg = a->N / 256;
      if (nseg > max_seg) nseg = max_seg;
      if (nseg < 1) nseg = 1;
    }
    int seg_len = (a->N + nseg - 1) / nseg;
    seg_len = (seg_len + 127) / 128 * 128;
    pl.nseg = (a->N + seg_len - 1) / seg_len;
    pl.seg_len = seg_len;
    pl.ws_bytes = pl.nseg > 1 ? align_up((size_t)lanes * pl.nseg * pl.state_floats * 4, 256) : 0;
    pl.part_off = pl.ws_bytes;
    pl.part_bytes = a->y != nullptr ? align_up(prefill_tc_partial_bytes(a), 256) : 0;
    pl.ws_bytes += pl.part_bytes;
    if (a->path == FLARE_PATH_AUTO && a->lengths == nullptr) {
      pl.gate_off = pl.ws_bytes;
      pl.gate_bytes = align_up((size_t)(1 + lanes) * sizeof(int), 256);
      pl.ws_bytes += pl.gate_bytes;
    }
    return pl;
  }
  const int dd = walk_exact_dd(a->M, a->Dv);
  const int dtiles = (a->Dv + 32 * dd - 1) / (32 * dd);
  const int64_t ctas = lanes * dtiles;
  const int64_t slots = 2LL * sm_count();
  const int unit = a->block_size > 16 ? a->block_size : 16;
  int nseg = 1;
  if (ctas * 2 <= slots) {
    nseg = (int)((slots + ctas - 1) / ctas);
    const int max_seg = a->N / (4 * unit);
    if (nseg > max_seg) nseg = max_seg;
    if (nseg < 1) nseg = 1;
  }
  int seg_len = (a->N + nseg - 1) / nseg;
  seg_len = (seg_len + unit - 1) / unit * unit;
  nseg = (a->N + seg_len - 1) / seg_len;
  pl.nseg = nseg;
  pl.seg_len = seg_len;
  pl.state_floats = (size_t)2 * a->M + (size_t)a->M * a->Dv;
  pl.ws_bytes = nseg > 1 ? align_up((size_t)lanes * nseg * pl.state_floats * 4, 256) : 0;
  return pl;
}

void fill_walk(WalkParams& w, const flare_fwd_args_t* a) {
  memset(&w, 0, sizeof(w));
  w.q = a->q; w.k = a->k; w.v = a->v; w.qd = a->q_dec; w.kd = a->k_dec;
  w.y = a->y; w.mask = a->mask;
  w.B = a->B; w.N = a->N; w.H = a->H; w.M = a->M; w.Dk = a->Dk; w.Dv = a->Dv;
  w.q_stride_h = a->q_stride_h; w.q_stride_m = a->q_stride_m;
  w.k_stride_b = a->k_stride_b; w.k_stride_n = a->k_stride_n; w.k_stride_h = a->k_stride_h;
  w.v_stride_b = a->v_stride_b; w.v_stride_n = a->v_stride_n; w.v_stride_h = a->v_stride_h;
  w.qd_stride_b = a->qd_stride_b; w.qd_stride_n = a->qd_stride_n; w.qd_stride_h = a->qd_stride_h;
  w.kd_stride_h = a->kd_stride_h; w.kd_stride_m = a->kd_stride_m;
  w.y_stride_b = a->y_stride_b; w.y_stride_n = a->y_stride_n; w.y_stride_h = a->y_stride_h;
  w.scale = a->scale; w.power = a->power;
  w.dtype = a->dtype; w.variant = a->variant; w.block_size = a->block_size;
}

int launch_walk(const flare_fwd_args_t* a, const FwdPlan& pl, const WalkParams& w, int nseg_grid, cudaStream_t stream) {
  if (!pl.use_tc) return launch_walk_exact(w, nseg_grid, stream);
  TcParams t;
  memset(&t, 0, sizeof(t));
  t.y = w.write_y ? w.y : nullptr;
  t.y_stride_b = w.y_stride_b; t.y_stride_n = w.y_stride_n; t.y_stride_h = w.y_stride_h;
  t.q = w.q; t.q_stride_h = w.q_stride_h; t.q_stride_m = w.q_stride_m;
  t.N = w.N; t.H = w.H; t.M = w.M; t.Dv = w.Dv; t.scale = w.scale; t.seg_len = w.seg_len;
  t.in_m = w.in_m; t.in_d = w.in_d; t.in_u = w.in_u;
  t.in_lane_stride = w.in_lane_stride; t.in_seg_stride = w.in_seg_stride;
  t.out_m = w.out_m; t.out_d = w.out_d; t.out_u = w.out_u;
  t.out_lane_stride = w.out_lane_stride; t.out_seg_stride = w.out_seg_stride;
  t.out_mode = w.out_mode; t.nseg_total = w.nseg_total;
  if (pl.part_bytes > 0 && t.y != nullptr) {
    t.part_y = reinterpret_cast<char*>(a->workspace) + pl.part_off;
    t.part_lw = reinterpret_cast<float*>(reinterpret_cast<char*>(t.part_y) + prefill_tc_partial_lw_offset(a));
  }
  t.trace = g_trace;
  t.gate = g_gate;
  if (t.y != nullptr && g_keep.u != nullptr) {
    t.dump_u = g_keep.u; t.dump_c = g_keep.c; t.dump_d = g_keep.d; t.dump_nch = g_keep.nch;
  }
  return launch_prefill_tc(a, t, nseg_grid, stream);
}

int forward_tensor_or_exact(const flare_fwd_args_t* a, const FwdPlan& pl, cudaStream_t stream);

// The exact kernels standing by behind a tensor-core forward: one CTA per (lane, value tile) walks the whole sequence,
// but only for the lanes whose gate word the tensor kernels raised (inputs outside their numeric domain, e.g. score
// spreads of several hundred nats).  For in-domain calls this launch ends at once.
int launch_guard_walk(const flare_fwd_args_t* a, const int* lane_gates, cudaStream_t stream) {
  WalkParams w;
  fill_walk(w, a);
  w.seg_len = a->N;
  w.nseg_total = 1;
  w.in_m = a->state_in.m; w.in_d = a->state_in.d; w.in_u = a->state_in.u;
  w.in_lane_stride = 1; w.in_seg_stride = 0;
  w.out_m = a->state_out.m; w.out_d = a->state_out.d; w.out_u = a->state_out.u;
  w.out_lane_stride = 1; w.out_seg_stride = 0;
  w.out_mode = a->state_out.u != nullptr ? 2 : 0;
  w.write_y = a->y != nullptr;
  w.lse_dec = a->lse_dec; w.lse_enc = a->lse_enc;
  w.gate = lane_gates;
  w.gate_stride = 1;
  return launch_walk_exact(w, 1, stream);
}

// What an fp16 call that runs on bf16 copies (forward_cast below) still has to do once the tensor kernels are enqueued:
// y back to fp16, and then the standby walk of the flagged lanes on the caller's own fp16 tensors, so that the lanes
// whose score spreads left the tensor kernels' domain - where the rounding of q and k to bf16 would move the scores
// most - are computed from the unrounded inputs.
struct FinishCast {
  const flare_fwd_args_t* orig;
  const CastParams* y_back;  // null: no y wanted
  bool y_done;
};

int forward_run(const flare_fwd_args_t* a, cudaStream_t stream, FinishCast* fin = nullptr) {
  const FwdPlan pl = plan_forward(a);
  if (g_keep.u != nullptr) return forward_tensor_or_exact(a, pl, stream);  // the backward's own replay of the forward
  const int64_t lanes = (int64_t)a->B * a->H;
  int* gate = nullptr;
  size_t gate_bytes = 0;
  if (a->keep != nullptr) {
    // training: the chunk states and the gate words go to the caller's keep buffer
    const KeepLayout kl = keep_layout(*a);
    if (kl.total == 0 || !pl.use_tc || a->y == nullptr || a->lse_dec == nullptr || a->keep_bytes < kl.total ||
        (reinterpret_cast<uintptr_t>(a->keep) & 255u) != 0)
      return FLARE_ERR_BAD_CONFIG;
    char* kb = reinterpret_cast<char*>(a->keep);
    gate = reinterpret_cast<int*>(kb + kl.off_gate);
    gate_bytes = (size_t)(1 + lanes) * sizeof(int);
    g_keep = ChunkStates{kb + kl.off_u, reinterpret_cast<float*>(kb + kl.off_c), reinterpret_cast<float*>(kb + kl.off_d), kl.nch};
  } else if (pl.gate_bytes > 0) {
    if (a->workspace == nullptr || a->workspace_bytes < pl.ws_bytes || !aligned16(a->workspace)) return FLARE_ERR_WORKSPACE;
    gate = reinterpret_cast<int*>(reinterpret_cast<char*>(a->workspace) + pl.gate_off);
    gate_bytes = pl.gate_bytes;
  }
  if (gate == nullptr) return forward_tensor_or_exact(a, pl, stream);
  const cudaError_t e = cudaMemsetAsync(gate, 0, gate_bytes, stream);
  if (e != cudaSuccess) {
    g_keep = ChunkStates{nullptr, nullptr, nullptr, 0};
    set_cuda_error(e, "cudaMemsetAsync (gate words)");
    return FLARE_ERR_CUDA;
  }
  g_gate = gate;
  int rc = forward_tensor_or_exact(a, pl, stream);
  g_gate = nullptr;
  g_keep = ChunkStates{nullptr, nullptr, nullptr, 0};
  if (rc != FLARE_OK) return rc;
  if (a->path == FLARE_PATH_AUTO && a->lengths == nullptr) {
    const flare_fwd_args_t* walk_args = a;
    if (fin != nullptr) {
      if (fin->y_back != nullptr) {
        rc = launch_cast_rows(*fin->y_back, stream);
        if (rc != FLARE_OK) return rc;
        fin->y_done = true;
      }
      walk_args = fin->orig;
    }
    rc = launch_guard_walk(walk_args, gate + 1, stream);
    g_last_launches += 1;
  }
  return rc;
}

int forward_tensor_or_exact(const flare_fwd_args_t* a, const FwdPlan& pl, cudaStream_t stream) {
  if (a->lengths != nullptr && !pl.use_tc) return FLARE_ERR_UNSUPPORTED;  // per-row lengths exist on the tensor path only
  if (pl.ws_bytes > 0 && (a->workspace == nullptr || a->workspace_bytes < pl.ws_bytes || !aligned16(a->workspace)))
    return FLARE_ERR_WORKSPACE;
  const int64_t lanes = (int64_t)a->B * a->H;
  const bool have_out = a->state_out.u != nullptr;
  WalkParams w;
  fill_walk(w, a);
  w.seg_len = pl.seg_len;
  w.nseg_total = pl.nseg;
  if (pl.nseg == 1) {
    w.in_m = a->state_in.m; w.in_d = a->state_in.d; w.in_u = a->state_in.u;
    w.in_lane_stride = 1; w.in_seg_stride = 0;
    w.out_m = a->state_out.m; w.out_d = a->state_out.d; w.out_u = a->state_out.u;
    w.out_lane_stride = 1; w.out_seg_stride = 0;
    w.out_mode = have_out ? 2 : 0;
    w.write_y = a->y != nullptr;
    w.lse_dec = a->lse_dec; w.lse_enc = a->lse_enc;
    g_last_launches = 1 + ((pl.part_bytes > 0 && w.write_y) ? 1 : 0);  // + merge of the latent groups
    DominantKernelTimer timer(stream);
    return launch_walk(a, pl, w, 1, stream);
  }
  // segmented: (A) local state of every segment but the last, (B) exclusive scan with the carry-in,
  // (C) walk every segment from its prefix state and emit the outputs.
  float* seg_m = reinterpret_cast<float*>(a->workspace);
  float* seg_d = seg_m + (size_t)lanes * pl.nseg * a->M;
  float* seg_u = seg_d + (size_t)lanes * pl.nseg * a->M;
  WalkParams wa = w;
  wa.y = nullptr; wa.write_y = 0; wa.lse_dec = nullptr; wa.lse_enc = nullptr;
  wa.out_m = seg_m; wa.out_d = seg_d; wa.out_u = seg_u;
  wa.out_lane_stride = pl.nseg; wa.out_seg_stride = 1; wa.out_mode = 1;
  int rc = launch_walk(a, pl, wa, pl.nseg - 1, stream);
  if (rc != FLARE_OK) return rc;
  FoldParams f;
  memset(&f, 0, sizeof(f));
  f.a_m = a->state_in.m; f.a_d = a->state_in.d; f.a_u = a->state_in.u;
  f.s_m = seg_m; f.s_d = seg_d; f.s_u = seg_u;
  f.lane_stride = pl.nseg; f.seg_stride = 1; f.count = pl.nseg; f.mode = 0;
  f.lanes = lanes; f.M = a->M; f.Dv = a->Dv; f.stablemax = a->variant == FLARE_STABLEMAX;
  rc = launch_fold(f, stream);
  if (rc != FLARE_OK) return rc;
  w.in_m = seg_m; w.in_d = seg_d; w.in_u = seg_u;
  w.in_lane_stride = pl.nseg; w.in_seg_stride = 1;
  w.out_m = a->state_out.m; w.out_d = a->state_out.d; w.out_u = a->state_out.u;
  w.out_lane_stride = 1; w.out_seg_stride = 0;
  w.out_mode = have_out ? 2 : 0;
  w.write_y = a->y != nullptr;
  w.lse_dec = a->lse_dec; w.lse_enc = a->lse_enc;
  g_last_launches = 2;
  if (!w.write_y && !have_out) return FLARE_OK;
  g_last_launches = 3 + ((pl.part_bytes > 0 && w.write_y) ? 1 : 0);
  DominantKernelTimer timer(stream);
  return launch_walk(a, pl, w, pl.nseg, stream);
}

// fp16 inputs on the tensor-core kernels.  The kernels multiply bf16 operands (the tensor-core products of E, R, W
// and the running state are bf16 whatever the inputs are), so an fp16 call is served by rounding q, k, v to bf16
// copies in the workspace, running the bf16 forward on those, and writing y back as fp16: three streaming passes
// around a kernel that is 40 to 60 times faster than the exact walk the call would otherwise take.  Lanes that the
// kernels flag as outside their numeric domain are recomputed by the exact kernels from the fp16 tensors themselves.
// States and log-sum-exps are fp32 on both sides and go straight to the caller's buffers.  Not for the training
// forward (no state is kept for a backward) and not with separate decode weights or a mask, which the tensor kernels
// do not take.
struct CastPlan {
  bool on;
  size_t off_q, off_k, off_v, off_y, total;
};

CastPlan plan_cast(const flare_fwd_args_t* a, flare_fwd_args_t* b) {
  CastPlan cp{false, 0, 0, 0, 0, 0};
  if (a->dtype != FLARE_F16 || a->path == FLARE_PATH_EXACT || a->keep != nullptr || a->q_dec != nullptr ||
      a->k_dec != nullptr || a->mask != nullptr || a->B == 0 || a->N == 0)
    return cp;
  // FLARE_B200_FP16_TENSOR=0 keeps fp16 calls on the exact kernels (q, k, v at their full fp16 precision)
  if (const char* env = getenv("FLARE_B200_FP16_TENSOR"))
    if (env[0] == '0') return cp;
  *b = *a;
  b->dtype = FLARE_BF16;
  b->q_stride_m = a->Dk; b->q_stride_h = (int64_t)a->M * a->Dk;
  b->k_stride_h = a->Dk; b->k_stride_n = (int64_t)a->H * a->Dk; b->k_stride_b = (int64_t)a->N * b->k_stride_n;
  b->v_stride_h = a->Dv; b->v_stride_n = (int64_t)a->H * a->Dv; b->v_stride_b = (int64_t)a->N * b->v_stride_n;
  b->y_stride_h = a->Dv; b->y_stride_n = (int64_t)a->H * a->Dv; b->y_stride_b = (int64_t)a->N * b->y_stride_n;
  if (!prefill_tc_supported(b)) return cp;
  const size_t rows = (size_t)a->B * a->N * a->H;
  cp.on = true;
  cp.off_q = 0;
  cp.off_k = align_up((size_t)a->H * a->M * a->Dk * 2, 256);
  cp.off_v = cp.off_k + align_up(rows * a->Dk * 2, 256);
  cp.off_y = cp.off_v + align_up(rows * a->Dv * 2, 256);
  cp.total = cp.off_y + (a->y != nullptr ? align_up(rows * a->Dv * 2, 256) : 0);
  return cp;
}

int forward_cast(const flare_fwd_args_t* a, flare_fwd_args_t& b, const CastPlan& cp, cudaStream_t stream) {
  const size_t inner = plan_forward(&b).ws_bytes;
  if (a->workspace == nullptr || a->workspace_bytes < cp.total + inner || !aligned16(a->workspace)) return FLARE_ERR_WORKSPACE;
  char* ws = reinterpret_cast<char*>(a->workspace);
  b.q = ws + cp.off_q; b.k = ws + cp.off_k; b.v = ws + cp.off_v;
  b.y = a->y != nullptr ? ws + cp.off_y : nullptr;
  b.workspace = inner > 0 ? ws + cp.total : nullptr;
  b.workspace_bytes = inner > 0 ? a->workspace_bytes - cp.total : 0;
  CastParams c;
  memset(&c, 0, sizeof(c));
  c.in = a->q; c.out = const_cast<void*>(b.q); c.n0 = 1; c.n1 = a->H; c.n2 = a->M; c.d = a->Dk;
  c.is1 = a->q_stride_h; c.is2 = a->q_stride_m; c.os1 = b.q_stride_h; c.os2 = b.q_stride_m;
  int rc = launch_cast_rows(c, stream);
  if (rc != FLARE_OK) return rc;
  c.in = a->k; c.out = const_cast<void*>(b.k); c.n0 = a->B; c.n1 = a->N; c.n2 = a->H; c.d = a->Dk;
  c.is0 = a->k_stride_b; c.is1 = a->k_stride_n; c.is2 = a->k_stride_h;
  c.os0 = b.k_stride_b; c.os1 = b.k_stride_n; c.os2 = b.k_stride_h;
  rc = launch_cast_rows(c, stream);
  if (rc != FLARE_OK) return rc;
  c.in = a->v; c.out = const_cast<void*>(b.v); c.d = a->Dv;
  c.is0 = a->v_stride_b; c.is1 = a->v_stride_n; c.is2 = a->v_stride_h;
  c.os0 = b.v_stride_b; c.os1 = b.v_stride_n; c.os2 = b.v_stride_h;
  rc = launch_cast_rows(c, stream);
  if (rc != FLARE_OK) return rc;
  CastParams yb = c;
  yb.in = b.y; yb.out = a->y; yb.to_f16 = 1;
  yb.is0 = b.y_stride_b; yb.is1 = b.y_stride_n; yb.is2 = b.y_stride_h;
  yb.os0 = a->y_stride_b; yb.os1 = a->y_stride_n; yb.os2 = a->y_stride_h;
  FinishCast fin{a, a->y != nullptr ? &yb : nullptr, false};
  rc = forward_run(&b, stream, &fin);  // gate words in b's workspace; the standby walk reads the caller's fp16 tensors
  if (rc != FLARE_OK) return rc;
  int casts = 3;
  if (a->y != nullptr) {
    if (!fin.y_done) {  // no standby on this path (forced tensor path, per-row lengths)
      rc = launch_cast_rows(yb, stream);
      if (rc != FLARE_OK) return rc;
    }
    ++casts;
  }
  g_last_launches += casts;
  return FLARE_OK;
}

}  // namespace

int forward_keep_states(const flare_fwd_args_t* a, const ChunkStates& keep, int* gate, cudaStream_t stream) {
  const int rc = check_forward(a);
  if (rc != FLARE_OK) return rc;
  if (!plan_forward(a).use_tc) return FLARE_ERR_UNSUPPORTED;
  g_keep = keep;
  g_gate = gate;  // raised by the kernels when a token leaves their numeric domain; no exact rerun here
  const int rc2 = forward_run(a, stream);
  g_gate = nullptr;
  g_keep = ChunkStates{nullptr, nullptr, nullptr, 0};
  return rc2;
}

int segment_prefix_states(const flare_fwd_args_t* f, int nseg, int seg_len, float* seg_m, float* seg_d, float* seg_u,
                          const flare_state_t* init, cudaStream_t stream, const int* gate) {
  flare_fwd_args_t a = *f;
  a.y = nullptr;
  a.mask = nullptr;
  a.lse_dec = a.lse_enc = nullptr;
  a.block_size = 1;  // the state at a segment boundary does not depend on the read-out mode
  memset(&a.state_in, 0, sizeof(a.state_in));
  memset(&a.state_out, 0, sizeof(a.state_out));
  a.state_out.m = seg_m; a.state_out.d = seg_d; a.state_out.u = seg_u;  // marks "a state is wanted" for the checks
  FwdPlan pl{false, nseg, seg_len, (size_t)2 * a.M + (size_t)a.M * a.Dv, 0, 0, 0, 0, 0};
  pl.use_tc = a.path != FLARE_PATH_EXACT && (seg_len % 128) == 0 && prefill_tc_supported(&a);
  const int64_t lanes = (int64_t)a.B * a.H;
  WalkParams w;
  fill_walk(w, &a);
  w.seg_len = seg_len;
  w.nseg_total = nseg;
  w.y = nullptr; w.write_y = 0;
  w.out_m = seg_m; w.out_d = seg_d; w.out_u = seg_u;
  w.out_lane_stride = nseg; w.out_seg_stride = 1; w.out_mode = 1;
  w.gate = gate; w.gate_stride = 0;  // (a gated pass always runs on the exact kernels: its caller forces that path)
  if (nseg > 1) {
    const int rc = launch_walk(&a, pl, w, nseg - 1, stream);  // local states of all segments but the last
    if (rc != FLARE_OK) return rc;
  }
  FoldParams fp;
  memset(&fp, 0, sizeof(fp));
  if (init != nullptr) {
    fp.a_m = init->m; fp.a_d = init->d; fp.a_u = init->u;
  }
  fp.s_m = seg_m; fp.s_d = seg_d; fp.s_u = seg_u;
  fp.lane_stride = nseg; fp.seg_stride = 1; fp.count = nseg; fp.mode = 0;
  fp.lanes = lanes; fp.M = a.M; fp.Dv = a.Dv; fp.stablemax = a.variant == FLARE_STABLEMAX;
  fp.gate = gate;
  return launch_fold(fp, stream);  // exclusive scan from the initial (or empty) state
}

}  // namespace flare

using namespace flare;

extern "C" {

size_t flare_forward_workspace_bytes(const flare_fwd_args_t* args) {
  if (check_forward(args) != FLARE_OK) return 0;
  flare_fwd_args_t b;
  const CastPlan cp = plan_cast(args, &b);
  if (cp.on) return cp.total + plan_forward(&b).ws_bytes;
  return plan_forward(args).ws_bytes;
}

size_t flare_forward_keep_bytes(const flare_fwd_args_t* args) {
  if (check_forward(args) != FLARE_OK || args->B == 0 || args->N == 0) return 0;
  if (!plan_forward(args).use_tc) return 0;
  return keep_layout(*args).total;
}

int flare_forward(const flare_fwd_args_t* args, flare_stream_t stream) {
  const int rc = check_forward(args);
  if (rc != FLARE_OK) return rc;
  if (args->B == 0 || args->N == 0) {
    // empty sequence: the state passes through unchanged
    if (args->state_out.u != nullptr && args->B > 0) {
      FoldParams f;
      memset(&f, 0, sizeof(f));
      f.a_m = args->state_in.m; f.a_d = args->state_in.d; f.a_u = args->state_in.u;
      f.count = 0; f.mode = 1;
      f.o_m = args->state_out.m; f.o_d = args->state_out.d; f.o_u = args->state_out.u;
      f.lanes = (int64_t)args->B * args->H; f.M = args->M; f.Dv = args->Dv;
      f.stablemax = args->variant == FLARE_STABLEMAX;
      f.count = 1; f.mode = 0;  // degenerate scan: writes `a` into slot 0 = the output state
      f.s_m = f.o_m; f.s_d = f.o_d; f.s_u = f.o_u; f.lane_stride = 1; f.seg_stride = 0;
      return launch_fold(f, stream);
    }
    return FLARE_OK;
  }
  flare_fwd_args_t b;
  const CastPlan cp = plan_cast(args, &b);
  if (cp.on) return forward_cast(args, b, cp, stream);
  return forward_run(args, stream);
}

static int check_backward(const flare_bwd_args_t* args) {
  if (args == nullptr) return FLARE_ERR_BAD_POINTER;
  flare_fwd_args_t chk = args->fwd;
  chk.y = const_cast<void*>(args->dy);  // reuse the forward validation for the shared fields
  chk.y_stride_b = args->dy_stride_b; chk.y_stride_n = args->dy_stride_n; chk.y_stride_h = args->dy_stride_h;
  chk.mask = nullptr;
  chk.state_in = flare_state_t{nullptr, nullptr, nullptr};
  chk.state_out = flare_state_t{nullptr, nullptr, nullptr};
  const int rc = check_forward(&chk);
  if (rc != FLARE_OK) return rc;
  if (args->fwd.B == 0 || args->fwd.N == 0) return FLARE_OK;
  if (!args->dq || !args->dk || !args->dv || !args->dy) return FLARE_ERR_BAD_POINTER;
  if ((args->fwd.q_dec != nullptr) != (args->dq_dec != nullptr)) return FLARE_ERR_BAD_POINTER;
  if ((args->fwd.k_dec != nullptr) != (args->dk_dec != nullptr)) return FLARE_ERR_BAD_POINTER;
  return FLARE_OK;
}

// fp16 gradients on the tensor-core backward, the same way as the fp16 forward: bf16 copies of q, k, v and dY in the
// workspace, the bf16 backward (with its own replay of the forward, gate and exact standby) on those, dK and dV
// written back as fp16; dQ is fp32 on both sides.
namespace {
struct BwdCastPlan {
  bool on;
  size_t off_q, off_k, off_v, off_dy, off_dk, off_dv, total;
};

BwdCastPlan plan_bwd_cast(const flare_bwd_args_t* a, flare_bwd_args_t* b) {
  BwdCastPlan cp;
  memset(&cp, 0, sizeof(cp));
  const flare_fwd_args_t& f = a->fwd;
  if (f.dtype != FLARE_F16 || f.path == FLARE_PATH_EXACT || f.q_dec != nullptr || f.k_dec != nullptr || f.B == 0 || f.N == 0)
    return cp;
  if (const char* env = getenv("FLARE_B200_FP16_TENSOR"))
    if (env[0] == '0') return cp;
  *b = *a;
  flare_fwd_args_t& g = b->fwd;
  g.dtype = FLARE_BF16;
  g.q_stride_m = f.Dk; g.q_stride_h = (int64_t)f.M * f.Dk;
  g.k_stride_h = f.Dk; g.k_stride_n = (int64_t)f.H * f.Dk; g.k_stride_b = (int64_t)f.N * g.k_stride_n;
  g.v_stride_h = f.Dv; g.v_stride_n = (int64_t)f.H * f.Dv; g.v_stride_b = (int64_t)f.N * g.v_stride_n;
  b->dy_stride_h = f.Dv; b->dy_stride_n = (int64_t)f.H * f.Dv; b->dy_stride_b = (int64_t)f.N * b->dy_stride_n;
  g.keep = nullptr; g.keep_bytes = 0;  // an fp16 forward keeps nothing: the backward replays it
  b->y = nullptr; b->lse_dec = nullptr;
  if (!bwd_tc_supported(*b)) return cp;
  const size_t rows = (size_t)f.B * f.N * f.H;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off += align_up(bytes, 256);
    return o;
  };
  cp.on = true;
  cp.off_q = take((size_t)f.H * f.M * f.Dk * 2);
  cp.off_k = take(rows * f.Dk * 2);
  cp.off_v = take(rows * f.Dv * 2);
  cp.off_dy = take(rows * f.Dv * 2);
  cp.off_dk = take(rows * f.Dk * 2);
  cp.off_dv = take(rows * f.Dv * 2);
  cp.total = off;
  return cp;
}

int backward_cast(const flare_bwd_args_t* a, flare_bwd_args_t& b, const BwdCastPlan& cp, cudaStream_t stream) {
  const flare_fwd_args_t& f = a->fwd;
  const size_t inner = bwd_tc_workspace_bytes(b);
  if (f.workspace == nullptr || f.workspace_bytes < cp.total + inner || (reinterpret_cast<uintptr_t>(f.workspace) & 255u))
    return FLARE_ERR_WORKSPACE;
  char* ws = reinterpret_cast<char*>(f.workspace);
  flare_fwd_args_t& g = b.fwd;
  g.q = ws + cp.off_q; g.k = ws + cp.off_k; g.v = ws + cp.off_v;
  b.dy = ws + cp.off_dy; b.dk = ws + cp.off_dk; b.dv = ws + cp.off_dv;
  g.workspace = ws + cp.total;
  g.workspace_bytes = f.workspace_bytes - cp.total;
  CastParams c;
  memset(&c, 0, sizeof(c));
  c.in = f.q; c.out = const_cast<void*>(g.q); c.n0 = 1; c.n1 = f.H; c.n2 = f.M; c.d = f.Dk;
  c.is1 = f.q_stride_h; c.is2 = f.q_stride_m; c.os1 = g.q_stride_h; c.os2 = g.q_stride_m;
  int rc = launch_cast_rows(c, stream);
  if (rc != FLARE_OK) return rc;
  c.in = f.k; c.out = const_cast<void*>(g.k); c.n0 = f.B; c.n1 = f.N; c.n2 = f.H; c.d = f.Dk;
  c.is0 = f.k_stride_b; c.is1 = f.k_stride_n; c.is2 = f.k_stride_h;
  c.os0 = g.k_stride_b; c.os1 = g.k_stride_n; c.os2 = g.k_stride_h;
  rc = launch_cast_rows(c, stream);
  if (rc != FLARE_OK) return rc;
  c.in = f.v; c.out = const_cast<void*>(g.v); c.d = f.Dv;
  c.is0 = f.v_stride_b; c.is1 = f.v_stride_n; c.is2 = f.v_stride_h;
  c.os0 = g.v_stride_b; c.os1 = g.v_stride_n; c.os2 = g.v_stride_h;
  rc = launch_cast_rows(c, stream);
  if (rc != FLARE_OK) return rc;
  c.in = a->dy; c.out = const_cast<void*>(b.dy);
  c.is0 = a->dy_stride_b; c.is1 = a->dy_stride_n; c.is2 = a->dy_stride_h;
  c.os0 = b.dy_stride_b; c.os1 = b.dy_stride_n; c.os2 = b.dy_stride_h;
  rc = launch_cast_rows(c, stream);
  if (rc != FLARE_OK) return rc;
  rc = bwd_tc(b, stream);
  if (rc != FLARE_OK) return rc;
  c.to_f16 = 1;
  c.in = b.dv; c.out = a->dv;
  c.is0 = c.os0 = b.dy_stride_b; c.is1 = c.os1 = b.dy_stride_n; c.is2 = c.os2 = b.dy_stride_h;
  rc = launch_cast_rows(c, stream);
  if (rc != FLARE_OK) return rc;
  c.in = b.dk; c.out = a->dk; c.d = f.Dk;
  c.is0 = c.os0 = g.k_stride_b; c.is1 = c.os1 = g.k_stride_n; c.is2 = c.os2 = g.k_stride_h;
  rc = launch_cast_rows(c, stream);
  if (rc != FLARE_OK) return rc;
  g_last_launches += 6;
  return FLARE_OK;
}
}  // namespace

size_t flare_backward_workspace_bytes(const flare_bwd_args_t* args) {
  if (check_backward(args) != FLARE_OK) return 0;
  {
    flare_bwd_args_t b;
    const BwdCastPlan cp = plan_bwd_cast(args, &b);
    if (cp.on) return cp.total + bwd_tc_workspace_bytes(b);
  }
  if (bwd_tc_supported(*args)) return bwd_tc_workspace_bytes(*args);
  return bwd_exact_workspace_bytes(*args);
}

int flare_backward(const flare_bwd_args_t* args, flare_stream_t stream) {
  const int rc = check_backward(args);
  if (rc != FLARE_OK) return rc;
  g_last_launches = 0;
  {
    flare_bwd_args_t b;
    const BwdCastPlan cp = plan_bwd_cast(args, &b);
    if (cp.on) return backward_cast(args, b, cp, stream);
  }
  if (bwd_tc_supported(*args)) return bwd_tc(*args, stream);
  return bwd_exact(*args, stream);
}

int flare_decode_step(const flare_decode_args_t* a, flare_stream_t stream) {
  if (a == nullptr) return FLARE_ERR_BAD_POINTER;
  if (a->B < 0 || a->H <= 0 || a->M <= 0 || a->Dk <= 0 || a->Dv <= 0) return FLARE_ERR_BAD_SHAPE;
  if ((a->M % 16) || (a->Dk % 16) || (a->Dv % 16)) return FLARE_ERR_BAD_SHAPE;
  if (a->dtype != FLARE_F32 && a->dtype != FLARE_BF16 && a->dtype != FLARE_F16) return FLARE_ERR_BAD_DTYPE;
  if (a->B == 0) return FLARE_OK;
  if (!a->q || !a->k || !a->v || !a->y || !a->state.m || !a->state.d || !a->state.u) return FLARE_ERR_BAD_POINTER;
  if (!aligned16(a->q) || !aligned16(a->k_dec) || !aligned16(a->y) || !aligned16(a->state.u)) return FLARE_ERR_BAD_POINTER;
  if (!mult8(a->q_stride_h) || !mult8(a->q_stride_m)) return FLARE_ERR_BAD_POINTER;
  if (a->k_dec && (!mult8(a->kd_stride_h) || !mult8(a->kd_stride_m))) return FLARE_ERR_BAD_POINTER;
  if (!decode_step_supported(a->M, a->Dk, a->Dv)) return FLARE_ERR_UNSUPPORTED;
  DecodeParams p;
  memset(&p, 0, sizeof(p));
  p.q = a->q; p.k = a->k; p.v = a->v; p.qd = a->q_dec; p.kd = a->k_dec; p.y = a->y; p.mask = a->mask;
  p.m = a->state.m; p.d = a->state.d; p.u = a->state.u;
  p.B = a->B; p.H = a->H; p.M = a->M; p.Dk = a->Dk; p.Dv = a->Dv;
  p.q_stride_h = a->q_stride_h; p.q_stride_m = a->q_stride_m;
  p.k_stride_b = a->k_stride_b; p.k_stride_h = a->k_stride_h;
  p.v_stride_b = a->v_stride_b; p.v_stride_h = a->v_stride_h;
  p.qd_stride_b = a->qd_stride_b; p.qd_stride_h = a->qd_stride_h;
  p.kd_stride_h = a->kd_stride_h; p.kd_stride_m = a->kd_stride_m;
  p.scale = a->scale; p.dtype = a->dtype;
  return launch_decode_step(p, stream);
}

int flare_state_merge(const flare_state_t* a, const flare_state_t* b, const flare_state_t* out, int64_t lanes, int32_t M,
                      int32_t Dv, int32_t count, flare_stream_t stream) {
  if (!a || !b || !out || !b->m || !b->d || !b->u || !out->m || !out->d || !out->u) return FLARE_ERR_BAD_POINTER;
  if (lanes < 0 || M <= 0 || Dv <= 0 || count < 1) return FLARE_ERR_BAD_SHAPE;
  FoldParams f;
  memset(&f, 0, sizeof(f));
  f.a_m = a->m; f.a_d = a->d; f.a_u = a->u;
  f.s_m = b->m; f.s_d = b->d; f.s_u = b->u;
  f.lane_stride = 1; f.seg_stride = lanes; f.count = count; f.mode = 1;
  f.o_m = out->m; f.o_d = out->d; f.o_u = out->u;
  f.lanes = lanes; f.M = M; f.Dv = Dv;
  return launch_fold(f, stream);
}

const char* flare_status_string(int status) {
  switch (status) {
    case FLARE_OK: return "ok";
    case FLARE_ERR_BAD_SHAPE: return "bad shape: sizes must be positive and M, Dk, Dv multiples of 16";
    case FLARE_ERR_UNSUPPORTED: return "shape not supported by the kernels";
    case FLARE_ERR_BAD_POINTER: return "missing tensor, or pointer/stride not 16-byte aligned";
    case FLARE_ERR_WORKSPACE: return "workspace missing or too small";
    case FLARE_ERR_BAD_DTYPE: return "unsupported dtype";
    case FLARE_ERR_BAD_CONFIG: return "invalid variant / block_size / mask combination";
    case FLARE_ERR_CUDA: return "CUDA runtime error";
    case FLARE_ERR_TOO_LARGE: return "request exceeds the fixed capacity of this entry point";
    default: return "unknown status";
  }
}

const char* flare_last_cuda_error(void) { return g_cuda_error; }

int flare_abi_version(void) { return 2; }

void flare_profile_enable(int on) {
  if (on) profile_clear();
  g_prof_on = on != 0;
}
int flare_profile_count(void) { return g_prof_count; }
int flare_profile_entry(int i, const char** name, float* ms) {
  if (i < 0 || i >= g_prof_count || name == nullptr || ms == nullptr) return FLARE_ERR_BAD_POINTER;
  FLARE_CUDA_CHECK(cudaEventSynchronize(g_prof[i].end));
  FLARE_CUDA_CHECK(cudaEventElapsedTime(ms, g_prof[i].begin, g_prof[i].end));
  *name = g_prof[i].name;
  return FLARE_OK;
}

void flare_set_kernel_events(void* begin_event, void* end_event) {
  g_ev_begin = static_cast<cudaEvent_t>(begin_event);
  g_ev_end = static_cast<cudaEvent_t>(end_event);
}

int flare_last_launch_count(void) { return g_last_launches; }

void flare_set_trace_buffer(void* device_buffer) { g_trace = static_cast<long long*>(device_buffer); }

int flare_forward_uses_tensor_path(const flare_fwd_args_t* args) {
  if (check_forward(args) != FLARE_OK) return 0;
  flare_fwd_args_t b;
  if (plan_cast(args, &b).on) return 1;
  return plan_forward(args).use_tc ? 1 : 0;
}

int flare_backward_uses_tensor_path(const flare_bwd_args_t* args) {
  if (check_backward(args) != FLARE_OK) return 0;
  flare_bwd_args_t b;
  if (plan_bwd_cast(args, &b).on) return 1;
  return bwd_tc_supported(*args) ? 1 : 0;
}

int flare_device_status(int reset) {
  int v = 0;
  const int rc = prefill_tc_error_flag(&v, reset != 0);
  if (rc != FLARE_OK) return -rc;
  return v;
}

/* sizeof of the argument structs, so a foreign-language binding can verify its own layout */
size_t flare_abi_sizeof(int which) {
  switch (which) {
    case 0: return sizeof(flare_fwd_args_t);
    case 1: return sizeof(flare_bwd_args_t);
    case 2: return sizeof(flare_decode_args_t);
    case 3: return sizeof(flare_state_t);
    default: return 0;
  }
}

}  // extern "C"
