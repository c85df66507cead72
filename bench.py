"""Benchmark of the Causal FLARE hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--skip-decode]

One JSON line on stdout (rank 0).  Metric: chunked causal prefill throughput in Mtok/s on the
BASELINE "C2" workload (B=8, N=8192, H=16, M=128 latents, D=64, bf16 in / fp32 accumulate), one full
workload per GPU (weak scaling: batch x head lanes are independent, no data-path collective).
A step = one forward over the whole batch.  Extra keys: ``decode`` (C3: 512 single-token steps on a
B=64, H=32, M=256, D=128 fp32 state, tok/s and achieved HBM GB/s), ``roofline``, ``cpu_baseline``,
``e2e`` (host buffers, copies inside the timed region), ``clocks``, ``gpu_launches``.

``--impl reference`` times the reference algorithm's CPU path (the oracle port of the reference's
PyTorch loop) on the host cores, on a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "causal-flare_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

C2 = dict(B=8, N=8192, H=16, M=128, Dk=64, Dv=64)
C3 = dict(B=64, H=32, M=256, Dk=128, Dv=128, prefix=32768, steps=512)
L2_BYTES = 126e6


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the GPU runs the timed workload.

    nvidia-smi takes a while to come up and its start-up holds driver locks that stall kernel launches, so the sampler
    is started - and has delivered its first sample - before the warm-up; ``begin()`` marks the start of the timed
    region, and ``hold_load()`` keeps the same (untimed) workload running after it until a few samples have been taken
    under that load (the timed region itself is a few milliseconds).  One process, on rank 0, samples all GPUs of the
    job: every query takes driver locks that delay launches on every GPU of the node, and eight pollers at 20 ms cost
    the slowest of eight ranks 0.7 ms of a 10 ms timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, indices, active: bool = True):
        self.indices = list(indices)
        self.active = active
        self.samples = []
        self.first = 0  # samples before this index were taken before the timed region
        self.proc = None
        self.up = threading.Event()

    def __enter__(self):
        if not self.active:
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", ",".join(str(i) for i in self.indices), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20" if len(self.indices) == 1 else "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            self.up.wait(timeout=3.0)
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)
                self.up.set()

    def begin(self):
        self.first = len(self.samples)

    def hold_load(self, fn, polls=4, max_seconds=0.5):
        """Run ``fn`` (the timed step, now untimed) until ``polls`` queries have been answered since ``begin()``; ranks
        without the sampler keep their GPU under the same load for as long as that takes at most."""
        if self.active and (self.proc is None or not self.up.is_set()):
            return
        end = time.monotonic() + (max_seconds if self.active else 0.3)
        want = polls * len(self.indices)
        while (not self.active or len(self.samples) - self.first < want) and time.monotonic() < end:
            for _ in range(8):
                fn()
            torch.cuda.current_stream().synchronize()

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        rows = self.samples[self.first:] or self.samples
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(s[0]) for s in rows if s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in rows if s[1].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(rows)}


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def device_inputs(cfg, seed, dtype=torch.bfloat16):
    """N(0,1) inputs generated on the device from a seeded generator (values only matter statistically here;
    the parity tests use the CPU-seeded generator shared with the oracle)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(cfg["H"], cfg["M"], cfg["Dk"], generator=g, device="cuda").to(dtype)
    k = torch.randn(cfg["B"], cfg["N"], cfg["H"], cfg["Dk"], generator=g, device="cuda").to(dtype)
    v = torch.randn(cfg["B"], cfg["N"], cfg["H"], cfg["Dv"], generator=g, device="cuda").to(dtype)
    return q, k, v


def bench_prefill(args, rank, world):
    import causal_flare as cf
    from causal_flare import _lib

    lib = _lib.load()
    cfg = C2
    q, k, v = device_inputs(cfg, seed=1234 + rank)
    tokens = cfg["B"] * cfg["N"]
    fn = lambda: cf.flare_autoregressive_triton(q, k, v)  # noqa: E731

    ev_b = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ev_e = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    for e in ev_b + ev_e:
        e.record()  # materialise the handles
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    with ClockSampler(range(world), active=rank == 0) as clk:
        for _ in range(args.warmup):
            fn()
        barrier(world)
        clk.begin()
        t0.record()
        for i in range(args.steps):
            lib.flare_set_kernel_events(ev_b[i].cuda_event, ev_e[i].cuda_event)
            y = fn()
        t1.record()
        lib.flare_set_kernel_events(None, None)
        barrier(world)
        clk.hold_load(fn)  # the same workload, untimed, until nvidia-smi has sampled it a few times
    launches = lib.flare_last_launch_count() * args.steps
    ms = t0.elapsed_time(t1)
    ms = max_over_ranks(ms, world)
    kern_ms = statistics.mean(b.elapsed_time(e) for b, e in zip(ev_b, ev_e))
    value = world * tokens * args.steps / (ms * 1e-3) / 1e6

    # ---- end to end: pinned host buffers in, result back to the host, every step ---------------------
    kh, vh = k.cpu().pin_memory(), v.cpu().pin_memory()
    yh = torch.empty(y.shape, dtype=y.dtype).pin_memory()
    kd, vd = torch.empty_like(k), torch.empty_like(v)

    # The batch is cut into slices that flow through three streams (upload, kernels, download) linked by events, so
    # the upload engine never waits for a download and consecutive steps overlap (PCIe is full duplex).
    n_slices = 8
    bs = cfg["B"] // n_slices
    s_in, s_cp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(n_slices)]
    ev_cp = [torch.cuda.Event() for _ in range(n_slices)]

    def e2e_step():
        for sl in range(n_slices):
            rows = slice(sl * bs, (sl + 1) * bs)
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_cp[sl])  # the previous step's kernels have read this slice of the device buffers
                kd[rows].copy_(kh[rows], non_blocking=True)
                vd[rows].copy_(vh[rows], non_blocking=True)
                ev_in[sl].record(s_in)
            with torch.cuda.stream(s_cp):
                s_cp.wait_event(ev_in[sl])
                yy = cf.flare_autoregressive_triton(q, kd[rows], vd[rows])
                ev_cp[sl].record(s_cp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cp[sl])
                yh[rows].copy_(yy, non_blocking=True)
                yy.record_stream(s_out)

    def e2e_join():
        cur = torch.cuda.current_stream()
        for st in (s_in, s_cp, s_out):
            cur.wait_stream(st)

    e2e_steps = max(2, min(args.steps, 5))
    if args.skip_e2e:
        e2e_steps = 0
        return dict(value=value, ms_per_step=ms / args.steps, e2e=None, roofline=_roofline(cfg, q, k, v, y, kern_ms),
                    clocks=clk.summary(), gpu_launches=launches, tokens_per_step=tokens)
    for st in (s_in, s_cp, s_out):
        st.wait_stream(torch.cuda.current_stream())
    e2e_step()
    e2e_join()
    barrier(world)
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for st in (s_in, s_cp, s_out):
        st.wait_stream(torch.cuda.current_stream())
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()
    s1.record()
    barrier(world)
    e2e_ms = max_over_ranks(s0.elapsed_time(s1), world)
    e2e = {
        "value": world * tokens * e2e_steps / (e2e_ms * 1e-3) / 1e6, "unit": "Mtok/s",
        "h2d_bytes_per_step": kh.numel() * 2 + vh.numel() * 2, "d2h_bytes_per_step": yh.numel() * 2,
        "steps": e2e_steps, "call": "causal_flare.flare_autoregressive_triton(q, k[rows], v[rows]) per batch row, "
        "upload / kernel / download streams linked by events, pinned host K/V in and Y out",
    }

    return dict(value=value, ms_per_step=ms / args.steps, e2e=e2e, roofline=_roofline(cfg, q, k, v, y, kern_ms),
                clocks=clk.summary(), gpu_launches=launches, tokens_per_step=tokens)


# DRAM traffic of one C2 forward launch as measured by ncu (268.8 MB read + 106.3 MB written; part of Y is still in L2
# when the kernel ends, hence below the algorithmic bytes)
NCU_TRAFFIC_C2_BYTES = 375_030_000
# DRAM traffic of one C3 decode step as measured by ncu (profiles/decode_step_c3.md)
NCU_TRAFFIC_C3_STEP_BYTES = 500_000_000


def _roofline(cfg, q, k, v, y, kern_ms):
    """Algorithmic bytes of one forward = K + V read, Y written, Q read (bf16) over the dominant kernel's time."""
    pk = peaks()
    alg_bytes = (k.numel() + v.numel() + y.numel()) * 2 + q.numel() * 2
    alg_flops = 6.0 * cfg["M"] * cfg["Dk"] * cfg["B"] * cfg["N"] * cfg["H"]
    achieved = alg_bytes / (kern_ms * 1e-3) / 1e9
    return {
        "bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
        "traffic": NCU_TRAFFIC_C2_BYTES, "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu "
        "capture of this kernel on this workload (profiles/prefill_tc_c2.md)", "peak_source": pk["source"],
        "kernel_ms": kern_ms,
        "kernel": "dominant forward kernel (CUDA events recorded around it inside flare_forward)",
        "algorithmic_bytes": alg_bytes,
        "tensor_frac": alg_flops / (kern_ms * 1e-3) / 1e12 / pk["bf16_tflops"],
    }


def _shape_roofline(rows, M, Dk, Dv, ms, flops_per_md, tensors):
    """Both roofline fractions of a whole step timed with CUDA events: algorithmic bytes (`tensors` bf16 tensors of
    `rows` x D) over the measured HBM peak, algorithmic flops (flops_per_md x M x D per row) over the measured bf16 peak."""
    pk = peaks()
    alg_bytes = tensors * rows * Dv * 2
    alg_flops = float(flops_per_md) * M * Dk * rows
    gbs = alg_bytes / (ms * 1e-3) / 1e9
    tfs = alg_flops / (ms * 1e-3) / 1e12
    return {"hbm_gbs": gbs, "hbm_frac": gbs / pk["hbm_gbs"], "tflops": tfs, "tensor_frac": tfs / pk["bf16_tflops"],
            "algorithmic_bytes": alg_bytes, "algorithmic_flops": alg_flops, "peak_source": pk["source"]}


def bench_decode(args, rank, world):
    import causal_flare as cf

    c = C3
    B, H, M, Dk, Dv = c["B"], c["H"], c["M"], c["Dk"], c["Dv"]
    sc = Dk ** -0.5
    g = torch.Generator(device="cuda").manual_seed(99 + rank)
    q = torch.randn(H, M, Dk, generator=g, device="cuda").bfloat16()
    # prefix prefill in batch slices (K+V of the full prefix would be 69 GB)
    state = {"m": torch.empty(B, H, M, device="cuda"), "d": torch.empty(B, H, M, device="cuda"),
             "u": torch.empty(B, H, M, Dv, device="cuda")}
    sl = 4
    prefix = args.decode_prefix
    for b0 in range(0, B, sl):
        kk = torch.randn(sl, prefix, H, Dk, generator=g, device="cuda").bfloat16()
        vv = torch.randn(sl, prefix, H, Dv, generator=g, device="cuda").bfloat16()
        _, st = cf.flare_autoregressive_prefill_triton(q, kk, vv, scale=sc)
        for key in state:
            state[key][b0:b0 + sl] = st[key]
        del kk, vv, st
    steps = args.decode_steps
    ks = torch.randn(steps, B, H, Dk, generator=g, device="cuda").bfloat16()
    vs = torch.randn(steps, B, H, Dv, generator=g, device="cuda").bfloat16()
    for i in range(min(8, steps)):
        cf.flare_autoregressive_decode_triton(q, ks[i], vs[i], state, scale=sc)
    barrier(world)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(steps):
        y, state = cf.flare_autoregressive_decode_triton(q, ks[i], vs[i], state, scale=sc)
    t1.record()
    barrier(world)
    ms = max_over_ranks(t0.elapsed_time(t1), world)
    assert torch.isfinite(y.float()).all()
    step_bytes = 2 * B * H * M * Dv * 4 + 4 * B * H * M * 4 + H * M * Dk * 2 + B * H * (Dk + Dv) * 2 + B * H * Dv * 2
    # the same tokens as one fused multi-step call: prefill continuing from the state (the state stays on chip)
    kk, vv = ks.transpose(0, 1).contiguous(), vs.transpose(0, 1).contiguous()
    for _ in range(2):
        cf.flare_autoregressive_prefill_triton(q, kk, vv, state=state, scale=sc)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(3):
        cf.flare_autoregressive_prefill_triton(q, kk, vv, state=state, scale=sc)
    f1.record()
    torch.cuda.synchronize()
    fused_ms = f0.elapsed_time(f1) / 3
    del kk, vv
    pk = peaks()
    gbs = step_bytes * steps / (ms * 1e-3) / 1e9
    return {
        "workload": f"C3 decode B={B} H={H} M={M} D={Dk}, fp32 state after a {prefix}-token bf16 prefix, {steps} steps",
        "tok_per_s": world * B * steps / (ms * 1e-3), "us_per_step": ms * 1e3 / steps, "hbm_gbs": gbs,
        "hbm_frac": gbs / pk["hbm_gbs"], "bytes_per_step": step_bytes, "gpu_launches": steps,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                     "traffic": NCU_TRAFFIC_C3_STEP_BYTES, "algorithmic_bytes": step_bytes, "peak_source": pk["source"],
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one decode_step_kernel launch "
                                       "(profiles/decode_step_c3.md)"},
        "state_bytes": B * H * M * Dv * 4, "l2": "state 268 MB > 126 MB L2",
        "fused_multi_step": {"call": f"one flare_autoregressive_prefill_triton(state=...) over the same {steps} tokens",
                             "ms": fused_ms, "tok_per_s": B * steps / (fused_ms * 1e-3)},
    }


def bench_seqpar(args, rank, world):
    """C5: block-causal long context, tokens sharded across the GPUs (state-only pass, all-gather of the span
    states, fold of the lower ranks, span pass with carry-in).  One GPU: the whole sequence, no exchange."""
    from causal_flare import _ops, parallel

    B, N, H, M, D, bs = 2, args.seqpar_tokens, 32, 256, 128, 64
    span = N // world
    g = torch.Generator(device="cuda").manual_seed(5 + rank)
    q = torch.randn(H, M, D, generator=torch.Generator(device="cuda").manual_seed(5), device="cuda").bfloat16()
    k = torch.randn(B, span, H, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, span, H, D, generator=g, device="cuda").bfloat16()
    sc = D ** -0.5

    def step():
        if world == 1:
            return _ops.forward(q, k, v, scale=sc, block_size=bs)[0]
        return parallel.sequence_parallel_prefill(q, k, v, scale=sc, block_size=bs)[0]

    for _ in range(max(args.warmup, 3)):
        y = step()
    steps = min(args.steps, 20)
    barrier(world)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        y = step()
    t1.record()
    barrier(world)
    ms = max_over_ranks(t0.elapsed_time(t1), world) / steps
    assert torch.isfinite(y.float()).all() and _ops.device_status() == 0
    fwd_bwd_ms = None
    if args.seqpar_backward:
        dy = torch.randn(B, span, H, D, generator=g, device="cuda").bfloat16()

        def train_step():
            if world == 1:
                _ops.forward(q, k, v, scale=sc, block_size=bs)
                return _ops.backward(q, k, v, dy, scale=sc, block_size=bs)[0]
            parallel.sequence_parallel_prefill(q, k, v, scale=sc, block_size=bs)
            if H % world == 0:  # re-sharded by heads: whole sequences on the tensor-core backward
                return parallel.sequence_parallel_backward_by_heads(q, k, v, dy, scale=sc, block_size=bs)[0]
            _, _, prefix = parallel.sequence_parallel_prefill(q, k, v, scale=sc, block_size=bs, return_prefix=True)
            return parallel.sequence_parallel_backward(q, k, v, dy, scale=sc, prefix_state=prefix, block_size=bs)[0]

        train_step()
        barrier(world)
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(2):
            dq = train_step()
        b1.record()
        barrier(world)
        fwd_bwd_ms = max_over_ranks(b0.elapsed_time(b1), world) / 2
        assert torch.isfinite(dq).all()
    return {"metric": "block-causal long-context prefill throughput", "fwd_bwd_ms": fwd_bwd_ms, "value": B * N / (ms * 1e-3) / 1e6, "unit": "Mtok/s",
            "n_gpus": world, "steps": steps, "ms_per_step": ms, "scaling": "strong", "higher_is_better": True,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"C5 semi-AR B={B} N={N} H={H} M={M} D={D} block={bs}, {span} tokens per GPU",
                       "parallelism": f"sequence parallel over {world} GPU(s), one all-gather of span states per step; "
                                      "backward: all-to-all to a head sharding and back"}}


def bench_strong(args, rank, world):
    """The FIXED C2 workload sharded by heads over the ranks (strong scaling; lanes are independent, so no collective):
    rank r runs heads [r H / world, (r + 1) H / world).  Rank 0 also times the whole workload alone for the ratio."""
    import causal_flare as cf

    cfg = C2
    q, k, v = device_inputs(cfg, seed=4321)  # the same tensors on every rank
    hp = cfg["H"] // world
    h0 = rank * hp
    qs, ks, vs = q[h0:h0 + hp], k[:, :, h0:h0 + hp], v[:, :, h0:h0 + hp]  # strided views: no copies
    steps = min(args.steps, 20)

    def timed(fn):
        for _ in range(3):
            fn()
        barrier(world)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            fn()
        t1.record()
        barrier(world)
        return t0.elapsed_time(t1) / steps

    full_ms = timed(lambda: cf.flare_autoregressive_triton(q, k, v))  # every rank runs it; rank 0's number is reported
    split_ms = max_over_ranks(timed(lambda: cf.flare_autoregressive_triton(qs, ks, vs)), world)
    tokens = cfg["B"] * cfg["N"]
    return {"workload": f"fixed C2 (B={cfg['B']} N={cfg['N']} H={cfg['H']}), {hp} heads = {hp * cfg['B']} lanes per GPU",
            "scaling": "strong", "n_gpus": world, "ms_one_gpu": full_ms, "ms_split": split_ms,
            "value": tokens / (split_ms * 1e-3) / 1e6, "unit": "Mtok/s", "speedup": full_ms / split_ms}


def seqpar_check(rank, world):
    """Reduced block-causal shape: this rank's span of the sequence-parallel run against a local run of the whole
    sequence (every rank generates the same inputs).  Returns the max-abs difference of y."""
    from causal_flare import _ops, parallel

    B, H, M, D, bs = 1, 2, 256, 128, 64
    span = 512
    N = span * world
    g = torch.Generator(device="cuda").manual_seed(77)
    q = torch.randn(H, M, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    sc = D ** -0.5
    whole = _ops.forward(q, k, v, scale=sc, block_size=bs)[0]
    lo = rank * span
    mine = parallel.sequence_parallel_prefill(q, k[:, lo:lo + span], v[:, lo:lo + span], scale=sc, block_size=bs)[0]
    return max_over_ranks(float((mine.float() - whole[:, lo:lo + span].float()).abs().max()), world)


def bench_other_shapes(which="all"):
    """Short device-timed runs of the other benchmark shapes (not the headline metric): training-shape forward and
    forward+backward, and the long block-causal shape on one GPU."""
    import causal_flare as cf

    def timed(fn, warm=2, n=5):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / n

    out = {}
    g = torch.Generator(device="cuda").manual_seed(7)
    B, N, H, M, D = 4, 4096, 16, 64, 128
    q = torch.randn(H, M, D, generator=g, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16().requires_grad_()
    dy = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    with torch.no_grad():
        out["C4_forward_ms"] = timed(lambda: cf.flare_autoregressive_triton(q, k, v))

    def train_step(fn):
        q.grad = k.grad = v.grad = None
        fn(q, k, v).backward(dy)

    out["C4_fwd_bwd_softmax_ms"] = timed(lambda: train_step(cf.flare_autoregressive_triton), n=3)
    out["C4"] = f"B={B} N={N} H={H} M={M} D={D} bf16"
    # forward + backward: 21 M D flop per (token, head); reads Q, K, V, dY and writes Y, dK, dV = 6 tensors
    out["C4_fwd_bwd_softmax_roofline"] = _shape_roofline(B * N * H, M, D, D, out["C4_fwd_bwd_softmax_ms"], flops_per_md=21, tensors=6)
    if which == "train":
        return out
    from causal_flare.autoregressive import flare_autoregressive_stablemax_triton

    out["C4_fwd_bwd_stablemax_ms"] = timed(lambda: train_step(flare_autoregressive_stablemax_triton), n=3)
    out["C4_fwd_bwd_stablemax_roofline"] = _shape_roofline(B * N * H, M, D, D, out["C4_fwd_bwd_stablemax_ms"], flops_per_md=21, tensors=6)
    out["C4"] = f"B={B} N={N} H={H} M={M} D={D} bf16"
    del q, k, v, dy
    B, N, H, M, D, bs = 2, 65536, 32, 256, 128, 64
    q = torch.randn(H, M, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    with torch.no_grad():
        out["C5_one_gpu_semi_ar_forward_ms"] = timed(
            lambda: cf.flare_semi_autoregressive_trition(q, k, v, block_size=bs, chunk_size=64), n=3)
    out["C5"] = f"B={B} N={N} H={H} M={M} D={D} block={bs} bf16, whole sequence on one GPU"
    out["C5_roofline"] = _shape_roofline(B * N * H, M, D, D, out["C5_one_gpu_semi_ar_forward_ms"], flops_per_md=6, tensors=3)
    del q, k, v
    # the headline shape with fp16 inputs: bf16 copies of q, k, v in the workspace, tensor-core kernels, y back as fp16
    c = C2
    q = torch.randn(c["H"], c["M"], c["Dk"], generator=g, device="cuda").half()
    k = torch.randn(c["B"], c["N"], c["H"], c["Dk"], generator=g, device="cuda").half()
    v = torch.randn(c["B"], c["N"], c["H"], c["Dv"], generator=g, device="cuda").half()
    with torch.no_grad():
        out["C2_fp16_forward_ms"] = timed(lambda: cf.flare_autoregressive_triton(q, k, v))
    del q, k, v
    B, N, H, M, D = 4, 4096, 16, 64, 128  # the training shape with fp16 tensors
    q = torch.randn(H, M, D, generator=g, device="cuda").half().requires_grad_()
    k = torch.randn(B, N, H, D, generator=g, device="cuda").half().requires_grad_()
    v = torch.randn(B, N, H, D, generator=g, device="cuda").half().requires_grad_()
    dy = torch.randn(B, N, H, D, generator=g, device="cuda").half()
    out["C4_fp16_fwd_bwd_softmax_ms"] = timed(lambda: train_step(cf.flare_autoregressive_triton), n=3)
    return out


def cpu_reference_sample(threads=None):
    """The reference algorithm on the host cores over the whole C2 workload, fp32: the reference's three-phase chunked
    formulation (``flare_causal_chunked``) and its token recurrence, both as restated by the oracle; the faster of the
    two is the baseline.  The thread count is set explicitly (a launcher may have pinned OMP_NUM_THREADS to 1)."""
    from oracle import flare_oracle as orc

    torch.set_num_threads(threads or os.cpu_count() or 1)
    cfg = C2
    Bs, Ns = cfg["B"], cfg["N"]  # the whole C2 workload: several seconds per formulation on 16-32 host cores
    q, k, v = orc.make_inputs(Bs, Ns, cfg["H"], cfg["M"], cfg["Dk"], cfg["Dv"], seed0=0, dtype=torch.bfloat16)
    orc.ar_forward(q, k[:, :16], v[:, :16], dtype=torch.float32)
    times = {}
    t = time.perf_counter()
    orc.ar_forward_chunked(q, k, v, chunk_size=64, dtype=torch.float32)
    times["chunked (three phases, chunk 64)"] = time.perf_counter() - t
    t = time.perf_counter()
    orc.ar_forward(q, k, v, dtype=torch.float32)
    times["token recurrence"] = time.perf_counter() - t
    best = min(times, key=times.get)
    dt = times[best]
    return dict(value=Bs * Ns / dt / 1e6, unit="Mtok/s", cores=torch.get_num_threads(), kind="port", seconds=dt,
                sample=f"{Bs} of {cfg['B']} batch rows, all {Ns} tokens and {cfg['H']} heads, fp32; oracle port of the "
                       f"reference's PyTorch path, faster of two formulations: {best} "
                       f"({', '.join(f'{k_}: {v_:.1f} s' for k_, v_ in times.items())})")


def gpu_reference_leg():
    """The reference's own GPU (Triton) kernels on this box, when its package can be imported from the directory named
    by FLARE_REFERENCE_PATH: C2 forward under the same events.  Baseline only; nothing in the product imports it.  The
    reference checkout does not travel to the benchmark box and its sources are not part of this repository, so the
    usual answer is `unavailable`."""
    path = os.environ.get("FLARE_REFERENCE_PATH", "")
    if not path or not os.path.isdir(path):
        return {"unavailable": "the reference package is not present on this box (set FLARE_REFERENCE_PATH to a checkout)"}
    import subprocess as sp

    code = (
        "import sys, json, torch; sys.path.insert(0, sys.argv[1]); import causal_flare as ref;"
        "g = torch.Generator(device='cuda').manual_seed(1234);"
        "q = torch.randn(16, 128, 64, generator=g, device='cuda').bfloat16();"
        "k = torch.randn(8, 8192, 16, 64, generator=g, device='cuda').bfloat16();"
        "v = torch.randn(8, 8192, 16, 64, generator=g, device='cuda').bfloat16();"
        "f = lambda: ref.flare_autoregressive_triton(q, k, v);"
        "[f() for _ in range(3)]; torch.cuda.synchronize();"
        "a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True);"
        "a.record(); [f() for _ in range(10)]; b.record(); torch.cuda.synchronize();"
        "print(json.dumps({'C2_forward_ms': a.elapsed_time(b) / 10}))"
    )
    try:  # a separate interpreter: the reference package has the same import name as this one
        out = sp.run([sys.executable, "-c", code, path], capture_output=True, text=True, timeout=600)
        if out.returncode != 0:
            return {"unavailable": (out.stderr.strip().splitlines() or ["failed"])[-1][:300]}
        return json.loads(out.stdout.strip().splitlines()[-1])
    except Exception as exc:  # noqa: BLE001
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


def config_block(world):
    c = C2
    return {"workload": f"C2 chunked causal prefill forward B={c['B']} N={c['N']} H={c['H']} M={c['M']} D={c['Dk']} "
                        "bf16 in / fp32 accumulate, one full workload per GPU", "global_batch": c["B"] * world,
            "seq_len": c["N"], "parallelism": f"batch x head lanes, {world} GPU(s), no collective",
            "l2": "K+V+Y = 403 MB per step > 126 MB L2 (no flush needed)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-decode", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--decode-prefix", type=int, default=C3["prefix"])
    ap.add_argument("--decode-steps", type=int, default=C3["steps"])
    ap.add_argument("--only", default="all", choices=["all", "prefill", "decode", "seqpar", "train"],
                    help="profiling aid: run one section only (the JSON line then lacks the other)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--seqpar-backward", action="store_true", help="with --only seqpar: also time forward+backward")
    ap.add_argument("--seqpar-tokens", type=int, default=65536,
                    help="with --only seqpar: sequence length (the C5 shape has 65536; shorter for profiler captures)")
    ap.add_argument("--skip-other", action="store_true", help="skip the short runs of the other benchmark shapes")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        steps = max(1, min(args.steps, 3))
        for _ in range(min(args.warmup, 1)):
            cpu_reference_sample()
        runs = [cpu_reference_sample() for _ in range(steps)]
        best = max(runs, key=lambda r: r["value"])
        val = sum(r["value"] for r in runs) / len(runs)
        line = {
            "impl": "reference", "metric": "prefill throughput", "value": val, "unit": "Mtok/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * sum(r["seconds"] for r in runs) / len(runs),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_block(1),
            "cpu_baseline": dict(value=val, unit="Mtok/s", cores=best["cores"], kind="port", sample=best["sample"]),
            "e2e": {"value": val, "unit": "Mtok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
        print(json.dumps(line))
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    rank, world, _ = dist_setup(args.gpus)
    if args.only == "train":
        if rank == 0:
            print(json.dumps({"metric": "training step time", "unit": "ms", "other_shapes": bench_other_shapes("train")}))
        return
    if args.only == "seqpar":
        res = bench_seqpar(args, rank, world)
        if rank == 0:
            print(json.dumps(res))
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()
        return
    if args.only == "decode":
        dec = bench_decode(args, rank, world)
        if rank == 0:
            print(json.dumps({"metric": "decode throughput", "value": dec["tok_per_s"], "unit": "tok/s", "decode": dec}))
        return
    pre = bench_prefill(args, rank, world)
    dec = None if (args.skip_decode or args.only == "prefill") else bench_decode(args, rank, world)
    other = None
    if world == 1 and args.only == "all" and not args.skip_other:
        other = bench_other_shapes()
    strong = seqpar = None
    if world > 1 and args.only == "all" and not args.skip_other:
        # the two multi-GPU partitions of the path: fixed workload split by heads (no collective), and the long
        # block-causal sequence split by tokens (one all-gather of span states in the forward; the backward re-shards
        # K, V, dY by heads with one all-to-all, runs whole sequences on the tensor-core backward and brings dK, dV
        # back with a second all-to-all)
        strong = bench_strong(args, rank, world)
        args.seqpar_backward = True
        sp_args = argparse.Namespace(**vars(args))
        sp_args.steps = min(args.steps, 10)
        seqpar = bench_seqpar(sp_args, rank, world)
        seqpar["check_max_abs_vs_one_gpu"] = seqpar_check(rank, world)
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        cpu = cpu_reference_sample()
        cpu.pop("seconds", None)
    if rank == 0:
        line = {
            "metric": "prefill throughput", "value": pre["value"], "unit": "Mtok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": pre["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_block(world),
            "roofline": pre["roofline"], "cpu_baseline": cpu, "e2e": pre["e2e"], "gpu_launches": pre["gpu_launches"],
            "clocks": pre["clocks"], "decode": dec, "other_shapes": other, "strong": strong, "seqpar": seqpar,
            "gpu_reference": gpu_reference_leg() if (world == 1 and args.only == "all" and not args.skip_other) else None,
        }
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
