"""Thin torch-side launch helpers over the C ABI: allocate outputs, fill argument structs, call."""

from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib


def default_path() -> int:
    """Kernel path selector: FLARE_B200_PATH = auto (default) | exact | tensor."""
    return {"auto": _lib.PATH_AUTO, "exact": _lib.PATH_EXACT, "tensor": _lib.PATH_TENSOR}[
        os.environ.get("FLARE_B200_PATH", "auto").strip().lower()]


def device_status(reset: bool = True) -> int:
    """Health word of the tensor-core kernels (synchronises the device).  0: nothing to report.  Bit 0: a bounded wait
    gave up, results are invalid.  Bit 1: some call's inputs were outside the numeric domain of the tensor kernels
    (score spreads of several hundred nats); calls on the default path (auto) were completed by the exact kernels on
    their own and are correct, calls that forced ``FLARE_B200_PATH=tensor`` are not."""
    return _lib.load().flare_device_status(1 if reset else 0)


def _prep(t, dtype):
    if t is None:
        return None
    if t.dtype != dtype:
        t = t.to(dtype)
    return _lib.kernel_ready(t)


def forward(Q, K, V, *, scale, Q_dec=None, K_dec=None, variant=_lib.SOFTMAX, power=2.0, block_size=1, mask=None,
            state_in=None, want_state=False, want_lse=False, out_dtype=None, out_bhnd=False, path=None,
            want_y=True, keep_for_backward=None):
    """Run flare_forward.  Q_dec / K_dec are None for the shared-weight default.

    ``keep_for_backward``: a dict (or None).  When the call runs on the tensor-core kernels, the forward leaves in it
    what ``backward(..., saved=...)`` needs to skip its own replay of the forward ("y", "lse_dec", "keep"); the dict
    stays empty for every other problem.

    Returns (Y, state_out | None, lse_dec | None, lse_enc | None)."""
    _lib.load()
    if path is None:
        path = default_path()
    dev = K.device
    dt = K.dtype
    _lib.dtype_code(dt)
    B, N, H, Dk = K.shape
    M, Dv = Q.shape[1], V.shape[-1]
    q, k, v = _prep(Q, dt), _prep(K, dt), _prep(V, dt)
    qd, kd = _prep(Q_dec, dt), _prep(K_dec, dt)
    y = None
    if want_y:
        if out_bhnd:
            y_store = torch.empty((B, H, N, Dv), device=dev, dtype=dt)
            y = y_store.permute(0, 2, 1, 3)
        else:
            y_store = torch.empty((B, N, H, Dv), device=dev, dtype=dt)
            y = y_store
    st_out = None
    if want_state:
        st_out = {
            "m": torch.empty((B, H, M), device=dev, dtype=torch.float32),
            "d": torch.empty((B, H, M), device=dev, dtype=torch.float32),
            "u": torch.empty((B, H, M, Dv), device=dev, dtype=torch.float32),
        }
    lse_dec = lse_enc = None
    if want_lse:
        lse_dec = torch.empty((B, H, N), device=dev, dtype=torch.float32)
        if block_size > 1:
            lse_enc = torch.empty((B, H, N // block_size, M), device=dev, dtype=torch.float32)
    if mask is not None:
        if block_size > 1:
            raise ValueError("attention masks are not supported together with block_size > 1 (block-causal read-out)")
        mask = mask.to(device=dev, dtype=torch.int32).contiguous()
    if mask is not None and B > 0 and N > 0 and _masked_on_tensor_path(q, k, v, qd, kd, y, st_out, scale, variant, power,
                                                                      block_size, path, want_lse):
        _forward_compacted(q, k, v, y, mask, scale=scale, variant=variant, power=power, state_in=state_in,
                           st_out=st_out, path=path)
    elif B > 0 and N > 0 or want_state:
        args = _lib.make_fwd_args(q, k, v, qd, kd, y, scale=scale, variant=variant, power=power,
                                  block_size=block_size, mask=mask, state_in=state_in, state_out=st_out,
                                  lse_dec=lse_dec, lse_enc=lse_enc, path=path)
        keep = None
        if keep_for_backward is not None and y is not None and out_dtype in (None, dt):
            need = _lib.load().flare_forward_keep_bytes(C.byref(args))
            if need > 0:
                if lse_dec is None:
                    lse_dec = torch.empty((B, H, N), device=dev, dtype=torch.float32)
                    args.lse_dec = lse_dec.data_ptr()
                keep = torch.empty(need, dtype=torch.uint8, device=dev)
                args.keep, args.keep_bytes = keep.data_ptr(), need
        _lib.run_forward(args, dev)
        if keep is not None:
            keep_for_backward.update(y=y, lse_dec=lse_dec, keep=keep)
            if not want_lse:
                lse_dec = None
    out = None
    if want_y:
        out = y_store if out_dtype in (None, dt) else y_store.to(out_dtype)
    return out, st_out, lse_dec, lse_enc


def _masked_on_tensor_path(q, k, v, qd, kd, y, st_out, scale, variant, power, block_size, path, want_lse) -> bool:
    """True when the same call without the mask would run on the tensor-core kernels (they take per-row lengths, not
    arbitrary masks, so a masked call is served by compacting the valid tokens to the front of every row)."""
    if path == _lib.PATH_EXACT or want_lse or qd is not None or kd is not None or (y is None and st_out is None):
        return False
    probe = _lib.make_fwd_args(q, k, v, None, None, y, scale=scale, variant=variant, power=power, block_size=block_size,
                               state_out=st_out, path=path)
    return _lib.load().flare_forward_uses_tensor_path(C.byref(probe)) == 1


def _forward_compacted(q, k, v, y, mask, *, scale, variant, power, state_in, st_out, path):
    """Masked forward on the tensor path: gather the valid tokens of every batch row to the front (stable order), run
    the kernel with per-row lengths, scatter the outputs back; masked positions get y = 0 and leave the state as is."""
    B, N, H, Dk = k.shape
    Dv = v.shape[-1]
    valid = mask != 0
    order = torch.argsort((~valid).to(torch.uint8), dim=1, stable=True)  # valid positions first, original order kept
    lens = valid.sum(dim=1).to(torch.int32)
    idx = order[:, :, None, None]
    kc = torch.gather(k, 1, idx.expand(B, N, H, Dk))
    vc = torch.gather(v, 1, idx.expand(B, N, H, Dv))
    yc = torch.empty((B, N, H, Dv), device=k.device, dtype=k.dtype) if y is not None else None
    args = _lib.make_fwd_args(q, kc, vc, None, None, yc, scale=scale, variant=variant, power=power, state_in=state_in,
                              state_out=st_out, path=path, lengths=lens)
    _lib.run_forward(args, k.device)
    if y is not None:
        pad = torch.arange(N, device=k.device)[None, :] >= lens[:, None]
        yc.masked_fill_(pad[:, :, None, None], 0)  # rows beyond a row's length were not written by the kernel
        y.scatter_(1, idx.expand(B, N, H, Dv), yc)


def backward(Q, K, V, dY, *, scale, Q_dec=None, K_dec=None, variant=_lib.SOFTMAX, power=2.0, block_size=1,
             dy_bhnd=False, path=None, saved=None):
    """Run flare_backward.  ``saved``: what a forward with ``keep_for_backward`` left behind (or None / empty: the
    backward replays the forward itself).  Returns fp32 dQ, input-dtype dK, dV, and dQ_dec / dK_dec (or None)."""
    _lib.load()
    if path is None:
        path = default_path()
    dev = K.device
    dt = K.dtype
    B, N, H, Dk = K.shape
    M, Dv = Q.shape[1], V.shape[-1]
    q, k, v = _prep(Q, dt), _prep(K, dt), _prep(V, dt)
    qd, kd = _prep(Q_dec, dt), _prep(K_dec, dt)
    dy = dY.permute(0, 2, 1, 3) if dy_bhnd else dY
    dy = _prep(dy, dt)
    # the kernels write every element of every gradient; only an empty problem needs explicit zeros
    alloc = torch.empty if (B > 0 and N > 0) else torch.zeros
    dq = alloc((H, M, Dk), device=dev, dtype=torch.float32)
    dk = alloc((B, N, H, Dk), device=dev, dtype=dt)
    dv = alloc((B, N, H, Dv), device=dev, dtype=dt)
    dqd = alloc((B, N, H, Dk), device=dev, dtype=dt) if qd is not None else None
    dkd = alloc((H, M, Dk), device=dev, dtype=torch.float32) if kd is not None else None
    if B > 0 and N > 0:
        a = _lib.BwdArgs()
        a.fwd = _lib.make_fwd_args(q, k, v, qd, kd, None, scale=scale, variant=variant, power=power,
                                   block_size=block_size, path=path)
        a.dy = dy.data_ptr()
        a.dy_stride_b, a.dy_stride_n, a.dy_stride_h = dy.stride(0), dy.stride(1), dy.stride(2)
        a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        a.dq_dec, a.dk_dec = _lib.ptr(dqd), _lib.ptr(dkd)
        if saved:
            ys = saved["y"]
            a.y = ys.data_ptr()
            a.y_stride_b, a.y_stride_n, a.y_stride_h = ys.stride(0), ys.stride(1), ys.stride(2)
            a.lse_dec = saved["lse_dec"].data_ptr()
            a.fwd.keep, a.fwd.keep_bytes = saved["keep"].data_ptr(), saved["keep"].numel()
        _lib.run_backward(a, dev)
    return dq, dk, dv, dqd, dkd


def backward_span_begin(Q, K, V, dY, *, scale, state_in, variant=_lib.SOFTMAX, power=2.0, block_size=1):
    """First phase of the backward of a span of a longer sequence (shared decode weights): replays the span from
    ``state_in`` (forward state of the tokens before it; None for the first span) and returns a context whose
    ``summary`` = {"b0", "c0", "gam", "rho_first"} (fp32 [B,H,M(,Dv)]) describes the span to the spans on its left."""
    lib = _lib.load()
    dev, dt = K.device, K.dtype
    B, N, H, Dk = K.shape
    M, Dv = Q.shape[1], V.shape[-1]
    keep = dict(q=_prep(Q, dt), k=_prep(K, dt), v=_prep(V, dt), dy=_prep(dY, dt))
    keep["dq"] = torch.zeros((H, M, Dk), device=dev, dtype=torch.float32)
    keep["dk"] = torch.zeros((B, N, H, Dk), device=dev, dtype=dt)
    keep["dv"] = torch.zeros((B, N, H, Dv), device=dev, dtype=dt)
    f32 = dict(device=dev, dtype=torch.float32)  # explicit: the kernels write fp32 whatever torch's default dtype is
    summary = {"b0": torch.empty((B, H, M, Dv), **f32), "c0": torch.empty((B, H, M), **f32),
               "gam": torch.empty((B, H, M), **f32), "rho_first": torch.empty((B, H, M), **f32)}
    keep["st"] = None if state_in is None else {key: state_in[key].float().contiguous() for key in ("m", "d", "u")}
    a = _lib.BwdArgs()
    a.fwd = _lib.make_fwd_args(keep["q"], keep["k"], keep["v"], None, None, None, scale=scale, variant=variant,
                               power=power, block_size=block_size, state_in=keep["st"])
    dy = keep["dy"]
    a.dy = dy.data_ptr()
    a.dy_stride_b, a.dy_stride_n, a.dy_stride_h = dy.stride(0), dy.stride(1), dy.stride(2)
    a.dq, a.dk, a.dv = keep["dq"].data_ptr(), keep["dk"].data_ptr(), keep["dv"].data_ptr()
    a.span_b0, a.span_c0 = summary["b0"].data_ptr(), summary["c0"].data_ptr()
    a.span_gam, a.span_rho_first = summary["gam"].data_ptr(), summary["rho_first"].data_ptr()
    a.phase = 1
    need = lib.flare_backward_workspace_bytes(C.byref(a))
    keep["ws"] = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)  # holds the planes across both phases
    a.fwd.workspace, a.fwd.workspace_bytes = keep["ws"].data_ptr(), need
    _lib.check(lib.flare_backward(C.byref(a), _lib.stream_handle(dev)), "flare_backward (span, phase 1)")
    return {"args": a, "keep": keep, "summary": summary, "device": dev}


def backward_span_finish(ctx, carry):
    """Second phase: ``carry`` = {"b", "c", "rho"} entering from the tokens after the span (None for the last span).
    Returns (dQ fp32 - this span's part, to be summed over the spans -, dK, dV in the input dtype)."""
    lib = _lib.load()
    a, keep = ctx["args"], ctx["keep"]
    if carry is not None:
        keep["carry"] = [carry[key].float().contiguous() for key in ("b", "c", "rho")]
        a.carry_b, a.carry_c, a.carry_rho = (t.data_ptr() for t in keep["carry"])
    a.phase = 2
    _lib.check(lib.flare_backward(C.byref(a), _lib.stream_handle(ctx["device"])), "flare_backward (span, phase 2)")
    return keep["dq"], keep["dk"], keep["dv"]


def decode_step(Q, k, v, state, *, scale, q_dec=None, K_dec=None, mask=None):
    """One token: k, v [B,H,D]; state updated in place.  Returns y [B,H,Dv] in k's dtype."""
    lib = _lib.load()
    dev = k.device
    dt = k.dtype
    B, H, Dk = k.shape
    M, Dv = Q.shape[1], v.shape[-1]
    q = _prep(Q, dt)
    kd = _prep(K_dec, dt)
    k = k if k.stride(-1) == 1 else k.contiguous()
    v = v.to(dt) if v.dtype != dt else v
    v = v if v.stride(-1) == 1 else v.contiguous()
    if q_dec is not None:
        q_dec = q_dec.to(dt) if q_dec.dtype != dt else q_dec
        q_dec = q_dec if q_dec.stride(-1) == 1 else q_dec.contiguous()
    y = torch.empty((B, H, Dv), device=dev, dtype=dt)
    a = _lib.DecodeArgs()
    a.q, a.k, a.v, a.q_dec, a.k_dec, a.y = q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr(q_dec), _lib.ptr(kd), y.data_ptr()
    if mask is not None:
        mask = mask.to(device=dev, dtype=torch.int32).contiguous()
    a.mask = _lib.ptr(mask)
    a.state = _lib.state_struct(state)
    a.B, a.H, a.M, a.Dk, a.Dv = B, H, M, Dk, Dv
    a.q_stride_h, a.q_stride_m = q.stride(0), q.stride(1)
    a.k_stride_b, a.k_stride_h = k.stride(0), k.stride(1)
    a.v_stride_b, a.v_stride_h = v.stride(0), v.stride(1)
    if q_dec is not None:
        a.qd_stride_b, a.qd_stride_h = q_dec.stride(0), q_dec.stride(1)
    if kd is not None:
        a.kd_stride_h, a.kd_stride_m = kd.stride(0), kd.stride(1)
    a.scale = float(scale)
    a.dtype = _lib.dtype_code(dt)
    rc = lib.flare_decode_step(C.byref(a), _lib.stream_handle(dev))
    if rc == 2:
        # shape outside the streaming kernel (value width not a power of two): general walk with N = 1
        out, new_state, _, _ = forward(
            Q, k[:, None], v[:, None], scale=scale, Q_dec=None if q_dec is None else q_dec[:, None], K_dec=K_dec,
            mask=None if mask is None else mask.view(B, 1), state_in=state, want_state=True)
        for key in ("m", "d", "u"):
            state[key].copy_(new_state[key])
        return out[:, 0]
    _lib.check(rc, "flare_decode_step")
    return y


def merge_stacked(a, stacked, count):
    """Fold the first ``count`` states of ``stacked`` ({"m": [n, B, H, M], "d": ..., "u": [n, B, H, M, Dv]}, fp32,
    contiguous) in order into ``a``; returns a new state dict."""
    lib = _lib.load()
    dev = a["u"].device
    B, H, M, Dv = a["u"].shape
    a32 = {k: a[k].float().contiguous() for k in ("m", "d", "u")}
    for k in ("m", "d", "u"):
        if stacked[k].dtype != torch.float32 or not stacked[k].is_contiguous():
            raise ValueError("stacked states must be contiguous fp32 tensors")
    out = {k: torch.empty_like(a32[k]) for k in ("m", "d", "u")}
    sa = _lib.state_struct(a32)
    sb = _lib.State(stacked["m"].data_ptr(), stacked["d"].data_ptr(), stacked["u"].data_ptr())
    so = _lib.state_struct(out)
    rc = lib.flare_state_merge(C.byref(sa), C.byref(sb), C.byref(so), B * H, M, Dv, int(count), _lib.stream_handle(dev))
    _lib.check(rc, "flare_state_merge")
    return out


def merge_states(a, b_list):
    """Fold the states in ``b_list`` (in order) into ``a``; returns a new state dict."""
    lib = _lib.load()
    dev = a["u"].device
    B, H, M, Dv = a["u"].shape
    a32 = {k: a[k].float().contiguous() for k in ("m", "d", "u")}
    bm = torch.stack([b["m"].float() for b in b_list]).contiguous()
    bd = torch.stack([b["d"].float() for b in b_list]).contiguous()
    bu = torch.stack([b["u"].float() for b in b_list]).contiguous()
    out = {k: torch.empty_like(a32[k]) for k in ("m", "d", "u")}
    sa = _lib.state_struct(a32)
    sb = _lib.State(bm.data_ptr(), bd.data_ptr(), bu.data_ptr())
    so = _lib.state_struct(out)
    rc = lib.flare_state_merge(C.byref(sa), C.byref(sb), C.byref(so), B * H, M, Dv, len(b_list), _lib.stream_handle(dev))
    _lib.check(rc, "flare_state_merge")
    return out
