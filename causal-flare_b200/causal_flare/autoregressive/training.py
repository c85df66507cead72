"""Autoregressive (token-causal) softmax FLARE: training forward + recompute-based backward.

Interface of the operator this replaces: ``AutoRegressiveFLARE`` / ``flare_autoregressive_triton``
(reference: causal_flare/autoregressive/training.py:731-911, :4921-4937).
"""

from __future__ import annotations

import torch
from torch import autograd

from .. import _lib, _ops
from .._common import _normalize_input_precision, _refresh_profile_totals, _resolve_attn_scale, _timed
from .._reference_utils import resolve_flare_causal_decode_inputs


class AutoRegressiveFLARE(autograd.Function):
    """y_t = sum_m softmax_m(a_t)[m] * z_t[m],  z_t[m] = softmax-weighted mean of v_{<=t} under scores k.q_m."""

    @staticmethod
    def forward(ctx, Q, K, V, scale=None, chunk_size=None, input_precision=None, profile=False, Q_dec=None, K_dec=None):
        assert Q.dim() == 3 and K.dim() == 4 and V.dim() == 4, (
            "Q, K, V must be 3D and 4D tensors respectively "
            f"got Q.dim()={Q.dim()}, K.dim()={K.dim()}, V.dim()={V.dim()}"
        )
        assert K.shape[:3] == V.shape[:3], (
            f"Expected K/V to agree on [B, N, H]. Got K.shape={K.shape} and V.shape={V.shape}"
        )
        assert Q.size(0) == K.size(2) and Q.size(2) == K.size(3), (
            f"Expected Q [H, M, D_k] and K [B, N, H, D_k]. Got Q.shape={Q.shape} and K.shape={K.shape}"
        )
        H, M, D_score = Q.shape
        D_value = V.size(3)
        Q_dec, K_dec, separate_Q_dec, separate_K_dec, shared = resolve_flare_causal_decode_inputs(Q, K, Q_dec, K_dec)
        if shared:
            # decode tensors that ARE the encode tensors (same objects) take the shared-weight path: one score
            # matrix, decode-side gradients folded into dQ / dK, None returned for the aliased arguments
            separate_Q_dec = separate_K_dec = False
        scale = _resolve_attn_scale(scale, D_score)
        _normalize_input_precision(input_precision)
        chunk_size = 64 if chunk_size is None else int(chunk_size)
        assert M % 16 == 0, f"M must be divisible by 16. Got M={M}."
        assert D_score % 16 == 0, f"score_head_dim must be divisible by 16. Got score_head_dim={D_score}."
        assert D_value % 16 == 0, f"value_head_dim must be divisible by 16. Got value_head_dim={D_value}."
        assert chunk_size % 16 == 0, f"CHUNK_SIZE must be divisible by 16. Got CHUNK_SIZE={chunk_size}."
        if not K.is_cuda:
            raise RuntimeError("flare_autoregressive requires CUDA tensors.")

        profile_data = {"forward": {}, "backward": {}} if profile else None
        qd = Q_dec if separate_Q_dec else None
        kd = K_dec if separate_K_dec else None
        # with gradients wanted, the tensor-core forward keeps its per-chunk states for the backward
        kept = {} if any(ctx.needs_input_grad[:3]) else None
        Y, _, _, _ = _timed(
            K.device, profile_data["forward"] if profile else None, "flare_forward",
            lambda: _ops.forward(Q, K, V, scale=scale, Q_dec=qd, K_dec=kd, keep_for_backward=kept),
        )
        saved = [Q, K, V]
        if separate_Q_dec:
            saved.append(Q_dec)
        if separate_K_dec:
            saved.append(K_dec)
        ctx.has_kept = bool(kept)
        if kept:
            saved += [kept["y"], kept["lse_dec"], kept["keep"]]  # through save_for_backward: y is this node's output
        ctx.save_for_backward(*saved)
        ctx.scale = scale
        ctx.separate_Q_dec = separate_Q_dec
        ctx.separate_K_dec = separate_K_dec
        ctx.profile_timings = profile_data
        if profile:
            _refresh_profile_totals(profile_data)
            return Y, profile_data
        return Y

    @staticmethod
    def backward(ctx, dO, dTimings=None):
        if dO is None:
            return (None,) * 9
        saved = list(ctx.saved_tensors)
        Q, K, V = saved[:3]
        rest = saved[3:]
        Q_dec = rest.pop(0) if ctx.separate_Q_dec else None
        K_dec = rest.pop(0) if ctx.separate_K_dec else None
        kept = dict(y=rest[0], lse_dec=rest[1], keep=rest[2]) if ctx.has_kept else None
        prof = ctx.profile_timings
        dq, dk, dv, dqd, dkd = _timed(
            K.device, prof["backward"] if prof is not None else None, "flare_backward",
            lambda: _ops.backward(Q, K, V, dO, scale=ctx.scale, Q_dec=Q_dec, K_dec=K_dec, saved=kept),
        )
        if prof is not None:
            _refresh_profile_totals(prof)
        return (
            dq.to(Q.dtype), dk.to(K.dtype), dv.to(V.dtype), None, None, None, None,
            None if dqd is None else dqd.to(Q_dec.dtype),
            None if dkd is None else dkd.to(K_dec.dtype),
        )


def flare_autoregressive_triton(Q, K, V, scale=None, chunk_size=None, input_precision=None, profile=False,
                                Q_dec=None, K_dec=None):
    """Causal FLARE forward (differentiable).  Q [H,M,Dk]; K [B,N,H,Dk]; V [B,N,H,Dv] -> Y [B,N,H,Dv] in K.dtype.

    ``chunk_size`` and ``input_precision`` are validated and otherwise unused: tiling is fixed by the
    kernels.  With ``profile=True`` returns ``(Y, timings)``; the backward section of ``timings`` is
    filled in place when the output is differentiated."""
    return AutoRegressiveFLARE.apply(Q, K, V, scale, chunk_size, input_precision, profile, Q_dec, K_dec)


ChunkedFLARE = AutoRegressiveFLARE
flare_chunk_triton = flare_autoregressive_triton
