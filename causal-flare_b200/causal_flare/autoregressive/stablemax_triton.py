"""Stablemax-encoder FLARE: the encoder weight exp(s) is replaced by sigma(s) = (1+s)^p (s >= 0),
(1-s)^-p (s < 0); the decode side stays a softmax over the latents.

Interface of the operator this replaces: ``FLAREAutoregressiveStablemaxTriton`` /
``flare_autoregressive_stablemax_triton`` (reference: causal_flare/autoregressive/stablemax_triton.py:1707-2465).
"""

from __future__ import annotations

import torch
from torch import autograd

from .. import _lib, _ops
from .._common import _normalize_input_precision, _resolve_attn_scale
from .._reference_utils import resolve_flare_causal_decode_inputs, validate_flare_qkv_layouts


class FLAREAutoregressiveStablemaxTriton(autograd.Function):
    """Always returns five gradients (Q, K, V, Q_dec, K_dec); when the decode tensors are the encode tensors
    themselves autograd adds the two contributions, as with the operator this replaces."""

    @staticmethod
    def forward(ctx, Q, K, V, Q_dec, K_dec, scale=None, chunk_size=None, power: float = 2.0, input_precision=None):
        B, N, H, M, D_score, D_value = validate_flare_qkv_layouts(Q, K, V, name="Stablemax Triton FLARE")
        scale_f = _resolve_attn_scale(scale, D_score)
        _normalize_input_precision(input_precision)
        Q_dec_r, K_dec_r, _, _, _ = resolve_flare_causal_decode_inputs(Q, K, Q_dec, K_dec)
        if chunk_size is not None and int(chunk_size) % 16 != 0:
            raise ValueError(
                "FLAREAutoregressiveStablemaxTriton requires a chunk size divisible by 16. "
                f"Got chunk_size={int(chunk_size)}."
            )
        ctx.meta = (B, N, H, M, D_score, D_value)
        ctx.dtypes = (Q.dtype, K.dtype, V.dtype, Q_dec_r.dtype, K_dec_r.dtype)
        ctx.scale, ctx.power = scale_f, float(power)
        ctx.alias_q = Q_dec_r is K
        ctx.alias_k = K_dec_r is Q
        if N == 0:
            ctx.empty = True
            return torch.empty((B, 0, H, D_value), device=V.device, dtype=V.dtype)
        ctx.empty = False
        if not K.is_cuda:
            raise RuntimeError("flare_autoregressive_stablemax requires CUDA tensors.")
        kept = {} if (ctx.alias_q and ctx.alias_k and any(ctx.needs_input_grad[:5])) else None
        Y, _, _, _ = _ops.forward(Q, K, V, scale=scale_f, Q_dec=None if ctx.alias_q else Q_dec_r,
                                  K_dec=None if ctx.alias_k else K_dec_r, variant=_lib.STABLEMAX, power=float(power),
                                  out_dtype=V.dtype, keep_for_backward=kept)
        ctx.has_kept = bool(kept)
        extra = [kept["y"], kept["lse_dec"], kept["keep"]] if kept else []
        ctx.save_for_backward(Q, K, V, Q_dec_r, K_dec_r, *extra)
        return Y

    @staticmethod
    def backward(ctx, dY):
        B, N, H, M, Dk, Dv = ctx.meta
        qdt, kdt, vdt, qddt, kddt = ctx.dtypes
        if ctx.empty:
            dev = dY.device
            return (
                torch.zeros((H, M, Dk), device=dev, dtype=qdt), torch.zeros((B, N, H, Dk), device=dev, dtype=kdt),
                torch.zeros((B, N, H, Dv), device=dev, dtype=vdt), torch.zeros((B, N, H, Dk), device=dev, dtype=qddt),
                torch.zeros((H, M, Dk), device=dev, dtype=kddt), None, None, None, None,
            )
        Q, K, V, Q_dec, K_dec = ctx.saved_tensors[:5]
        kept = dict(zip(("y", "lse_dec", "keep"), ctx.saved_tensors[5:8])) if ctx.has_kept else None
        if ctx.alias_q and ctx.alias_k:
            # Both decode tensors ARE the encode tensors: one score matrix, the decode-side gradients folded into dQ /
            # dK by the kernels (autograd would add the two contributions of the same tensor anyway), which is the
            # shape class of the tensor-core backward.  The two decode slots then receive no separate gradient.
            dq, dk, dv, _, _ = _ops.backward(Q, K, V, dY, scale=ctx.scale, variant=_lib.STABLEMAX, power=ctx.power,
                                             saved=kept)
            return dq.to(qdt), dk.to(kdt), dv.to(vdt), None, None, None, None, None, None
        # Run the kernels with the decode tensors treated as separate so the five gradients come out unfolded.
        dq, dk, dv, dqd, dkd = _ops.backward(Q, K, V, dY, scale=ctx.scale, Q_dec=Q_dec, K_dec=K_dec,
                                             variant=_lib.STABLEMAX, power=ctx.power)
        return dq.to(qdt), dk.to(kdt), dv.to(vdt), dqd.to(qddt), dkd.to(kddt), None, None, None, None


def flare_autoregressive_stablemax_triton(Q, K, V, scale=None, eps=None, profile=False, chunk_size=None, Q_dec=None,
                                          K_dec=None, power: float = 2.0, write_gate=False, write_gate_fixed_value=None,
                                          write_gate_tensor=None, state=None, attention_mask=None, return_state=False,
                                          input_precision=None):
    if eps is not None:
        raise NotImplementedError("flare_autoregressive_stablemax_triton does not use eps.")
    if profile:
        raise NotImplementedError("flare_autoregressive_stablemax_triton does not support profile=True")
    if state is not None:
        raise NotImplementedError("flare_autoregressive_stablemax_triton does not support recurrent state")
    if attention_mask is not None:
        raise NotImplementedError("flare_autoregressive_stablemax_triton does not support attention_mask")
    if return_state:
        raise NotImplementedError("flare_autoregressive_stablemax_triton does not support return_state=True")
    if write_gate or write_gate_fixed_value is not None or write_gate_tensor is not None:
        raise NotImplementedError("flare_autoregressive_stablemax_triton currently implements the non-write-gated path only.")
    Q_dec_r, K_dec_r, _, _, _ = resolve_flare_causal_decode_inputs(Q, K, Q_dec, K_dec)
    return FLAREAutoregressiveStablemaxTriton.apply(Q, K, V, Q_dec_r, K_dec_r, scale, chunk_size, power, input_precision)
