"""Recurrent (un-chunked) autoregressive FLARE.  Output layout is [B, H, N, D] in Q.dtype.

Interface of the operator this replaces: ``RecurrentFLARE`` / ``flare_recurrent_triton``
(reference: causal_flare/autoregressive/recurrent.py:288-414, :1191-1204).  The math is the same
token recurrence as the chunked operator, so both share the sequential-walk kernels; the backward is
the O(N) reverse recurrence instead of the reference's O(N^2) kernels.
"""

from __future__ import annotations

from torch import autograd

from .. import _ops
from .._common import _resolve_attn_scale
from .._reference_utils import resolve_flare_causal_decode_inputs


class RecurrentFLARE(autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, scale=None, block_m=None, block_d=None, Q_dec=None, K_dec=None, block_t=None):
        if Q.dim() != 3 or K.dim() != 4 or V.dim() != 4:
            raise ValueError(
                "Recurrent FLARE expects Q [H, M, D] and K/V [B, N, H, D]. "
                f"Got Q.dim()={Q.dim()}, K.dim()={K.dim()}, V.dim()={V.dim()}"
            )
        if K.size() != V.size():
            raise ValueError(f"K and V must have the same shape. Got K.shape={K.shape} and V.shape={V.shape}")
        if Q.size(0) != K.size(2) or Q.size(2) != K.size(3):
            raise ValueError(
                "Expected Q [H, M, D] and K/V [B, N, H, D] with matching H,D. "
                f"Got Q.shape={Q.shape} and K.shape={K.shape}"
            )
        H, M, D = Q.size()
        scale = _resolve_attn_scale(scale, D)
        Q_dec, K_dec, sep_q, sep_k, shared = resolve_flare_causal_decode_inputs(Q, K, Q_dec, K_dec)
        if shared:
            sep_q = sep_k = False
        if (M % 16) != 0 or (D % 16) != 0:
            raise ValueError(f"RecurrentFLARE requires M and D be multiples of 16. Got M={M}, D={D}")
        if block_t is not None and int(block_t) not in (1, 16, 32):
            raise ValueError(f"block_t must be one of (1, 16, 32). Got block_t={block_t}")
        if not K.is_cuda:
            raise RuntimeError("flare_recurrent requires CUDA tensors.")
        Y, _, _, _ = _ops.forward(Q, K, V, scale=scale, Q_dec=Q_dec if sep_q else None, K_dec=K_dec if sep_k else None,
                                  out_bhnd=True, out_dtype=Q.dtype)
        saved = [Q, K, V] + ([Q_dec] if sep_q else []) + ([K_dec] if sep_k else [])
        ctx.save_for_backward(*saved)
        ctx.scale, ctx.sep_q, ctx.sep_k = scale, sep_q, sep_k
        return Y

    @staticmethod
    def backward(ctx, dY):
        if dY is None:
            return (None,) * 9
        saved = list(ctx.saved_tensors)
        Q, K, V = saved[:3]
        rest = saved[3:]
        Q_dec = rest.pop(0) if ctx.sep_q else None
        K_dec = rest.pop(0) if ctx.sep_k else None
        dq, dk, dv, dqd, dkd = _ops.backward(Q, K, V, dY, scale=ctx.scale, Q_dec=Q_dec, K_dec=K_dec, dy_bhnd=True)
        return (
            dq.to(Q.dtype), dk.to(K.dtype), dv.to(V.dtype), None, None, None,
            None if dqd is None else dqd.to(Q_dec.dtype), None if dkd is None else dkd.to(K_dec.dtype), None,
        )


def flare_recurrent_triton(Q, K, V, scale=None, *, block_m=None, block_d=None, Q_dec=None, K_dec=None, block_t=None):
    """Recurrent FLARE; returns Y [B, H, N, D].  The block_* tile hints are accepted and ignored."""
    return RecurrentFLARE.apply(Q, K, V, scale, block_m, block_d, Q_dec, K_dec, block_t)
