"""Semi-autoregressive (block-causal) FLARE: every token of block g reads the latent state after ALL
tokens of blocks <= g.

Interface of the operator this replaces: ``SemiAutoRegressiveFLARE`` / ``flare_semi_autoregressive_trition``
(sic) (reference: causal_flare/semi_autoregressive/training.py:3990-4106).  Returns ``(Y, aux)`` with
``aux = {"LSE_dec": [B,H,N], "LSE_enc": [B,H,N/block_size,M]}`` (natural-log units, fp32).
"""

from __future__ import annotations

from torch import autograd

from .. import _ops
from .._common import _normalize_input_precision, _refresh_profile_totals, _resolve_attn_scale, _timed
from .._reference_utils import resolve_flare_causal_decode_inputs, validate_flare_qkv_layouts
from .reference import _validate_block_causal_config


class SemiAutoRegressiveFLARE(autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, scale=None, block_size=None, chunk_size=None, input_precision=None, profile=False,
                Q_dec=None, K_dec=None):
        B, N, H, M, D_score, D_value = validate_flare_qkv_layouts(Q, K, V, name="SemiAutoRegressiveFLARE")
        block_size, chunk_size, _, _, _ = _validate_block_causal_config(
            N=N, block_size=block_size, chunk_size=chunk_size, name="SemiAutoRegressiveFLARE")
        resolved_scale = _resolve_attn_scale(scale, D_score)
        _normalize_input_precision(input_precision)
        Q_dec, K_dec, sep_q, sep_k, shared = resolve_flare_causal_decode_inputs(Q, K, Q_dec, K_dec)
        if shared:
            sep_q = sep_k = False
        if not K.is_cuda:
            raise RuntimeError("flare_semi_autoregressive requires CUDA tensors.")
        profile_data = {"forward": {}, "backward": {}} if profile else None
        kept = {} if any(ctx.needs_input_grad[:3]) else None
        Y, _, lse_dec, lse_enc = _timed(
            K.device, profile_data["forward"] if profile else None, "flare_forward",
            lambda: _ops.forward(Q, K, V, scale=resolved_scale, Q_dec=Q_dec if sep_q else None,
                                 K_dec=K_dec if sep_k else None, block_size=block_size, want_lse=True, out_dtype=V.dtype,
                                 keep_for_backward=kept),
        )
        ctx.has_kept = bool(kept)
        aux = {"LSE_dec": lse_dec, "LSE_enc": lse_enc}
        saved = [Q, K, V] + ([Q_dec] if sep_q else []) + ([K_dec] if sep_k else [])
        if kept:
            saved += [kept["y"], kept["lse_dec"], kept["keep"]]
        ctx.save_for_backward(*saved)
        ctx.scale, ctx.block_size, ctx.sep_q, ctx.sep_k = resolved_scale, block_size, sep_q, sep_k
        ctx.profile_timings = profile_data
        ctx.mark_non_differentiable(lse_dec, lse_enc)
        if profile:
            _refresh_profile_totals(profile_data)
            return Y, aux, profile_data
        return Y, aux

    @staticmethod
    def backward(ctx, dY, *unused):
        if dY is None:
            return (None,) * 10
        saved = list(ctx.saved_tensors)
        Q, K, V = saved[:3]
        rest = saved[3:]
        Q_dec = rest.pop(0) if ctx.sep_q else None
        K_dec = rest.pop(0) if ctx.sep_k else None
        kept = dict(y=rest[0], lse_dec=rest[1], keep=rest[2]) if ctx.has_kept else None
        prof = ctx.profile_timings
        dq, dk, dv, dqd, dkd = _timed(
            K.device, prof["backward"] if prof is not None else None, "flare_backward",
            lambda: _ops.backward(Q, K, V, dY, scale=ctx.scale, Q_dec=Q_dec, K_dec=K_dec, block_size=ctx.block_size,
                                  saved=kept),
        )
        if prof is not None:
            _refresh_profile_totals(prof)
        return (
            dq.to(Q.dtype), dk.to(K.dtype), dv.to(V.dtype), None, None, None, None, None,
            None if dqd is None else dqd.to(Q_dec.dtype), None if dkd is None else dkd.to(K_dec.dtype),
        )


def flare_semi_autoregressive_trition(Q, K, V, *, block_size, chunk_size, scale=None, input_precision=None,
                                      profile: bool = False, Q_dec=None, K_dec=None):
    """Block-causal FLARE.  ``block_size`` (multiple of 16, divides N) and ``chunk_size`` (16/32/64/128, divides
    block_size) are both required; ``chunk_size`` does not change the result."""
    return SemiAutoRegressiveFLARE.apply(Q, K, V, scale, block_size, chunk_size, input_precision, profile, Q_dec, K_dec)
