"""Cached inference for the block-causal operator is not defined by the operator API this package
mirrors (reference: causal_flare/semi_autoregressive/inference.py:1-36): both entry points raise."""

from torch import autograd


class SemiAutoRegressivePrefillFLARE(autograd.Function):
    @staticmethod
    def forward(ctx, *args, **kwargs):
        raise NotImplementedError("SemiAutoRegressivePrefillFLARE is not implemented yet.")


class SemiAutoRegressiveDecodeFLARE(autograd.Function):
    @staticmethod
    def forward(ctx, *args, **kwargs):
        raise NotImplementedError("SemiAutoRegressiveDecodeFLARE is not implemented yet.")


def flare_semi_autoregressive_prefill_trition(*args, **kwargs):
    raise NotImplementedError("flare_semi_autoregressive_prefill_trition is not implemented yet.")


def flare_semi_autoregressive_decode_trition(*args, **kwargs):
    raise NotImplementedError("flare_semi_autoregressive_decode_trition is not implemented yet.")


def flare_semi_autoregressive_block_prefill(Q, K, V, *, block_size, state=None, scale=None):
    """Block-granular cached inference for the block-causal operator (no counterpart in the reference, whose cached
    entry points above are stubs).

    K, V hold whole blocks ([B, T, H, D], ``T % block_size == 0``).  Every token reads the latent state at the end of
    its own block; ``state`` (the ``(m, d, u)`` dict of the autoregressive prefill API, or None for an empty state)
    carries the blocks seen so far, so a long sequence can be fed block by block - decoding is the case T == block_size.
    Returns ``(Y [B, T, H, Dv] in V's dtype, state)``; the returned state is a fresh set of tensors.
    """
    from .. import _ops
    from .._common import _resolve_attn_scale
    from ..autoregressive.inference import _canonicalize_flare_state, _init_flare_recurrent_state

    if K.dim() != 4 or V.dim() != 4 or Q.dim() != 3:
        raise ValueError("expected Q [H, M, D], K / V [B, T, H, D]")
    B, T, H, Dk = K.shape
    M, Dv = Q.shape[1], V.shape[-1]
    if block_size < 16 or block_size % 16 != 0:
        raise ValueError(f"block_size must be a positive multiple of 16. Got block_size={block_size}")
    if T % block_size != 0:
        raise ValueError(f"block-granular prefill needs whole blocks: T={T} is not a multiple of block_size={block_size}")
    st = _init_flare_recurrent_state(B, H, M, Dv, K.device) if state is None else \
        _canonicalize_flare_state(state, B, H, M, Dv, K.device)
    if T == 0:
        return V.new_empty((B, 0, H, Dv)), st
    Y, st_out, _, _ = _ops.forward(Q, K, V, scale=_resolve_attn_scale(scale, Dk), block_size=block_size, state_in=st,
                                   want_state=True, out_dtype=V.dtype)
    return Y, st_out
