"""Cached inference for the block-causal operator.

The operator API this package mirrors does not define it (reference: causal_flare/semi_autoregressive/inference.py:1-36:
both entry points and both autograd classes raise ``NotImplementedError``); those names are kept here with the
reference's signatures and behaviour.  Beside them this module offers what a serving loop needs:
``flare_semi_autoregressive_block_prefill`` (whole blocks on top of a carried state) and
``flare_semi_autoregressive_token_decode`` (one token at a time, outputs released block by block)."""

import torch
from torch import autograd


class SemiAutoRegressivePrefillFLARE(autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, state=None, scale=None, attention_mask=None, Q_dec=None, K_dec=None):
        raise NotImplementedError("SemiAutoRegressivePrefillFLARE is not implemented yet.")

    @staticmethod
    def backward(ctx, dY, dState=None):
        raise NotImplementedError("SemiAutoRegressivePrefillFLARE backward is not implemented yet.")


class SemiAutoRegressiveDecodeFLARE(autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, state=None, scale=None, Q_dec=None, K_dec=None):
        raise NotImplementedError("SemiAutoRegressiveDecodeFLARE is not implemented yet.")

    @staticmethod
    def backward(ctx, dY, dState=None):
        raise NotImplementedError("SemiAutoRegressiveDecodeFLARE backward is not implemented yet.")


def flare_semi_autoregressive_prefill_trition(Q, K, V, *, state=None, scale=None, attention_mask=None, Q_dec=None,
                                              K_dec=None):
    raise NotImplementedError("flare_semi_autoregressive_prefill_trition is not implemented yet.")


def flare_semi_autoregressive_decode_trition(Q, K, V, *, state=None, scale=None, Q_dec=None, K_dec=None):
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


class SemiAutoRegressiveTokenCache:
    """What token-by-token decoding of the block-causal operator carries between calls: the latent state ``(m, d, u)``
    of the COMPLETED blocks, and the keys / values of the tokens of the block in progress (at most ``block_size - 1``
    of them), whose outputs are still pending because every token reads the state at the END of its block."""

    def __init__(self, state, block_size):
        self.state = state
        self.block_size = int(block_size)
        self.k_buf = None  # [B, block_size, H, Dk], filled up to `count`
        self.v_buf = None
        self.count = 0

    @property
    def pending(self) -> int:
        """Tokens received whose outputs have not been released yet."""
        return self.count


def flare_semi_autoregressive_token_decode(Q, K, V, cache=None, *, block_size, scale=None):
    """One decode token of the block-causal operator (no counterpart in the reference).

    K, V: ``[B, H, D]`` or ``[B, 1, H, D]``.  Streaming semantics: the operator's output for a token is defined by the
    latent state at the end of the token's block, so nothing can be emitted for a block before its last token has
    arrived.  The call therefore buffers the token and returns ``(None, cache)`` while the block is incomplete; the
    call that delivers the block's last token returns ``(Y [B, block_size, H, Dv], cache)`` with the outputs of ALL
    tokens of that block - exactly what ``flare_semi_autoregressive_trition`` gives for them in a full-sequence call -
    and folds the block into the carried state.  ``cache`` is None for the first token (or a
    ``SemiAutoRegressiveTokenCache`` built on the state returned by ``flare_semi_autoregressive_block_prefill``)."""
    from ..autoregressive.inference import _init_flare_recurrent_state

    if (K.dim() == 4 and K.shape[1] != 1) or (V.dim() == 4 and V.shape[1] != 1):
        raise ValueError(f"token decode takes one token: K / V [B, H, D] or [B, 1, H, D]. Got K={tuple(K.shape)}, V={tuple(V.shape)}")
    K = K[:, 0] if K.dim() == 4 else K
    V = V[:, 0] if V.dim() == 4 else V
    if K.dim() != 3 or V.dim() != 3 or Q.dim() != 3:
        raise ValueError("expected Q [H, M, D], K / V [B, H, D]")
    if block_size < 16 or block_size % 16 != 0:
        raise ValueError(f"block_size must be a positive multiple of 16. Got block_size={block_size}")
    B, H, Dk = K.shape
    M, Dv = Q.shape[1], V.shape[-1]
    if cache is None:
        cache = SemiAutoRegressiveTokenCache(_init_flare_recurrent_state(B, H, M, Dv, K.device), block_size)
    if cache.block_size != block_size:
        raise ValueError(f"cache was built for block_size={cache.block_size}, call uses block_size={block_size}")
    if cache.k_buf is None:
        cache.k_buf = torch.empty((B, block_size, H, Dk), device=K.device, dtype=K.dtype)
        cache.v_buf = torch.empty((B, block_size, H, Dv), device=V.device, dtype=V.dtype)
    cache.k_buf[:, cache.count].copy_(K)
    cache.v_buf[:, cache.count].copy_(V)
    cache.count += 1
    if cache.count < block_size:
        return None, cache
    Y, cache.state = flare_semi_autoregressive_block_prefill(Q, cache.k_buf, cache.v_buf, block_size=block_size,
                                                             state=cache.state, scale=scale)
    cache.count = 0
    return Y, cache
