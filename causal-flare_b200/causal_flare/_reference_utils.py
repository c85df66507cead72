"""Layout validation and the decode-weight aliasing rule of the public operators."""

from __future__ import annotations


def validate_flare_qkv_layouts(Q, K, V, *, name: str):
    """Q [H, M, D_k]; K [B, N, H, D_k]; V [B, N, H, D_v].  Returns (B, N, H, M, D_k, D_v)."""
    if Q.dim() != 3 or K.dim() != 4 or V.dim() != 4:
        raise ValueError(
            f"{name} expects Q [H, M, D_k] and K/V [B, N, H, D]. "
            f"Got Q.dim()={Q.dim()}, K.dim()={K.dim()}, V.dim()={V.dim()}"
        )
    if K.shape[:3] != V.shape[:3]:
        raise ValueError(f"{name} expects K and V to agree on [B, N, H]. Got K.shape={K.shape} and V.shape={V.shape}")
    if Q.size(0) != K.size(2) or Q.size(2) != K.size(3):
        raise ValueError(
            f"{name} expects Q [H, M, D_k] and K [B, N, H, D_k] with matching H,D_k. "
            f"Got Q.shape={Q.shape} and K.shape={K.shape}"
        )
    return V.shape[0], V.shape[1], Q.shape[0], Q.shape[1], Q.shape[2], V.shape[3]


def resolve_flare_causal_decode_inputs(Q_enc, K_enc, Q_dec=None, K_dec=None):
    """Decode weights default to the encode tensors.  Passing the very same tensor object
    (``Q_dec is K_enc`` / ``K_dec is Q_enc``) counts as the default; an equal-valued copy is separate.

    Returns (Q_dec, K_dec, separate_Q_dec, separate_K_dec, weight_sharing)."""
    separate_Q_dec = Q_dec is not None
    separate_K_dec = K_dec is not None
    default_q = (not separate_Q_dec) or (Q_dec is K_enc)
    default_k = (not separate_K_dec) or (K_dec is Q_enc)
    if separate_Q_dec:
        if Q_dec.dim() != 4:
            raise ValueError(
                f"Expected Q_dec [B, N, H, D]. Got Q_dec.dim()={Q_dec.dim()} and Q_dec.shape={tuple(Q_dec.shape)}"
            )
        if Q_dec.size() != K_enc.size():
            raise ValueError(
                f"Q_dec and K_enc must have the same shape. Got Q_dec.shape={Q_dec.shape} and K_enc.shape={K_enc.shape}"
            )
    else:
        Q_dec = K_enc
    if separate_K_dec:
        if K_dec.dim() != 3:
            raise ValueError(
                f"Expected K_dec [H, M, D]. Got K_dec.dim()={K_dec.dim()} and K_dec.shape={tuple(K_dec.shape)}"
            )
        if K_dec.size() != Q_enc.size():
            raise ValueError(
                f"K_dec and Q_enc must have the same shape. Got K_dec.shape={K_dec.shape} and Q_enc.shape={Q_enc.shape}"
            )
    else:
        K_dec = Q_enc
    return Q_dec, K_dec, separate_Q_dec, separate_K_dec, default_q and default_k
