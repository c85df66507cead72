"""Cached inference: chunked prefill with carry-in state and the single-token decode step.

Interface of the operators these replace: ``flare_autoregressive_prefill_triton`` /
``flare_autoregressive_decode_triton`` (reference: causal_flare/autoregressive/inference.py:492-820).
The recurrent state is a dict of fp32 tensors {"m": [B,H,M], "d": [B,H,M], "u": [B,H,M,Dv]}: running
max, denominator and un-normalised numerator of every latent's softmax over the tokens seen so far.
Note the default ``scale=1.0`` of both wrappers (the training operator defaults to Dk ** -0.5).
"""

from __future__ import annotations

import torch

from .. import _ops
from .._common import _normalize_input_precision, _refresh_profile_totals, _timed
from .._reference_utils import resolve_flare_causal_decode_inputs


def _init_flare_recurrent_state(batch_size, num_heads, num_latents, value_head_dim, device, dtype=torch.float32):
    return {
        "m": torch.full((batch_size, num_heads, num_latents), -torch.inf, device=device, dtype=dtype),
        "d": torch.zeros((batch_size, num_heads, num_latents), device=device, dtype=dtype),
        "u": torch.zeros((batch_size, num_heads, num_latents, value_head_dim), device=device, dtype=dtype),
    }


def _canonicalize_flare_state(state, batch_size, num_heads, num_latents, value_head_dim, device):
    """None -> empty state; otherwise validate keys/shapes and view as fp32 on ``device`` (no copy if already so)."""
    if state is None:
        return _init_flare_recurrent_state(batch_size, num_heads, num_latents, value_head_dim, device)
    if not isinstance(state, dict):
        raise ValueError(f"FLARE recurrent state must be a dict with keys {'m', 'd', 'u'}. Got {type(state)}")
    if not all(k in state for k in ("m", "d", "u")):
        raise ValueError(f"Invalid FLARE recurrent state keys: {list(state.keys())}")
    m = state["m"].to(device=device, dtype=torch.float32)
    d = state["d"].to(device=device, dtype=torch.float32)
    u = state["u"].to(device=device, dtype=torch.float32)
    exp_s = (batch_size, num_heads, num_latents)
    exp_u = (batch_size, num_heads, num_latents, value_head_dim)
    if tuple(m.shape) != exp_s or tuple(d.shape) != exp_s or tuple(u.shape) != exp_u:
        raise ValueError(
            "Invalid FLARE recurrent state shapes. "
            f"Expected m/d={exp_s}, u={exp_u}; got m={tuple(m.shape)}, d={tuple(d.shape)}, u={tuple(u.shape)}"
        )
    return {"m": m, "d": d, "u": u}


def _merge_flare_stats(m_a, d_a, u_a, m_b, d_b, u_b):
    """Associative merge of two states (inf-safe), computed by the CUDA fold kernel."""
    lead = m_a.shape[:-1]
    M, Dv = u_a.shape[-2], u_a.shape[-1]

    def as4(m, d, u):
        return {"m": m.reshape(1, -1, M), "d": d.reshape(1, -1, M), "u": u.reshape(1, -1, M, Dv)}

    out = _ops.merge_states(as4(m_a, d_a, u_a), [as4(m_b, d_b, u_b)])
    return out["m"].reshape(*lead, M), out["d"].reshape(*lead, M), out["u"].reshape(*lead, M, Dv)


def _canonicalize_kv_for_decode(K, V):
    if K.dim() == 4 and K.shape[1] == 1:
        K = K[:, 0]
    if V.dim() == 4 and V.shape[1] == 1:
        V = V[:, 0]
    if K.dim() != 3 or V.dim() != 3:
        raise ValueError(f"Decode expects K/V as [B, H, D] or [B, 1, H, D]. Got K={tuple(K.shape)}, V={tuple(V.shape)}")
    if K.shape[:2] != V.shape[:2]:
        raise ValueError(f"Decode expects K and V to agree on [B, H]. Got K={tuple(K.shape)}, V={tuple(V.shape)}")
    return K, V


def _canonicalize_q_dec_for_decode(Q_dec, K_step, K_input):
    """Returns the decode query as [B, H, D], or None when it is (by identity) the step's key."""
    if Q_dec is None or Q_dec is K_step or Q_dec is K_input:
        return None
    if Q_dec.dim() == 3:
        if Q_dec.shape != K_step.shape:
            raise ValueError(
                "Decode Q_dec must match K decode-step shape. "
                f"Got Q_dec.shape={tuple(Q_dec.shape)} and K.shape={tuple(K_step.shape)}"
            )
        return Q_dec
    if Q_dec.dim() == 4:
        if Q_dec.shape[0] != K_step.shape[0] or Q_dec.shape[2] != K_step.shape[1] or Q_dec.shape[3] != K_step.shape[2]:
            raise ValueError(
                "Decode Q_dec [B, 1, H, D] must match K [B, H, D]. "
                f"Got Q_dec.shape={tuple(Q_dec.shape)} and K.shape={tuple(K_step.shape)}"
            )
        if Q_dec.shape[1] != 1:
            raise ValueError(f"Decode Q_dec with rank-4 must have sequence length 1. Got Q_dec.shape={tuple(Q_dec.shape)}")
        return Q_dec[:, 0]
    raise ValueError(f"Decode Q_dec must be [B, H, D] or [B, 1, H, D]. Got Q_dec.shape={tuple(Q_dec.shape)}")


def flare_autoregressive_decode_triton(Q, K, V, state=None, scale=1.0, input_precision=None, attention_mask=None,
                                       Q_dec=None, K_dec=None, profile=False):
    """One decode token.  K, V: [B,H,D] or [B,1,H,D].  Returns ``(y [B,1,H,Dv] in V.dtype, state)``.

    The state tensors are updated IN PLACE when the passed state is already fp32 and contiguous
    (the returned dict then shares storage with the caller's)."""
    if not Q.is_cuda:
        raise RuntimeError("flare_autoregressive_decode requires CUDA tensors. ")
    K_input = K
    K, V = _canonicalize_kv_for_decode(K, V)
    _normalize_input_precision(input_precision)
    B, H, D_score = K.shape
    D_value = V.shape[-1]
    Hq, M, Dq = Q.shape
    if Hq != H or Dq != D_score:
        raise ValueError(f"Incompatible Q/K shapes. Q={tuple(Q.shape)}, K={tuple(K.shape)}")
    q_dec = _canonicalize_q_dec_for_decode(Q_dec, K, K_input)
    if q_dec is not None and q_dec.shape != K.shape:
        raise ValueError(f"Q_dec and K_enc must have the same shape. Got Q_dec.shape={q_dec.shape} and K_enc.shape={K.shape}")
    if K_dec is not None and K_dec is not Q:
        if K_dec.dim() != 3:
            raise ValueError(f"Expected K_dec [H, M, D]. Got K_dec.dim()={K_dec.dim()} and K_dec.shape={tuple(K_dec.shape)}")
        if K_dec.size() != Q.size():
            raise ValueError(f"K_dec and Q_enc must have the same shape. Got K_dec.shape={K_dec.shape} and Q_enc.shape={Q.shape}")
    else:
        K_dec = None
    if attention_mask is not None:
        if attention_mask.dim() == 2 and attention_mask.shape[1] == 1:
            attention_mask = attention_mask[:, 0]
        if attention_mask.dim() != 1 or attention_mask.shape[0] != B:
            raise ValueError(f"Decode attention_mask must be [B] or [B, 1]. Got {tuple(attention_mask.shape)}")
    st = _canonicalize_flare_state(state, B, H, M, D_value, K.device)
    st = {k: st[k].contiguous() for k in ("m", "d", "u")}
    profile_data = {"forward": {}} if profile else None
    y = _timed(
        K.device, profile_data["forward"] if profile else None, "flare_decode_step",
        lambda: _ops.decode_step(Q, K, V, st, scale=float(scale), q_dec=q_dec, K_dec=K_dec, mask=attention_mask),
    )
    y_out = y[:, None]
    if y_out.dtype != V.dtype:
        y_out = y_out.to(V.dtype)
    if profile:
        _refresh_profile_totals(profile_data)
        return (y_out, st), profile_data
    return y_out, st


def flare_autoregressive_prefill_triton(Q, K, V, state=None, scale=1.0, input_precision=None, attention_mask=None,
                                        Q_dec=None, K_dec=None, profile=False):
    """Prefill T tokens on top of an optional carry-in state.  Returns ``(Y [B,T,H,Dv] in V.dtype, state)``.

    A token whose ``attention_mask`` entry is 0 leaves the state untouched and yields y = 0."""
    if not Q.is_cuda:
        raise RuntimeError("flare_autoregressive_prefill requires CUDA tensors.")
    if K.dim() != 4 or V.dim() != 4:
        raise ValueError(f"Prefill expects K/V to be [B, T, H, D]. Got K={tuple(K.shape)}, V={tuple(V.shape)}")
    if K.shape[:3] != V.shape[:3]:
        raise ValueError(f"Prefill expects K and V to agree on [B, T, H]. Got K={tuple(K.shape)}, V={tuple(V.shape)}")
    B, T, H, D_score = K.shape
    D_value = V.shape[-1]
    if Q.dim() != 3:
        raise ValueError(f"Q must be [H, M, D]. Got Q={tuple(Q.shape)}")
    Hq, M, Dq = Q.shape
    if Hq != H or Dq != D_score:
        raise ValueError(f"Incompatible Q/K shapes. Q={tuple(Q.shape)}, K={tuple(K.shape)}")
    if attention_mask is not None and attention_mask.shape != (B, T):
        raise ValueError(f"attention_mask must be [B, T]. Got {tuple(attention_mask.shape)}")
    _normalize_input_precision(input_precision)
    Q_dec, K_dec, separate_Q_dec, separate_K_dec, shared = resolve_flare_causal_decode_inputs(Q, K, Q_dec, K_dec)
    if shared:
        separate_Q_dec = separate_K_dec = False
    st = _canonicalize_flare_state(state, B, H, M, D_value, K.device)
    if T == 0:
        return torch.empty((B, 0, H, D_value), device=K.device, dtype=V.dtype), st
    st = {k: st[k].contiguous() for k in ("m", "d", "u")}
    profile_data = {"forward": {}} if profile else None
    Y, st_out, _, _ = _timed(
        K.device, profile_data["forward"] if profile else None, "flare_forward",
        lambda: _ops.forward(Q, K, V, scale=float(scale), Q_dec=Q_dec if separate_Q_dec else None,
                             K_dec=K_dec if separate_K_dec else None, mask=attention_mask, state_in=st,
                             want_state=True, out_dtype=V.dtype),
    )
    if profile:
        _refresh_profile_totals(profile_data)
        return (Y, st_out), profile_data
    return Y, st_out


def flare_prefill(Q, K, V, state=None, scale=1.0, input_precision=None, attention_mask=None, impl="triton",
                  Q_dec=None, K_dec=None):
    if impl != "triton":
        raise ValueError(f"Unsupported impl={impl}. This package ships only the CUDA implementation ('triton' slot).")
    return flare_autoregressive_prefill_triton(Q=Q, K=K, V=V, Q_dec=Q_dec, K_dec=K_dec, state=state, scale=scale,
                                               input_precision=input_precision, attention_mask=attention_mask)


def flare_decode(Q, K, V, state, scale=1.0, input_precision=None, attention_mask=None, impl="triton",
                 Q_dec=None, K_dec=None):
    if impl != "triton":
        raise ValueError(f"Unsupported impl={impl}. This package ships only the CUDA implementation ('triton' slot).")
    return flare_autoregressive_decode_triton(Q=Q, K=K, V=V, state=state, Q_dec=Q_dec, K_dec=K_dec, scale=scale,
                                              input_precision=input_precision, attention_mask=attention_mask)
