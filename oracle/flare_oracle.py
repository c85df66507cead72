"""CPU oracle for Causal FLARE attention.  TEST INFRASTRUCTURE ONLY.

This module is a plain-PyTorch (CPU) restatement of the algorithm implemented by the
reference project's PyTorch paths.  It exists to check the CUDA library; it is never
imported by the product package.  Only the test-suite, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it.

Parity status: PINNED.  Every function below is checked against the outputs of the
reference's own functions (imported from the reference checkout when the fixtures
were generated, see ``tests/golden/make_golden.py``) and against the committed
fixtures under ``tests/golden/``.

Reference locations each function follows (paths inside the reference project):

* ``resolve_scale``            causal_flare/_common.py:201-204
* ``resolve_decode_inputs``    causal_flare/_reference_utils.py:24-57
* ``merge_states``             causal_flare/autoregressive/inference.py:194-228
* ``ar_forward``               causal_flare/autoregressive/reference.py:15-47 (definition),
                               causal_flare/autoregressive/inference.py:231-315 (online form,
                               state, mask), causal_flare/autoregressive/recurrent.py:17-57
* stablemax transform          causal_flare/autoregressive/stablemax.py:45-67, forward :588-632
* ``ar_forward_chunked``       causal_flare/autoregressive/reference.py:203-503, :514 (three-phase chunked form)
* ``semi_ar_forward``          causal_flare/semi_autoregressive/reference.py:308-497, :560-597
* closed-form gradients        derived from causal_flare/autoregressive/training.py:3728-4178,
                               cross-checked against autograd through the forward oracle

Layouts are the public ones: Q [H, M, Dk], K [B, N, H, Dk], V [B, N, H, Dv], Y [B, N, H, Dv].
State dict: {"m": [B, H, M], "d": [B, H, M], "u": [B, H, M, Dv]}.
"""

from __future__ import annotations

import math

import torch

NEG_INF = -float("inf")


# --------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------
def resolve_scale(scale, head_dim: int) -> float:
    if scale is not None:
        return float(scale)
    return 1.0 if head_dim <= 8 else head_dim ** -0.5


def resolve_decode_inputs(Q, K, Q_dec=None, K_dec=None):
    """Identity-based aliasing rule: ``Q_dec is K`` / ``K_dec is Q`` mean "not separate"."""
    sep_q = Q_dec is not None
    sep_k = K_dec is not None
    default_q = (not sep_q) or (Q_dec is K)
    default_k = (not sep_k) or (K_dec is Q)
    if not sep_q:
        Q_dec = K
    if not sep_k:
        K_dec = Q
    return Q_dec, K_dec, sep_q, sep_k, (default_q and default_k)


def init_state(B, H, M, Dv, dtype=torch.float32):
    return {
        "m": torch.full((B, H, M), NEG_INF, dtype=dtype),
        "d": torch.zeros((B, H, M), dtype=dtype),
        "u": torch.zeros((B, H, M, Dv), dtype=dtype),
    }


def stablemax_sigma(x: torch.Tensor, power: float = 2.0) -> torch.Tensor:
    pos = torch.where(x >= 0, x + 1.0, torch.ones_like(x))
    neg = torch.where(x < 0, 1.0 - x, torch.ones_like(x))
    return torch.where(x >= 0, pos ** power, neg ** (-power))


def stablemax_sigma_grad(x: torch.Tensor, power: float = 2.0) -> torch.Tensor:
    pos = torch.where(x >= 0, x + 1.0, torch.ones_like(x))
    neg = torch.where(x < 0, 1.0 - x, torch.ones_like(x))
    return torch.where(x >= 0, power * pos ** (power - 1.0), power * neg ** (-power - 1.0))


def _is_neg_inf(x):
    return torch.isinf(x) & (x < 0)


def merge_states(a, b):
    """Associative merge of two (m, d, u) states, safe for m = -inf."""
    m_a, d_a, u_a = a["m"], a["d"], a["u"]
    m_b, d_b, u_b = b["m"], b["d"], b["u"]
    m_new = torch.maximum(m_a, m_b)
    a_inf, b_inf, n_inf = _is_neg_inf(m_a), _is_neg_inf(m_b), _is_neg_inf(m_new)
    m_safe = torch.where(n_inf, torch.zeros_like(m_new), m_new)
    one, zero = torch.ones_like(m_new), torch.zeros_like(m_new)
    s_a = torch.where(a_inf & n_inf, one, torch.where(a_inf, zero, torch.exp(m_a - m_safe)))
    s_b = torch.where(b_inf & n_inf, one, torch.where(b_inf, zero, torch.exp(m_b - m_safe)))
    return {
        "m": m_new,
        "d": d_a * s_a + d_b * s_b,
        "u": u_a * s_a[..., None] + u_b * s_b[..., None],
    }


def _online_update(m, d, u, s_t, v_t):
    """One token of the inf-safe online-softmax recurrence. s_t [B,H,M], v_t [B,H,Dv]."""
    m_new = torch.maximum(m, s_t)
    m_inf, n_inf = _is_neg_inf(m), _is_neg_inf(m_new)
    m_safe = torch.where(n_inf, torch.zeros_like(m_new), m_new)
    gamma = torch.where(
        m_inf & n_inf,
        torch.ones_like(m_new),
        torch.where(m_inf, torch.zeros_like(m_new), torch.exp(m - m_safe)),
    )
    eta = torch.where(n_inf, torch.zeros_like(s_t), torch.exp(s_t - m_safe))
    d = d * gamma + eta
    u = u * gamma[..., None] + eta[..., None] * v_t[:, :, None, :]
    return m_new, d, u


# --------------------------------------------------------------------------------------
# autoregressive forward (softmax / stablemax encoders), with state and mask
# --------------------------------------------------------------------------------------
def ar_forward(
    Q,
    K,
    V,
    *,
    scale=None,
    Q_dec=None,
    K_dec=None,
    state=None,
    attention_mask=None,
    variant: str = "softmax",
    power: float = 2.0,
    dtype=torch.float64,
    return_state: bool = False,
):
    """Token-by-token causal FLARE.  Returns Y [B,N,H,Dv] (``dtype``) and optionally the state.

    softmax encoder:  z_t[m] = sum_{tau<=t} softmax_tau(s[tau,m]) v_tau, kept online as (m,d,u).
    stablemax encoder: exp() replaced by sigma(); state is (0, sum sigma, sum sigma v).
    decode side:      y_t = sum_m softmax_m(a[t,:])[m] z_t[m].
    A masked token (attention_mask == 0) leaves the state untouched and emits y = 0.
    """
    B, N, H, Dk = K.shape
    M = Q.shape[1]
    Dv = V.shape[-1]
    scale = resolve_scale(scale, Dk)
    Q_dec, K_dec, sep_q, sep_k, shared = resolve_decode_inputs(Q, K, Q_dec, K_dec)

    Qf = Q.to(dtype)
    Kf = K.to(dtype).permute(0, 2, 1, 3)  # [B,H,N,Dk]
    Vf = V.to(dtype).permute(0, 2, 1, 3)
    Qd = Q_dec.to(dtype).permute(0, 2, 1, 3) if sep_q else Kf
    Kd = K_dec.to(dtype) if sep_k else Qf

    if state is None:
        st = init_state(B, H, M, Dv, dtype)
        if variant == "stablemax":
            st["m"] = torch.zeros((B, H, M), dtype=dtype)
    else:
        st = {k: state[k].to(dtype).clone() for k in ("m", "d", "u")}
    m, d, u = st["m"], st["d"], st["u"]

    Y = torch.zeros((B, H, N, Dv), dtype=dtype)
    S_all = scale * torch.einsum("bhnd,hmd->bhnm", Kf, Qf)
    A_all = S_all if shared else scale * torch.einsum("bhnd,hmd->bhnm", Qd, Kd)
    for t in range(N):
        s_t = S_all[:, :, t]
        v_t = Vf[:, :, t]
        if attention_mask is not None:
            valid = attention_mask[:, t].to(torch.bool).view(B, 1, 1)
        else:
            valid = torch.ones((B, 1, 1), dtype=torch.bool)
        if variant == "softmax":
            s_in = torch.where(valid, s_t, torch.full_like(s_t, NEG_INF))
            m, d, u = _online_update(m, d, u, s_in, v_t)
        else:
            w = stablemax_sigma(s_t, power) * valid.to(dtype)
            d = d + w
            u = u + w[..., None] * v_t[:, :, None, :]
        d_safe = torch.where(d > 0, d, torch.ones_like(d))
        z = u / d_safe[..., None]
        a_t = torch.where(valid, A_all[:, :, t], torch.zeros_like(s_t))
        alpha = torch.softmax(a_t, dim=-1) * valid.to(dtype)
        Y[:, :, t] = torch.einsum("bhm,bhmd->bhd", alpha, z)
    Y = Y.permute(0, 2, 1, 3).contiguous()
    if return_state:
        return Y, {"m": m, "d": d, "u": u}
    return Y


def ar_forward_chunked(Q, K, V, *, scale=None, chunk_size=64, dtype=torch.float32):
    """Chunked causal FLARE forward, shared decode weights, no state / mask: the three phases of the reference's
    ``flare_causal_chunked`` (causal_flare/autoregressive/reference.py:203-503, :514): (1) per-chunk summaries
    (chunk max, sum of exp, exp-weighted sum of V) as batched products, (2) sequential prefix scan of the summaries
    over the chunks, (3) replay of the token recurrence inside every chunk from its prefix state.  The reference walks
    phase 3 chunk by chunk; here the chunks (independent once their prefix states are known) are replayed side by
    side, which is the same arithmetic in a different loop order."""
    B, N, H, Dk = K.shape
    M, Dv = Q.shape[1], V.shape[-1]
    C = int(chunk_size)
    scale = resolve_scale(scale, Dk)
    NC = (N + C - 1) // C
    pad = NC * C - N
    Qf = Q.to(dtype)
    Kf = K.to(dtype).permute(0, 2, 1, 3)
    Vf = V.to(dtype).permute(0, 2, 1, 3)
    S = scale * torch.einsum("bhnd,hmd->bhnm", Kf, Qf)
    if pad:
        S = torch.cat([S, torch.full((B, H, pad, M), NEG_INF, dtype=dtype)], dim=2)
        Vf = torch.cat([Vf, torch.zeros((B, H, pad, Dv), dtype=dtype)], dim=2)
    Sc = S.view(B, H, NC, C, M)
    Vc = Vf.reshape(B, H, NC, C, Dv)
    # phase 1: chunk summaries
    cmax = Sc.amax(dim=3)
    cmax_safe = torch.where(_is_neg_inf(cmax), torch.zeros_like(cmax), cmax)
    cexp = torch.exp(Sc - cmax_safe.unsqueeze(3))
    cden = cexp.sum(dim=3)
    cnum = torch.einsum("bhctm,bhctd->bhcmd", cexp, Vc)
    # phase 2: exclusive prefix scan over the chunks
    pm = torch.empty((B, H, NC, M), dtype=dtype)
    pd = torch.empty((B, H, NC, M), dtype=dtype)
    pu = torch.empty((B, H, NC, M, Dv), dtype=dtype)
    m = torch.full((B, H, M), NEG_INF, dtype=dtype)
    d = torch.zeros((B, H, M), dtype=dtype)
    u = torch.zeros((B, H, M, Dv), dtype=dtype)
    for c in range(NC):
        pm[:, :, c], pd[:, :, c], pu[:, :, c] = m, d, u
        m_new = torch.maximum(m, cmax[:, :, c])
        m_safe = torch.where(_is_neg_inf(m_new), torch.zeros_like(m_new), m_new)
        a = torch.where(_is_neg_inf(m), torch.zeros_like(m), torch.exp(m - m_safe))
        b = torch.where(_is_neg_inf(cmax[:, :, c]), torch.zeros_like(m), torch.exp(cmax[:, :, c] - m_safe))
        d = d * a + cden[:, :, c] * b
        u = u * a[..., None] + cnum[:, :, c] * b[..., None]
        m = m_new
    # phase 3: token replay inside the chunks
    Y = torch.zeros((B, H, NC, C, Dv), dtype=dtype)
    m, d, u = pm, pd, pu
    for t in range(C):
        s_t = Sc[:, :, :, t]
        v_t = Vc[:, :, :, t]
        m_new = torch.maximum(m, s_t)
        m_safe = torch.where(_is_neg_inf(m_new), torch.zeros_like(m_new), m_new)
        gamma = torch.where(_is_neg_inf(m), torch.zeros_like(m), torch.exp(m - m_safe))
        eta = torch.where(_is_neg_inf(s_t), torch.zeros_like(s_t), torch.exp(s_t - m_safe))
        d = d * gamma + eta
        u = u * gamma[..., None] + eta[..., None] * v_t[:, :, :, None, :]
        m = m_new
        z = u / torch.where(d > 0, d, torch.ones_like(d))[..., None]
        alpha = torch.softmax(torch.where(_is_neg_inf(s_t), torch.zeros_like(s_t), s_t), dim=-1)
        Y[:, :, :, t] = torch.einsum("bhcm,bhcmd->bhcd", alpha, z)
    return Y.reshape(B, H, NC * C, Dv)[:, :, :N].permute(0, 2, 1, 3).contiguous()


def decode_step(Q, k, v, state, *, scale=1.0, q_dec=None, K_dec=None, attention_mask=None, dtype=torch.float64):
    """One decode token: k, v [B,H,D].  Returns y [B,1,H,Dv] and the new state."""
    Kp = k[:, None]
    Qd = None if q_dec is None else q_dec[:, None]
    mask = None if attention_mask is None else attention_mask.reshape(-1, 1)
    y, st = ar_forward(
        Q, Kp, v[:, None], scale=scale, Q_dec=Qd, K_dec=K_dec, state=state,
        attention_mask=mask, dtype=dtype, return_state=True,
    )
    return y, st


# --------------------------------------------------------------------------------------
# semi-autoregressive (block-causal) forward
# --------------------------------------------------------------------------------------
def semi_ar_forward(Q, K, V, *, block_size, scale=None, Q_dec=None, K_dec=None, dtype=torch.float64):
    """Every token of block g reads the latent state after ALL tokens of blocks <= g.

    Returns (Y [B,N,H,Dv], LSE_dec [B,H,N], LSE_enc [B,H,NB,M]) in natural-log units.
    """
    B, N, H, Dk = K.shape
    M = Q.shape[1]
    Dv = V.shape[-1]
    assert N % block_size == 0
    NB = N // block_size
    scale = resolve_scale(scale, Dk)
    Q_dec, K_dec, sep_q, sep_k, shared = resolve_decode_inputs(Q, K, Q_dec, K_dec)
    Qf = Q.to(dtype)
    Kf = K.to(dtype).permute(0, 2, 1, 3)
    Vf = V.to(dtype).permute(0, 2, 1, 3)
    Qd = Q_dec.to(dtype).permute(0, 2, 1, 3) if sep_q else Kf
    Kd = K_dec.to(dtype) if sep_k else Qf

    S = scale * torch.einsum("bhnd,hmd->bhnm", Kf, Qf)
    A = S if shared else scale * torch.einsum("bhnd,hmd->bhnm", Qd, Kd)
    lse_dec = torch.logsumexp(A, dim=-1)
    alpha = torch.exp(A - lse_dec[..., None])

    Y = torch.empty((B, H, N, Dv), dtype=dtype)
    lse_enc = torch.empty((B, H, NB, M), dtype=dtype)
    for g in range(NB):
        end = (g + 1) * block_size
        Sg = S[:, :, :end]  # [B,H,end,M]
        L = torch.logsumexp(Sg, dim=2)  # [B,H,M]
        P = torch.exp(Sg - L[:, :, None, :])
        z = torch.einsum("bhnm,bhnd->bhmd", P, Vf[:, :, :end])
        lse_enc[:, :, g] = L
        sl = slice(g * block_size, end)
        Y[:, :, sl] = torch.einsum("bhtm,bhmd->bhtd", alpha[:, :, sl], z)
    return Y.permute(0, 2, 1, 3).contiguous(), lse_dec, lse_enc


# --------------------------------------------------------------------------------------
# gradients: autograd through the oracle forward, and the closed form the kernels use
# --------------------------------------------------------------------------------------
def grads_autograd(forward_fn, tensors: dict, dY, dtype=torch.float64):
    """Gradients of <forward_fn(**tensors), dY> w.r.t. every tensor in ``tensors``."""
    leaves = {k: v.detach().to(dtype).clone().requires_grad_(True) for k, v in tensors.items() if v is not None}
    y = forward_fn(**leaves)
    if isinstance(y, tuple):
        y = y[0]
    g = torch.autograd.grad(y, list(leaves.values()), dY.to(dtype), allow_unused=True)
    return {("d" + k): gi for k, gi in zip(leaves.keys(), g)}


def ar_backward_closed_form(
    Q, K, V, dY, *, scale=None, Q_dec=None, K_dec=None, variant="softmax", power=2.0, block_size=1,
    dtype=torch.float64,
):
    """Closed-form reverse recurrence (the algorithm of the CUDA backward), block_size=1 is AR.

    With e[t,m] the normalised encoder weight of token t at its own read-out time
    (softmax: exp(s - L_t); stablemax: sigma(s)/D_t), the latent read-out obeys
    z_t = (1 - e_t) z_{t-1} + e_t v_t.  Reverse carries
        b_t = g_t dY_t + (1 - e_{t+1}) b_{t+1}       [M, Dv]
        c_t = g_t p_t  + (1 - e_{t+1}) c_{t+1}       [M],   p[t,m] = <z_t[m], dY_t>
    give dV_t = sum_m e b_t, dS_enc = e * slope * (<b_t, v_t> - c_t), dS_dec = g (p - <g,p>),
    slope = 1 (softmax) or sigma'(s)/sigma(s) (stablemax).  For block_size > 1 the state is
    read at block ends, so carries and weights are per block.
    """
    B, N, H, Dk = K.shape
    M = Q.shape[1]
    Dv = V.shape[-1]
    scale = resolve_scale(scale, Dk)
    Q_dec, K_dec, sep_q, sep_k, shared = resolve_decode_inputs(Q, K, Q_dec, K_dec)
    Qf = Q.to(dtype)
    Kf = K.to(dtype).permute(0, 2, 1, 3)
    Vf = V.to(dtype).permute(0, 2, 1, 3)
    dYf = dY.to(dtype).permute(0, 2, 1, 3)
    Qd = Q_dec.to(dtype).permute(0, 2, 1, 3) if sep_q else Kf
    Kd = K_dec.to(dtype) if sep_k else Qf

    S = scale * torch.einsum("bhnd,hmd->bhnm", Kf, Qf)
    A = S if shared else scale * torch.einsum("bhnd,hmd->bhnm", Qd, Kd)
    G = torch.softmax(A, dim=-1)
    assert N % block_size == 0
    NB = N // block_size

    if variant == "softmax":
        W = torch.exp(S - S.amax(dim=2, keepdim=True))  # unnormalised, common frame per latent
        slope = torch.ones_like(S)
    else:
        W = stablemax_sigma(S, power)
        slope = stablemax_sigma_grad(S, power) / W
    Dcum = torch.cumsum(W, dim=2)  # [B,H,N,M]
    Ucum = torch.cumsum(W[..., None] * Vf[:, :, :, None, :], dim=2)  # [B,H,N,M,Dv]
    blk_end = (torch.arange(N) // block_size + 1) * block_size - 1
    Dread = Dcum[:, :, blk_end]  # denominator at the read-out time of each token's block
    Z = Ucum[:, :, blk_end] / Dread[..., None]  # z seen by token t
    P = torch.einsum("bhtmd,bhtd->bhtm", Z, dYf)
    gp = (G * P).sum(-1, keepdim=True)
    dS_dec = G * (P - gp)

    # reverse carries in the un-normalised frame: bt = sum_{t' in blocks >= blk(t)} G dY / Dread
    GD = G / Dread
    bsum = torch.flip(torch.cumsum(torch.flip(GD[..., None] * dYf[:, :, :, None, :], [2]), 2), [2])
    csum = torch.flip(torch.cumsum(torch.flip(GD * P, [2]), 2), [2])
    blk_start = (torch.arange(N) // block_size) * block_size
    bt = bsum[:, :, blk_start]
    ct = csum[:, :, blk_start]
    dV = torch.einsum("bhtm,bhtmd->bhtd", W, bt)
    dS_enc = W * slope * (torch.einsum("bhtmd,bhtd->bhtm", bt, Vf) - ct)

    out = {}
    dQ = scale * torch.einsum("bhtm,bhtd->hmd", dS_enc, Kf)
    dK = scale * torch.einsum("bhtm,hmd->bhtd", dS_enc, Qf)
    dq_dec = scale * torch.einsum("bhtm,hmd->bhtd", dS_dec, Kd)
    dk_dec = scale * torch.einsum("bhtm,bhtd->hmd", dS_dec, Qd)
    if sep_q:
        out["dQ_dec"] = dq_dec.permute(0, 2, 1, 3).contiguous()
    else:
        dK = dK + dq_dec
    if sep_k:
        out["dK_dec"] = dk_dec
    else:
        dQ = dQ + dk_dec
    out["dQ"] = dQ
    out["dK"] = dK.permute(0, 2, 1, 3).contiguous()
    out["dV"] = dV.permute(0, 2, 1, 3).contiguous()
    return out


# --------------------------------------------------------------------------------------
# error metrics and seeded inputs shared by tests and the benchmark
# --------------------------------------------------------------------------------------
def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double()
    b = b.double()
    return float(torch.linalg.norm(a - b) / (torch.linalg.norm(b) + 1e-12))


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    if a.numel() == 0:
        return 0.0
    return float((a.double() - b.double()).abs().max())


def make_inputs(B, N, H, M, Dk, Dv=None, *, seed0=0, dtype=torch.float32, with_dy=False, batch_offset=0):
    """Seeded synthetic inputs: one CPU generator per batch element so any batch slice is reproducible.

    Q from seed0-1; K[b], V[b] (in that order) from seed0+b; dY[b] from seed0+10000+b.
    Values are drawn in fp32 and rounded to ``dtype``.
    """
    Dv = Dk if Dv is None else Dv
    g = torch.Generator("cpu").manual_seed((seed0 - 1) % (2 ** 31))
    Q = torch.randn(H, M, Dk, generator=g)
    Ks, Vs, dYs = [], [], []
    for b in range(batch_offset, batch_offset + B):
        g = torch.Generator("cpu").manual_seed(seed0 + b)
        Ks.append(torch.randn(N, H, Dk, generator=g))
        Vs.append(torch.randn(N, H, Dv, generator=g))
        if with_dy:
            g2 = torch.Generator("cpu").manual_seed(seed0 + 10_000 + b)
            dYs.append(torch.randn(N, H, Dv, generator=g2))
    K = torch.stack(Ks) if B else torch.empty(0, N, H, Dk)
    V = torch.stack(Vs) if B else torch.empty(0, N, H, Dv)
    out = [Q.to(dtype), K.to(dtype), V.to(dtype)]
    if with_dy:
        out.append(torch.stack(dYs).to(dtype))
    return tuple(out)
