"""Generate the golden fixtures in this directory from the REFERENCE implementation.

Run once, in a container that has the reference checkout:

    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

For every case it (1) runs the reference project's own PyTorch functions on seeded
inputs, (2) checks the CPU oracle (``oracle/flare_oracle.py``) against them, and
(3) stores inputs and reference outputs as ``<case>.npz`` (fp32) so that the
fixtures travel to machines that do not have the reference checkout.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import flare_oracle as orc  # noqa: E402

from causal_flare.autoregressive.reference import flare_causal_chunked, flare_causal_reference  # noqa: E402
from causal_flare.autoregressive.inference import flare_decode_pytorch, flare_prefill_pytorch  # noqa: E402
from causal_flare.autoregressive.recurrent import flare_recurrent_pytorch  # noqa: E402
from causal_flare.autoregressive.stablemax import flare_autoregressive_stablemax_pytorch  # noqa: E402
from causal_flare.semi_autoregressive.reference import (  # noqa: E402
    _block_causal_backward_pytorch,
    _block_causal_forward_pytorch,
    semi_autoregressive_flare_reference,
)


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu()
            v = v.numpy() if v.dtype != torch.bfloat16 else v.float().numpy()
        out[k] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(f"wrote {name}.npz ({sum(a.nbytes for a in out.values()) / 1e3:.0f} kB raw)")


def check(tag, ours, ref, atol=2e-5, rtol=1e-4):
    ours = ours.float()
    ref = ref.float()
    err = (ours - ref).abs().max().item() if ref.numel() else 0.0
    ok = torch.allclose(ours, ref, atol=atol, rtol=rtol)
    print(f"  oracle vs reference [{tag}]: max-abs {err:.3e} {'OK' if ok else 'MISMATCH'}")
    assert ok, tag


def randn_case(seed, B, N, H, M, Dk, Dv=None):
    Dv = Dk if Dv is None else Dv
    torch.manual_seed(seed)
    q = torch.randn(H, M, Dk)
    k = torch.randn(B, N, H, Dk)
    v = torch.randn(B, N, H, Dv)
    return q, k, v


def main():
    torch.set_num_threads(8)

    # ---- C1: the README recipe, B=1, N=256, H=8, M=64, D=32, fp32, seed 0 -----------------
    q, k, v = randn_case(0, 1, 256, 8, 64, 32)
    y_ref = flare_causal_reference(q, k, v)
    y_chk = flare_causal_chunked(q, k, v)
    y_orc = orc.ar_forward(q, k, v)
    print(f"C1 checksum y.double().sum() = {y_ref.double().sum().item():.6f}")
    check("C1 definitional", y_orc, y_ref)
    check("C1 chunked", y_orc, y_chk)
    check("C1 chunked port", orc.ar_forward_chunked(q, k, v, chunk_size=64), flare_causal_chunked(q, k, v, chunk_size=64), atol=0, rtol=0)
    save("ar_c1", q=q, k=k, v=v, y=y_ref, checksum=np.float64(y_ref.double().sum().item()))

    # ---- small AR forward+grad cases, the four decode-separation modes ---------------------
    for sep_q, sep_k in ((0, 0), (1, 0), (0, 1), (1, 1)):
        q, k, v = randn_case(1, 2, 37, 3, 16, 16, 32)
        torch.manual_seed(11)
        q_dec = torch.randn_like(k) if sep_q else None
        k_dec = torch.randn_like(q) if sep_k else None
        dy = torch.randn(2, 37, 3, 32)
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
        qd = q_dec.clone().requires_grad_(True) if sep_q else None
        kd = k_dec.clone().requires_grad_(True) if sep_k else None
        y = flare_causal_chunked(*leaves, Q_dec=qd, K_dec=kd, chunk_size=16)
        y_def = flare_causal_reference(q, k, v, Q_dec=q_dec, K_dec=k_dec)
        ins = leaves + [t for t in (qd, kd) if t is not None]
        grads = torch.autograd.grad(y, ins, dy)
        dq, dk, dv = grads[:3]
        rest = list(grads[3:])
        dqd = rest.pop(0) if sep_q else None
        dkd = rest.pop(0) if sep_k else None
        tag = f"ar_sep{sep_q}{sep_k}"
        check(tag + " y", orc.ar_forward(q, k, v, Q_dec=q_dec, K_dec=k_dec), y_def)
        check(tag + " y chunked", orc.ar_forward(q, k, v, Q_dec=q_dec, K_dec=k_dec), y)
        cf = orc.ar_backward_closed_form(q, k, v, dy, Q_dec=q_dec, K_dec=k_dec)
        check(tag + " dq", cf["dQ"], dq, atol=2e-4, rtol=1e-3)
        check(tag + " dk", cf["dK"], dk, atol=2e-4, rtol=1e-3)
        check(tag + " dv", cf["dV"], dv, atol=2e-4, rtol=1e-3)
        if sep_q:
            check(tag + " dq_dec", cf["dQ_dec"], dqd, atol=2e-4, rtol=1e-3)
        if sep_k:
            check(tag + " dk_dec", cf["dK_dec"], dkd, atol=2e-4, rtol=1e-3)
        ag = orc.grads_autograd(
            lambda Q, K, V, Q_dec=None, K_dec=None: orc.ar_forward(Q, K, V, Q_dec=Q_dec, K_dec=K_dec),
            {"Q": q, "K": k, "V": v, "Q_dec": q_dec, "K_dec": k_dec}, dy)
        check(tag + " autograd dq", ag["dQ"], dq, atol=2e-4, rtol=1e-3)
        arrays = dict(q=q, k=k, v=v, dy=dy, y=y_def, dq=dq, dk=dk, dv=dv)
        if sep_q:
            arrays.update(q_dec=q_dec, dq_dec=dqd)
        if sep_k:
            arrays.update(k_dec=k_dec, dk_dec=dkd)
        save(tag, **arrays)

    # ---- recurrent (output layout [B,H,N,D]) --------------------------------------------------
    q, k, v = randn_case(2, 1, 16, 2, 16, 16)
    y_rec = flare_recurrent_pytorch(q, k, v)
    check("recurrent", orc.ar_forward(q, k, v).permute(0, 2, 1, 3), y_rec)
    save("recurrent", q=q, k=k, v=v, y_bhnd=y_rec)

    # ---- cached inference: masked prefill, decode, continuation (shapes of the reference's
    #      cached regression suite: B=2,H=4,M=32,T=17,D=32, scale=D^-0.5, mask prob 0.2) ------
    torch.manual_seed(0)
    B, H, M, T, D = 2, 4, 32, 17, 32
    scale = D ** -0.5
    q = torch.randn(H, M, D)
    k = torch.randn(B, T, H, D)
    v = torch.randn(B, T, H, D)
    mask = (torch.rand(B, T) > 0.2).to(torch.int32)
    mask[1, 0] = 0  # a lane whose first token is masked: exercises the -inf state algebra
    k2 = torch.randn(B, 1, H, D)
    v2 = torch.randn(B, 1, H, D)
    mask2 = torch.tensor([1, 0], dtype=torch.int32).view(B, 1)
    y1, s1 = flare_prefill_pytorch(q, k, v, scale=scale, attention_mask=mask)
    y2, s2 = flare_decode_pytorch(q, k2, v2, s1, scale=scale, attention_mask=mask2)
    yo, so = orc.ar_forward(q, k, v, scale=scale, attention_mask=mask, return_state=True)
    check("prefill masked y", yo, y1)
    for key in "mdu":
        fin = torch.isfinite(s1[key])
        check("prefill masked state " + key, torch.where(fin, so[key].float(), torch.zeros(())),
              torch.where(fin, s1[key], torch.zeros(())))
    yo2, so2 = orc.decode_step(q, k2[:, 0], v2[:, 0], so, scale=scale, attention_mask=mask2)
    check("decode masked y", yo2, y2)
    y1u, s1u = flare_prefill_pytorch(q, k, v, scale=scale)
    y2u, s2u = flare_decode_pytorch(q, k2, v2, s1u, scale=scale)
    yo_u, so_u = orc.ar_forward(q, k, v, scale=scale, return_state=True)
    check("prefill y", yo_u, y1u)
    check("prefill u", so_u["u"], s1u["u"])
    yo2u, so2u = orc.decode_step(q, k2[:, 0], v2[:, 0], so_u, scale=scale)
    check("decode y", yo2u, y2u)
    check("decode u", so2u["u"], s2u["u"])
    save("cached", q=q, k=k, v=v, mask=mask, k2=k2, v2=v2, mask2=mask2, scale=np.float64(scale),
         y1=y1, m1=s1["m"], d1=s1["d"], u1=s1["u"], y2=y2, m2=s2["m"], d2=s2["d"], u2=s2["u"],
         y1u=y1u, m1u=s1u["m"], d1u=s1u["d"], u1u=s1u["u"], y2u=y2u, m2u=s2u["m"], d2u=s2u["d"], u2u=s2u["u"])

    # ---- stablemax forward + grads, powers 1, 2, 3 ---------------------------------------------
    for power in (1.0, 2.0, 3.0):
        q, k, v = randn_case(3, 2, 40, 2, 32, 32)
        torch.manual_seed(13)
        dy = torch.randn_like(v)
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
        y = flare_autoregressive_stablemax_pytorch(*leaves, power=power, chunk_size=16)
        dq, dk, dv = torch.autograd.grad(y, leaves, dy)
        tag = f"stablemax_p{int(power)}"
        check(tag + " y", orc.ar_forward(q, k, v, variant="stablemax", power=power), y)
        cf = orc.ar_backward_closed_form(q, k, v, dy, variant="stablemax", power=power)
        check(tag + " dq", cf["dQ"], dq, atol=2e-4, rtol=1e-3)
        check(tag + " dk", cf["dK"], dk, atol=2e-4, rtol=1e-3)
        check(tag + " dv", cf["dV"], dv, atol=2e-4, rtol=1e-3)
        save(tag, q=q, k=k, v=v, dy=dy, y=y, dq=dq, dk=dk, dv=dv, power=np.float64(power))

    # ---- semi-autoregressive forward (+aux) and hand-written backward ---------------------------
    for sep in (0, 1):
        q, k, v = randn_case(4, 2, 96, 2, 16, 16, 32)
        torch.manual_seed(17)
        q_dec = torch.randn_like(k) if sep else None
        k_dec = torch.randn_like(q) if sep else None
        dy = torch.randn_like(v)
        y, aux = _block_causal_forward_pytorch(q, k, v, block_size=32, chunk_size=16, Q_dec=q_dec, K_dec=k_dec,
                                               return_aux=True)
        y_sdpa = semi_autoregressive_flare_reference(q, k, v, block_size=32, Q_dec=q_dec, K_dec=k_dec)
        dq, dk, dv, dqd, dkd = _block_causal_backward_pytorch(q, k, v, dy, block_size=32, chunk_size=16,
                                                              Q_dec=q_dec, K_dec=k_dec)
        tag = f"semi_ar_sep{sep}"
        yo, lse_dec, lse_enc = orc.semi_ar_forward(q, k, v, block_size=32, Q_dec=q_dec, K_dec=k_dec)
        check(tag + " y", yo, y)
        check(tag + " y sdpa", yo, y_sdpa)
        check(tag + " lse_dec", lse_dec, aux["LSE_dec"])
        check(tag + " lse_enc", lse_enc, aux["LSE_enc"])
        cf = orc.ar_backward_closed_form(q, k, v, dy, Q_dec=q_dec, K_dec=k_dec, block_size=32)
        check(tag + " dq", cf["dQ"], dq, atol=2e-4, rtol=1e-3)
        check(tag + " dk", cf["dK"], dk, atol=2e-4, rtol=1e-3)
        check(tag + " dv", cf["dV"], dv, atol=2e-4, rtol=1e-3)
        arrays = dict(q=q, k=k, v=v, dy=dy, y=y, lse_dec=aux["LSE_dec"], lse_enc=aux["LSE_enc"], dq=dq, dk=dk, dv=dv)
        if sep:
            check(tag + " dq_dec", cf["dQ_dec"], dqd, atol=2e-4, rtol=1e-3)
            check(tag + " dk_dec", cf["dK_dec"], dkd, atol=2e-4, rtol=1e-3)
            arrays.update(q_dec=q_dec, k_dec=k_dec, dq_dec=dqd, dk_dec=dkd)
        save(tag, **arrays)

    print("all oracle-vs-reference checks passed")


if __name__ == "__main__":
    main()
