"""Shared helpers for the parity tests."""
import torch

from oracle import flare_oracle as orc


def to_dev(*ts, dtype=None):
    out = []
    for t in ts:
        if t is None:
            out.append(None)
        else:
            t = t.cuda()
            out.append(t.to(dtype) if dtype is not None and t.is_floating_point() else t)
    return out


def assert_close(a, b, atol, rtol, what=""):
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())}/{a.numel()} elements out of tolerance; max-abs {float(err.max()):.3e}, "
        f"rel-L2 {orc.rel_l2(a, b):.3e}"
    )


def assert_bf16_gate(a, b, what="", max_abs=2e-2, rel_l2=5e-3):
    """The bf16-input gate: max-abs <= 2e-2 and rel-L2 <= 5e-3 against the fp32 oracle."""
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    assert torch.isfinite(a).all(), f"{what}: non-finite output"
    ma, rl = orc.max_abs(a, b), orc.rel_l2(a, b)
    assert ma <= max_abs and rl <= rel_l2, f"{what}: max-abs {ma:.3e} (<= {max_abs}), rel-L2 {rl:.3e} (<= {rel_l2})"
