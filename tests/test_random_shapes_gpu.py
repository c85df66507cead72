"""Seeded random sweep of shapes and modes on the GPU: the tensor-core kernels against the exact kernels (same inputs,
both through the C ABI), forward with carried states, both output layouts and the launch variants of the (128, 128)
head shape, and backward with and without the states kept by the forward.  The exact kernels are themselves held to
the oracle elsewhere; this sweep is for what fixed shape lists miss (it found a race between two roles of the prefill
kernel that only showed in single lanes with more than 128 latents)."""
import random

import pytest
import torch

from causal_flare import _lib, _ops

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6))


@pytest.mark.parametrize("seed", [11, 12])
def test_forward_random_shapes_tensor_vs_exact(seed, monkeypatch):
    rng = random.Random(seed)
    ran = 0
    for it in range(60):
        Dk, Dv = rng.choice([(64, 64), (128, 128), (64, 128), (128, 128)])
        M = rng.choice([16, 48, 64, 96, 128, 128, 192, 256, 256, 384, 512])
        bs = rng.choice([1, 1, 1, 16, 32, 64, 128])
        stable = bs == 1 and rng.random() < 0.3
        B, H = rng.choice([1, 2, 3]), rng.choice([1, 2, 5])
        N = rng.choice([1, 7, 64, 128, 200, 257, 640, 1000, 1536, 2500])
        if bs > 1:
            N = max(bs, N // bs * bs)
        monkeypatch.setenv("FLARE_B200_WIDE", rng.choice(["0", "1"]))
        monkeypatch.setenv("FLARE_B200_CLUSTER", rng.choice(["0", "1"]))
        monkeypatch.setenv("FLARE_B200_ROW_STORES", rng.choice(["0", "0", "1"]))
        g = torch.Generator(device="cuda").manual_seed(1000 * seed + it)
        q = torch.randn(H, M, Dk, generator=g, device="cuda").bfloat16()
        k = torch.randn(B, N, H, Dk, generator=g, device="cuda").bfloat16()
        v = torch.randn(B, N, H, Dv, generator=g, device="cuda").bfloat16()
        kw = dict(scale=Dk ** -0.5, block_size=bs, variant=_lib.STABLEMAX if stable else _lib.SOFTMAX,
                  power=rng.choice([1.0, 2.0, 3.0]))
        unit = max(bs, 16)
        st_in = None
        if rng.random() < 0.4 and N >= 2 * unit:
            cut = (N // 2) // unit * unit
            st_in = _ops.forward(q, k[:, :cut], v[:, :cut], path=_lib.PATH_EXACT, want_state=True, **kw)[1]
            k, v = k[:, cut:], v[:, cut:]
        bhnd = rng.random() < 0.3
        ye, se, _, _ = _ops.forward(q, k, v, path=_lib.PATH_EXACT, state_in=st_in, want_state=True, **kw)
        yt, st, _, _ = _ops.forward(q, k, v, path=_lib.PATH_TENSOR, state_in=st_in, want_state=True, out_bhnd=bhnd, **kw)
        assert _ops.device_status() == 0
        if bhnd:
            yt = yt.permute(0, 2, 1, 3)  # stored [B, H, N, Dv]
        ran += 1
        what = f"case {it}: B={B} N={k.shape[1]} H={H} M={M} D=({Dk},{Dv}) block={bs} stablemax={stable} carry={st_in is not None}"
        assert torch.isfinite(yt.float()).all(), what
        # both outputs are bf16 roundings of the same values: twice the gate of one of them against the oracle
        assert _rel(yt, ye) <= 6e-3, what
        lane = ((yt.float() - ye.float()).pow(2).sum(dim=(1, 3)) / ye.float().pow(2).sum(dim=(1, 3)).clamp_min(1e-12)).sqrt()
        assert float(lane.max()) <= 8e-3, what + f" (worst lane {float(lane.max()):.2e})"
        assert _rel(st["u"], se["u"]) <= 5e-3, what
        assert float(((st["d"] - se["d"]).abs() / se["d"].abs().clamp_min(1e-6)).max()) <= 5e-3, what
        assert float((st["m"] - se["m"]).abs().max()) <= 1e-3, what
    assert ran == 60


def test_backward_random_shapes_tensor_vs_exact(monkeypatch):
    rng = random.Random(21)
    for it in range(40):
        Dk, Dv = rng.choice([(64, 64), (128, 128), (64, 128)])
        M = rng.choice([16, 64, 96, 128, 192, 256, 512])
        bs = rng.choice([1, 1, 16, 32, 64, 128])
        stable = bs == 1 and rng.random() < 0.5
        B, H = rng.choice([1, 2]), rng.choice([1, 2, 3])
        N = rng.choice([64, 128, 200, 640, 1000, 1536])
        if bs > 1:
            N = max(bs, N // bs * bs)
        monkeypatch.setenv("FLARE_B200_WIDE", rng.choice(["0", "1"]))
        monkeypatch.setenv("FLARE_B200_CLUSTER", rng.choice(["0", "1"]))
        g = torch.Generator(device="cuda").manual_seed(5000 + it)
        q = torch.randn(H, M, Dk, generator=g, device="cuda").bfloat16()
        k = torch.randn(B, N, H, Dk, generator=g, device="cuda").bfloat16()
        v = torch.randn(B, N, H, Dv, generator=g, device="cuda").bfloat16()
        dy = torch.randn(B, N, H, Dv, generator=g, device="cuda").bfloat16()
        kw = dict(scale=Dk ** -0.5, block_size=bs, variant=_lib.STABLEMAX if stable else _lib.SOFTMAX,
                  power=rng.choice([1.0, 2.0, 3.0]))
        kept = {}
        if rng.random() < 0.5:
            _ops.forward(q, k, v, keep_for_backward=kept, **kw)
        a = _ops.backward(q, k, v, dy, path=_lib.PATH_TENSOR, saved=kept or None, **kw)[:3]
        b = _ops.backward(q, k, v, dy, path=_lib.PATH_EXACT, **kw)[:3]
        assert _ops.device_status() == 0
        what = f"case {it}: B={B} N={N} H={H} M={M} D=({Dk},{Dv}) block={bs} stablemax={stable} kept={bool(kept)}"
        for name, x, y in zip(("dQ", "dK", "dV"), a, b):
            assert torch.isfinite(x.float()).all(), what
            assert _rel(x, y) <= 8e-3, f"{what}: {name} {_rel(x, y):.2e}"
