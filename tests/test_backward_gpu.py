"""GPU parity of the backward passes (autograd through the public operators) against the gradients the
reference produces (golden fixtures) and against the CPU oracle's closed form on seeded inputs."""
import pytest
import torch

import causal_flare as cf
from causal_flare.autoregressive import flare_autoregressive_stablemax_triton
from oracle import flare_oracle as orc
from util import assert_bf16_gate, assert_close, to_dev

pytestmark = pytest.mark.gpu

GRAD32 = dict(atol=1e-3, rtol=1e-2)  # fp32 inputs: the reference's own unit-test gate for gradients


def leaves(*ts):
    return [None if t is None else t.detach().clone().requires_grad_(True) for t in ts]


def run_grads(fn, dy, q, k, v, qd=None, kd=None):
    q, k, v, qd, kd = leaves(q, k, v, qd, kd)
    y = fn(q, k, v, qd, kd)
    if isinstance(y, tuple):
        y = y[0]
    y.backward(dy)
    return dict(dq=q.grad, dk=k.grad, dv=v.grad, dq_dec=None if qd is None else qd.grad,
                dk_dec=None if kd is None else kd.grad)


@pytest.mark.parametrize("case", ["ar_sep00", "ar_sep10", "ar_sep01", "ar_sep11"])
def test_ar_grads_decode_separation_modes(golden, case):
    g = golden(case)
    q, k, v, qd, kd, dy = to_dev(g["q"], g["k"], g["v"], g.get("q_dec"), g.get("k_dec"), g["dy"])
    got = run_grads(lambda q, k, v, qd, kd: cf.flare_autoregressive_triton(q, k, v, Q_dec=qd, K_dec=kd), dy, q, k, v, qd, kd)
    for name in ("dq", "dk", "dv", "dq_dec", "dk_dec"):
        if name in g:
            assert got[name].shape == g[name].shape
            assert_close(got[name], g[name], what=f"{case} {name}", **GRAD32)


def test_alias_accumulation_and_determinism(golden):
    g = golden("ar_sep00")
    q, k, v, dy = to_dev(g["q"], g["k"], g["v"], g["dy"])
    a = run_grads(lambda q, k, v, qd, kd: cf.flare_autoregressive_triton(q, k, v), dy, q, k, v)
    # passing the same tensor objects as decode weights is the shared-weight path: grads are folded into dQ / dK
    ql, kl, vl = leaves(q, k, v)
    cf.flare_autoregressive_triton(ql, kl, vl, Q_dec=kl, K_dec=ql).backward(dy)
    assert torch.equal(a["dq"], ql.grad) and torch.equal(a["dk"], kl.grad) and torch.equal(a["dv"], vl.grad)
    b = run_grads(lambda q, k, v, qd, kd: cf.flare_autoregressive_triton(q, k, v), dy, q, k, v)
    for name in ("dq", "dk", "dv"):
        assert torch.equal(a[name], b[name]), f"{name} is not run-to-run deterministic"
    # an equal-valued copy is a separate tensor: its gradient is returned on its own, and the pieces add up
    c = run_grads(lambda q, k, v, qd, kd: cf.flare_autoregressive_triton(q, k, v, Q_dec=qd, K_dec=kd), dy, q, k, v,
                  k.clone(), q.clone())
    assert_close(c["dk"] + c["dq_dec"], a["dk"], what="dk pieces", atol=1e-5, rtol=1e-4)
    assert_close(c["dq"] + c["dk_dec"], a["dq"], what="dq pieces", atol=1e-4, rtol=1e-4)


def test_no_upstream_gradient_returns_none(golden):
    g = golden("ar_sep00")
    q, k, v = leaves(*to_dev(g["q"], g["k"], g["v"]))
    y = cf.flare_autoregressive_triton(q, k, v)
    assert y.requires_grad
    (y.sum() * 0).backward()
    assert float(k.grad.abs().max()) == 0.0


@pytest.mark.parametrize("shape", [(1, 7, 2, 16, 16, 16), (2, 129, 2, 32, 64, 128), (1, 200, 1, 48, 32, 48),
                                   (1, 96, 1, 256, 128, 128), (1, 40, 1, 512, 16, 32),
                                   (1, 1024, 2, 32, 32, 64), (1, 1100, 1, 64, 64, 32)])  # long: sequence segments
def test_ar_grads_fp32_shapes(shape):
    B, N, H, M, Dk, Dv = shape
    q, k, v, dy = orc.make_inputs(B, N, H, M, Dk, Dv, seed0=7, with_dy=True)
    ref = orc.ar_backward_closed_form(q, k, v, dy)
    got = run_grads(lambda q, k, v, qd, kd: cf.flare_autoregressive_triton(q, k, v), *to_dev(dy, q, k, v))
    assert_close(got["dq"], ref["dQ"], what="dq", **GRAD32)
    assert_close(got["dk"], ref["dK"], what="dk", **GRAD32)
    assert_close(got["dv"], ref["dV"], what="dv", **GRAD32)


def test_segmented_backward_separate_decode_weights_and_stablemax():
    # long sequence, few lanes: the replay and reverse walks run as concurrent sequence segments
    B, N, H, M, D = 1, 768, 2, 32, 32
    q, k, v, dy = orc.make_inputs(B, N, H, M, D, seed0=17, with_dy=True)
    g = torch.Generator().manual_seed(5)
    qd, kd = torch.randn(B, N, H, D, generator=g), torch.randn(H, M, D, generator=g)
    ref = orc.ar_backward_closed_form(q, k, v, dy, Q_dec=qd, K_dec=kd)
    got = run_grads(lambda q, k, v, qd, kd: cf.flare_autoregressive_triton(q, k, v, Q_dec=qd, K_dec=kd),
                    *to_dev(dy, q, k, v, qd, kd))
    for name, key in (("dq", "dQ"), ("dk", "dK"), ("dv", "dV"), ("dq_dec", "dQ_dec"), ("dk_dec", "dK_dec")):
        assert_close(got[name], ref[key], what=f"segmented {name}", **GRAD32)
    ref = orc.ar_backward_closed_form(q, k, v, dy, variant="stablemax", power=2.0)
    got = run_grads(lambda q, k, v, qd, kd: flare_autoregressive_stablemax_triton(q, k, v), *to_dev(dy, q, k, v))
    for name, key in (("dq", "dQ"), ("dk", "dK"), ("dv", "dV")):
        assert_close(got[name], ref[key], what=f"segmented stablemax {name}", **GRAD32)


@pytest.mark.parametrize("variant", ["softmax", "stablemax"])
def test_train_step_bf16_gate(variant):
    # reduced C4 (B=4, N=4096, H=16, M=64, D=128): same M and D, fewer lanes and tokens so the oracle runs in seconds
    B, N, H, M, D = 1, 512, 2, 64, 128
    q, k, v, dy = orc.make_inputs(B, N, H, M, D, seed0=0, dtype=torch.bfloat16, with_dy=True)
    if variant == "softmax":
        ref = orc.ar_backward_closed_form(q, k, v, dy)
        fn = lambda q, k, v, qd, kd: cf.flare_autoregressive_triton(q, k, v)  # noqa: E731
    else:
        ref = orc.ar_backward_closed_form(q, k, v, dy, variant="stablemax", power=2.0)
        fn = lambda q, k, v, qd, kd: flare_autoregressive_stablemax_triton(q, k, v)  # noqa: E731
    got = run_grads(fn, *to_dev(dy, q, k, v))
    for name, key in (("dq", "dQ"), ("dk", "dK"), ("dv", "dV")):
        assert got[name].dtype == torch.bfloat16
        assert_bf16_gate(got[name], ref[key], f"{variant} {name}")


@pytest.mark.parametrize("p", [1, 2, 3])
def test_stablemax_grads(golden, p):
    g = golden(f"stablemax_p{p}")
    q, k, v, dy = to_dev(g["q"], g["k"], g["v"], g["dy"])
    got = run_grads(lambda q, k, v, qd, kd: flare_autoregressive_stablemax_triton(q, k, v, power=g["power"]), dy, q, k, v)
    assert_close(got["dq"], g["dq"], what="dq", **GRAD32)
    assert_close(got["dk"], g["dk"], what="dk", **GRAD32)
    assert_close(got["dv"], g["dv"], what="dv", **GRAD32)


def test_stablemax_separate_decode_and_empty():
    q, k, v, dy = orc.make_inputs(1, 50, 2, 32, 32, seed0=3, with_dy=True)
    gq = torch.Generator().manual_seed(1)
    qd, kd = torch.randn(k.shape, generator=gq), torch.randn(q.shape, generator=gq)
    ref = orc.ar_backward_closed_form(q, k, v, dy, Q_dec=qd, K_dec=kd, variant="stablemax", power=2.0)
    got = run_grads(lambda q, k, v, qd, kd: flare_autoregressive_stablemax_triton(q, k, v, Q_dec=qd, K_dec=kd),
                    *to_dev(dy, q, k, v, qd, kd))
    for name, key in (("dq", "dQ"), ("dk", "dK"), ("dv", "dV"), ("dq_dec", "dQ_dec"), ("dk_dec", "dK_dec")):
        assert_close(got[name], ref[key], what=name, **GRAD32)
    ql, kl, vl = leaves(*to_dev(q, k[:, :0], v[:, :0]))
    y = flare_autoregressive_stablemax_triton(ql, kl, vl)
    y.sum().backward()
    assert ql.grad.shape == q.shape and float(ql.grad.abs().sum()) == 0.0 and kl.grad.shape == (1, 0, 2, 32)


@pytest.mark.parametrize("sep", [0, 1])
def test_semi_ar_grads(golden, sep):
    g = golden(f"semi_ar_sep{sep}")
    q, k, v, qd, kd, dy = to_dev(g["q"], g["k"], g["v"], g.get("q_dec"), g.get("k_dec"), g["dy"])
    fn = lambda q, k, v, qd, kd: cf.flare_semi_autoregressive_trition(q, k, v, block_size=32, chunk_size=16, Q_dec=qd, K_dec=kd)  # noqa: E731
    got = run_grads(fn, dy, q, k, v, qd, kd)
    for name in ("dq", "dk", "dv", "dq_dec", "dk_dec"):
        if name in g:
            assert_close(got[name], g[name], what=f"semi-AR {name}", **GRAD32)


def test_semi_ar_grads_bf16_tiled_value_dim():
    q, k, v, dy = orc.make_inputs(1, 256, 1, 256, 128, seed0=11, dtype=torch.bfloat16, with_dy=True)
    ref = orc.ar_backward_closed_form(q, k, v, dy, block_size=64)
    fn = lambda q, k, v, qd, kd: cf.flare_semi_autoregressive_trition(q, k, v, block_size=64, chunk_size=64)  # noqa: E731
    got = run_grads(fn, *to_dev(dy, q, k, v))
    for name, key in (("dq", "dQ"), ("dk", "dK"), ("dv", "dV")):
        assert_bf16_gate(got[name], ref[key], f"semi-AR bf16 {name}")


@pytest.mark.parametrize("N, bs", [(1024, 32), (1152, 48), (2048, 128)])
def test_semi_ar_grads_long_sequence_segments(N, bs):
    # few lanes, long sequence: the block-causal backward runs as concurrent sequence segments of whole blocks
    B, H, M, D = 1, 2, 32, 32
    q, k, v, dy = orc.make_inputs(B, N, H, M, D, seed0=23, with_dy=True)
    ref = orc.ar_backward_closed_form(q, k, v, dy, block_size=bs)
    got = run_grads(lambda q, k, v, qd, kd: cf.flare_semi_autoregressive_trition(q, k, v, block_size=bs, chunk_size=16),
                    *to_dev(dy, q, k, v))
    for name, key in (("dq", "dQ"), ("dk", "dK"), ("dv", "dV")):
        assert_close(got[name], ref[key], what=f"segmented semi-AR {name}", **GRAD32)


def test_recurrent_grads(golden):
    g = golden("recurrent")
    q, k, v = g["q"], g["k"], g["v"]
    dy = torch.randn(g["y_bhnd"].shape, generator=torch.Generator().manual_seed(2))
    ref = orc.ar_backward_closed_form(q, k, v, dy.permute(0, 2, 1, 3))
    got = run_grads(lambda q, k, v, qd, kd: cf.flare_recurrent_triton(q, k, v), *to_dev(dy, q, k, v))
    assert_close(got["dq"], ref["dQ"], what="dq", **GRAD32)
    assert_close(got["dk"], ref["dK"], what="dk", **GRAD32)
    assert_close(got["dv"], ref["dV"], what="dv", **GRAD32)


def test_profile_backward_timings_filled_in_place(golden):
    g = golden("ar_sep00")
    q, k, v = leaves(*to_dev(g["q"], g["k"], g["v"]))
    y, prof = cf.flare_autoregressive_triton(q, k, v, profile=True)
    assert prof["backward"] == {}
    y.backward(g["dy"].cuda())
    assert prof["backward_total_ms"] > 0 and prof["total_ms"] >= prof["forward_total_ms"]


@pytest.mark.parametrize("block_size, dtype", [(1, torch.float32), (32, torch.float32), (1, torch.bfloat16)])
def test_span_backward_four_spans_on_one_gpu(block_size, dtype):
    # the sequence-parallel backward with the ranks emulated in one process: every span is replayed from its prefix
    # state, the span summaries are combined right to left, every span is finished with its carry; the pieces must
    # equal the gradients of the whole sequence
    from causal_flare import _ops, parallel

    B, N, H, M, D, spans = 1, 1280, 2, 32, 64, 4
    q, k, v, dy = orc.make_inputs(B, N, H, M, D, seed0=29, dtype=dtype, with_dy=True)
    qc, kc, vc, dyc = to_dev(q, k, v, dy)
    sc = D ** -0.5
    span = N // spans
    state, ctxs = None, []
    for r in range(spans):
        sl = slice(r * span, (r + 1) * span)
        ctxs.append(_ops.backward_span_begin(qc, kc[:, sl], vc[:, sl], dyc[:, sl], scale=sc, state_in=state,
                                             block_size=block_size))
        _, state, _, _ = _ops.forward(qc, kc[:, sl], vc[:, sl], scale=sc, state_in=state, want_state=True, want_y=False)
    stacked = {key: torch.stack([c["summary"][key] for c in ctxs]) for key in ("b0", "c0", "gam", "rho_first")}
    dq = torch.zeros(H, M, D, device="cuda")
    dks, dvs = [], []
    for r in range(spans):
        dq_r, dk_r, dv_r = _ops.backward_span_finish(ctxs[r], parallel.right_carry(stacked, r))
        dq += dq_r
        dks.append(dk_r)
        dvs.append(dv_r)
    dq_f, dk_f, dv_f, _, _ = _ops.backward(qc, kc, vc, dyc, scale=sc, block_size=block_size)
    tol = dict(atol=2e-3, rtol=2e-2) if dtype == torch.float32 else dict(atol=5e-2, rtol=5e-2)
    assert_close(dq, dq_f, what="span dq", **tol)
    assert_close(torch.cat(dks, 1), dk_f, what="span dk", **tol)
    assert_close(torch.cat(dvs, 1), dv_f, what="span dv", **tol)
    if dtype == torch.float32:
        ref = orc.ar_backward_closed_form(q, k, v, dy, scale=sc, block_size=block_size)
        assert_close(torch.cat(dks, 1), ref["dK"], what="span dk vs oracle", **GRAD32)
        assert_close(torch.cat(dvs, 1), ref["dV"], what="span dv vs oracle", **GRAD32)
        assert_close(dq, ref["dQ"], what="span dq vs oracle", **GRAD32)
