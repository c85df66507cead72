"""CPU: the oracle reproduces every golden fixture generated from the reference implementation."""
import pytest
import torch

from oracle import flare_oracle as orc
from util import assert_close

FWD = dict(atol=2e-5, rtol=1e-4)
GRAD = dict(atol=2e-4, rtol=1e-3)


def test_c1_readme_case(golden):
    g = golden("ar_c1")
    y = orc.ar_forward(g["q"], g["k"], g["v"])
    assert_close(y, g["y"], what="C1 y", **FWD)
    assert abs(float(y.double().sum()) - g["checksum"]) < 1e-3


@pytest.mark.parametrize("chunk", [16, 64, 100])
def test_chunked_port_matches_fixture_and_token_oracle(golden, chunk):
    # the three-phase chunked formulation (what the CPU baseline of the benchmark times) against the reference's output
    g = golden("ar_c1")
    y = orc.ar_forward_chunked(g["q"], g["k"], g["v"], chunk_size=chunk)
    assert_close(y, g["y"], what="C1 y (chunked port)", **FWD)
    q, k, v = orc.make_inputs(2, 77, 2, 16, 16, 32, seed0=3)
    assert_close(orc.ar_forward_chunked(q, k, v, chunk_size=chunk), orc.ar_forward(q, k, v), what="ragged length", **FWD)


@pytest.mark.parametrize("case", ["ar_sep00", "ar_sep10", "ar_sep01", "ar_sep11"])
def test_ar_forward_and_grads(golden, case):
    g = golden(case)
    qd, kd = g.get("q_dec"), g.get("k_dec")
    y = orc.ar_forward(g["q"], g["k"], g["v"], Q_dec=qd, K_dec=kd)
    assert_close(y, g["y"], what="y", **FWD)
    cf = orc.ar_backward_closed_form(g["q"], g["k"], g["v"], g["dy"], Q_dec=qd, K_dec=kd)
    for name in ("dq", "dk", "dv", "dq_dec", "dk_dec"):
        if name in g:
            key = "d" + name[1:].upper()[0] + name[2:] if "_" in name else "d" + name[1:].upper()
            key = {"dq": "dQ", "dk": "dK", "dv": "dV", "dq_dec": "dQ_dec", "dk_dec": "dK_dec"}[name]
            assert_close(cf[key], g[name], what=name, **GRAD)
    ag = orc.grads_autograd(
        lambda Q, K, V, Q_dec=None, K_dec=None: orc.ar_forward(Q, K, V, Q_dec=Q_dec, K_dec=K_dec),
        {"Q": g["q"], "K": g["k"], "V": g["v"], "Q_dec": qd, "K_dec": kd}, g["dy"])
    assert_close(ag["dQ"], g["dq"], what="autograd dq", **GRAD)
    assert_close(ag["dK"], g["dk"], what="autograd dk", **GRAD)


def test_recurrent_layout(golden):
    g = golden("recurrent")
    y = orc.ar_forward(g["q"], g["k"], g["v"]).permute(0, 2, 1, 3)
    assert_close(y, g["y_bhnd"], what="recurrent y", **FWD)


def test_cached_prefill_decode(golden):
    g = golden("cached")
    y1, s1 = orc.ar_forward(g["q"], g["k"], g["v"], scale=g["scale"], attention_mask=g["mask"], return_state=True)
    assert_close(y1, g["y1"], what="masked prefill y", **FWD)
    fin = torch.isfinite(g["m1"])
    assert bool((torch.isfinite(s1["m"]) == fin).all())
    assert_close(torch.where(fin, s1["m"].float(), torch.zeros(())), torch.where(fin, g["m1"], torch.zeros(())), what="m", **FWD)
    assert_close(s1["u"], g["u1"], what="u", **FWD)
    y2, s2 = orc.decode_step(g["q"], g["k2"][:, 0], g["v2"][:, 0], s1, scale=g["scale"], attention_mask=g["mask2"])
    assert_close(y2, g["y2"], what="masked decode y", **FWD)
    assert_close(s2["u"], g["u2"], what="u2", **FWD)
    y1u, s1u = orc.ar_forward(g["q"], g["k"], g["v"], scale=g["scale"], return_state=True)
    assert_close(y1u, g["y1u"], what="prefill y", **FWD)
    y2u, s2u = orc.decode_step(g["q"], g["k2"][:, 0], g["v2"][:, 0], s1u, scale=g["scale"])
    assert_close(y2u, g["y2u"], what="decode y", **FWD)
    assert_close(s2u["d"], g["d2u"], what="d2u", **FWD)
    # continuation consistency: decode after prefill == last row of a longer prefill
    yfull = orc.ar_forward(g["q"], torch.cat([g["k"], g["k2"]], 1), torch.cat([g["v"], g["v2"]], 1), scale=g["scale"])
    assert_close(y2u, yfull[:, -1:], what="continuation", **FWD)


def test_merge_is_associative_and_matches_sequential(golden):
    g = golden("cached")
    q, k, v, sc = g["q"], g["k"], g["v"], g["scale"]
    _, s_all = orc.ar_forward(q, k, v, scale=sc, return_state=True)
    _, s_a = orc.ar_forward(q, k[:, :5], v[:, :5], scale=sc, return_state=True)
    _, s_b = orc.ar_forward(q, k[:, 5:11], v[:, 5:11], scale=sc, return_state=True)
    _, s_c = orc.ar_forward(q, k[:, 11:], v[:, 11:], scale=sc, return_state=True)
    left = orc.merge_states(orc.merge_states(s_a, s_b), s_c)
    right = orc.merge_states(s_a, orc.merge_states(s_b, s_c))
    for s in (left, right):
        z = s["u"] / s["d"][..., None]
        z_ref = s_all["u"] / s_all["d"][..., None]
        assert_close(z, z_ref, what="merged z", atol=1e-9, rtol=1e-7)
    empty = orc.init_state(*s_a["u"].shape, dtype=torch.float64)
    e = orc.merge_states(empty, s_a)
    assert_close(e["u"], s_a["u"], what="empty merge", atol=0, rtol=0)
    ee = orc.merge_states(empty, empty)
    assert bool(torch.isinf(ee["m"]).all()) and float(ee["d"].abs().sum()) == 0.0


@pytest.mark.parametrize("p", [1, 2, 3])
def test_stablemax(golden, p):
    g = golden(f"stablemax_p{p}")
    y = orc.ar_forward(g["q"], g["k"], g["v"], variant="stablemax", power=g["power"])
    assert_close(y, g["y"], what="y", **FWD)
    cf = orc.ar_backward_closed_form(g["q"], g["k"], g["v"], g["dy"], variant="stablemax", power=g["power"])
    assert_close(cf["dQ"], g["dq"], what="dq", **GRAD)
    assert_close(cf["dK"], g["dk"], what="dk", **GRAD)
    assert_close(cf["dV"], g["dv"], what="dv", **GRAD)


@pytest.mark.parametrize("sep", [0, 1])
def test_semi_ar(golden, sep):
    g = golden(f"semi_ar_sep{sep}")
    qd, kd = g.get("q_dec"), g.get("k_dec")
    y, lse_dec, lse_enc = orc.semi_ar_forward(g["q"], g["k"], g["v"], block_size=32, Q_dec=qd, K_dec=kd)
    assert_close(y, g["y"], what="y", **FWD)
    assert_close(lse_dec, g["lse_dec"], what="lse_dec", **FWD)
    assert_close(lse_enc, g["lse_enc"], what="lse_enc", **FWD)
    cf = orc.ar_backward_closed_form(g["q"], g["k"], g["v"], g["dy"], Q_dec=qd, K_dec=kd, block_size=32)
    assert_close(cf["dQ"], g["dq"], what="dq", **GRAD)
    assert_close(cf["dK"], g["dk"], what="dk", **GRAD)
    assert_close(cf["dV"], g["dv"], what="dv", **GRAD)
    if sep:
        assert_close(cf["dQ_dec"], g["dq_dec"], what="dq_dec", **GRAD)
        assert_close(cf["dK_dec"], g["dk_dec"], what="dk_dec", **GRAD)


def test_block_size_one_equals_autoregressive():
    q, k, v = orc.make_inputs(1, 32, 2, 16, 16)
    y_ar = orc.ar_forward(q, k, v)
    y_b16, _, _ = orc.semi_ar_forward(q, k, v, block_size=16)
    # the last token of every block sees exactly its causal prefix
    assert_close(y_b16[:, 15::16], y_ar[:, 15::16], what="block end", atol=1e-10, rtol=1e-8)
