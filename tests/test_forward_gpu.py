"""GPU parity of the forward operators, through the public API (and so through the C ABI), against the
golden fixtures from the reference and against the CPU oracle on seeded inputs."""
import pytest
import torch

import causal_flare as cf
from causal_flare.autoregressive import flare_autoregressive_stablemax_triton
from oracle import flare_oracle as orc
from util import assert_bf16_gate, assert_close, to_dev

pytestmark = pytest.mark.gpu

FWD32 = dict(atol=1e-5, rtol=1e-4)   # fp32 inputs: the reference's own unit-test gate
ST32 = dict(atol=2e-5, rtol=2e-4)


def test_c1_readme_case(golden):
    g = golden("ar_c1")
    q, k, v = to_dev(g["q"], g["k"], g["v"])
    y = cf.flare_autoregressive_triton(q, k, v)
    assert y.dtype == torch.float32 and y.shape == g["y"].shape
    assert_close(y, g["y"], what="C1", **FWD32)
    assert abs(float(y.double().sum()) - g["checksum"]) < 2e-3
    yb = cf.flare_autoregressive_triton(q.bfloat16(), k.bfloat16(), v.bfloat16())
    assert yb.dtype == torch.bfloat16
    ref = orc.ar_forward(g["q"].bfloat16(), g["k"].bfloat16(), g["v"].bfloat16())
    assert_bf16_gate(yb, ref, "C1 bf16")


@pytest.mark.parametrize("case", ["ar_sep00", "ar_sep10", "ar_sep01", "ar_sep11"])
def test_ar_forward_decode_separation_modes(golden, case):
    g = golden(case)
    q, k, v, qd, kd = to_dev(g["q"], g["k"], g["v"], g.get("q_dec"), g.get("k_dec"))
    y = cf.flare_autoregressive_triton(q, k, v, Q_dec=qd, K_dec=kd)
    assert_close(y, g["y"], what=case, **FWD32)


def test_alias_by_identity_is_bit_identical(golden):
    g = golden("ar_sep00")
    q, k, v = to_dev(g["q"], g["k"], g["v"])
    y0 = cf.flare_autoregressive_triton(q, k, v)
    y1 = cf.flare_autoregressive_triton(q, k, v, Q_dec=k, K_dec=q)
    assert torch.equal(y0, y1)
    y2 = cf.flare_autoregressive_triton(q, k, v)
    assert torch.equal(y0, y2), "forward must be run-to-run deterministic"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 7, 2, 16, 16, 16), (2, 129, 2, 32, 64, 128), (1, 300, 1, 48, 32, 48),
                                   (1, 64, 2, 128, 64, 64), (1, 40, 1, 256, 128, 128), (1, 33, 1, 512, 16, 32)])
def test_ar_forward_shapes_and_dtypes(shape, dtype):
    B, N, H, M, Dk, Dv = shape
    q, k, v = orc.make_inputs(B, N, H, M, Dk, Dv, seed0=5, dtype=dtype)
    ref = orc.ar_forward(q, k, v)
    y = cf.flare_autoregressive_triton(*to_dev(q, k, v))
    assert y.dtype == dtype and tuple(y.shape) == (B, N, H, Dv)
    if dtype == torch.float32:
        assert_close(y, ref, what=str(shape), **FWD32)
    else:
        assert_bf16_gate(y, ref, str(shape))


def test_segmented_walk_matches_single_segment():
    # few lanes and a long sequence: the library splits N into segments with a state scan in between
    q, k, v = orc.make_inputs(1, 2048, 1, 32, 32, seed0=9)
    ref = orc.ar_forward(q, k, v)
    y = cf.flare_autoregressive_triton(*to_dev(q, k, v))
    assert_close(y, ref, what="segmented", **FWD32)
    st0 = {kk: vv.float() for kk, vv in orc.ar_forward(q, k[:, :100], v[:, :100], scale=0.2, return_state=True)[1].items()}
    y2, st2 = cf.flare_autoregressive_prefill_triton(*to_dev(q, k[:, 100:], v[:, 100:]), scale=0.2,
                                                     state={a: b.cuda() for a, b in st0.items()})
    ref2, st_ref = orc.ar_forward(q, k, v, scale=0.2, return_state=True)
    assert_close(y2, ref2[:, 100:], what="segmented + carry-in", **FWD32)
    assert_close(st2["u"] / st2["d"][..., None], st_ref["u"] / st_ref["d"][..., None], what="state z", **ST32)


def test_strided_inputs_and_non_contiguous_views():
    q, k, v = orc.make_inputs(2, 50, 4, 16, 32, seed0=3)
    ref = orc.ar_forward(q[1:3], k[:, :, 1:3], v[:, :, 1:3])
    qc, kc, vc = to_dev(q, k, v)
    y = cf.flare_autoregressive_triton(qc[1:3], kc[:, :, 1:3], vc[:, :, 1:3])  # head-sliced views, no copy needed
    assert_close(y, ref, what="head slice", **FWD32)
    kt = kc.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)  # [B,H,N,D] storage viewed as [B,N,H,D]
    y2 = cf.flare_autoregressive_triton(qc, kt, vc)
    assert_close(y2, orc.ar_forward(q, k, v), what="bhnd storage", **FWD32)
    y3 = cf.flare_autoregressive_triton(qc[:, :, ::2].repeat(1, 1, 2)[..., :32], kc, vc)
    assert y3.shape == ref.shape[:2] + (4, 32)


def test_cached_prefill_decode_with_masks(golden):
    g = golden("cached")
    q, k, v, mask, k2, v2, mask2 = to_dev(g["q"], g["k"], g["v"], g["mask"], g["k2"], g["v2"], g["mask2"])
    sc = g["scale"]
    y1, s1 = cf.flare_autoregressive_prefill_triton(q, k, v, scale=sc, attention_mask=mask)
    assert_close(y1, g["y1"], what="masked prefill y", **FWD32)
    fin = torch.isfinite(g["m1"])
    assert bool((torch.isfinite(s1["m"]).cpu() == fin).all())
    assert_close(s1["d"], g["d1"], what="d1", **ST32)
    assert_close(s1["u"], g["u1"], what="u1", **ST32)
    y2, s2 = cf.flare_autoregressive_decode_triton(q, k2, v2, s1, scale=sc, attention_mask=mask2)
    assert y2.shape == (2, 1, 4, 32)
    assert_close(y2, g["y2"], what="masked decode y", **FWD32)
    assert_close(s2["u"], g["u2"], what="u2", **ST32)
    assert s2["u"].data_ptr() == s1["u"].data_ptr(), "decode updates the fp32 state in place"
    y1u, s1u = cf.flare_autoregressive_prefill_triton(q, k, v, scale=sc)
    assert_close(y1u, g["y1u"], what="prefill y", **FWD32)
    assert_close(s1u["m"], g["m1u"], what="m1u", **ST32)
    y2u, s2u = cf.flare_autoregressive_decode_triton(q, k2[:, 0], v2[:, 0], s1u, scale=sc)
    assert_close(y2u, g["y2u"], what="decode y", **FWD32)
    assert_close(s2u["m"], g["m2u"], what="m2u", **ST32)
    assert_close(s2u["d"], g["d2u"], what="d2u", **ST32)
    assert_close(s2u["u"], g["u2u"], what="u2u", **ST32)
    # masked prefill == token-by-token masked decode
    st = None
    ys = []
    for t in range(k.shape[1]):
        yt, st = cf.flare_autoregressive_decode_triton(q, k[:, t], v[:, t], st, scale=sc, attention_mask=mask[:, t])
        ys.append(yt)
    assert_close(torch.cat(ys, 1), g["y1"], what="decode loop", **FWD32)


def test_prefill_empty_sequence_and_default_scale():
    q, k, v = to_dev(*orc.make_inputs(2, 8, 2, 16, 16))
    y, st = cf.flare_autoregressive_prefill_triton(q, k[:, :0], v[:, :0])
    assert y.shape == (2, 0, 2, 16) and bool(torch.isinf(st["m"]).all()) and float(st["u"].abs().sum()) == 0
    y1, _ = cf.flare_autoregressive_prefill_triton(q, k, v)  # default scale is 1.0 here
    ref = orc.ar_forward(q.cpu(), k.cpu(), v.cpu(), scale=1.0)
    assert_close(y1, ref, what="scale=1 default", **FWD32)


@pytest.mark.parametrize("sep_q, sep_k", [(0, 0), (1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("shape", [(3, 2, 64, 32, 32), (2, 2, 256, 128, 128), (1, 1, 48, 16, 48)])
def test_decode_step_against_oracle(shape, sep_q, sep_k):
    B, H, M, Dk, Dv = shape
    q, k, v = orc.make_inputs(B, 9, H, M, Dk, Dv, seed0=21, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(5)
    qd = torch.randn(B, 9, H, Dk, generator=g).bfloat16() if sep_q else None
    kd = torch.randn(H, M, Dk, generator=g).bfloat16() if sep_k else None
    sc = Dk ** -0.5
    _, st = orc.ar_forward(q, k[:, :8], v[:, :8], scale=sc, Q_dec=None if qd is None else qd[:, :8], K_dec=kd,
                           return_state=True)
    y_ref, st_ref = orc.decode_step(q, k[:, 8], v[:, 8], st, scale=sc, q_dec=None if qd is None else qd[:, 8], K_dec=kd)
    st_gpu = {a: b.float().cuda() for a, b in st.items()}
    qc, kc, vc, qdc, kdc = to_dev(q, k, v, qd, kd)
    y, st_new = cf.flare_autoregressive_decode_triton(qc, kc[:, 8], vc[:, 8], st_gpu, scale=sc,
                                                      Q_dec=None if qd is None else qdc[:, 8], K_dec=kdc)
    assert y.dtype == torch.bfloat16
    assert_bf16_gate(y, y_ref, "decode y")
    for key in "mdu":
        assert_close(st_new[key], st_ref[key], what="state " + key, **ST32)


def test_recurrent_output_layout(golden):
    g = golden("recurrent")
    q, k, v = to_dev(g["q"], g["k"], g["v"])
    y = cf.flare_recurrent_triton(q, k, v)
    assert tuple(y.shape) == tuple(g["y_bhnd"].shape)
    assert_close(y, g["y_bhnd"], what="recurrent", **FWD32)
    y16 = cf.flare_recurrent_triton(q, k, v, block_t=16)
    assert torch.equal(y, y16)


@pytest.mark.parametrize("p", [1, 2, 3])
def test_stablemax_forward(golden, p):
    g = golden(f"stablemax_p{p}")
    q, k, v = to_dev(g["q"], g["k"], g["v"])
    y = flare_autoregressive_stablemax_triton(q, k, v, power=g["power"])
    assert_close(y, g["y"], what="stablemax", **FWD32)


def test_stablemax_forward_bf16_and_generic_power():
    q, k, v = orc.make_inputs(2, 200, 2, 64, 32, seed0=31, dtype=torch.bfloat16)
    for power in (2.0, 2.5):
        ref = orc.ar_forward(q, k, v, variant="stablemax", power=power)
        y = flare_autoregressive_stablemax_triton(*to_dev(q, k, v), power=power)
        assert y.dtype == torch.bfloat16
        assert_bf16_gate(y, ref, f"stablemax p={power}")
    e = flare_autoregressive_stablemax_triton(*to_dev(q, k[:, :0], v[:, :0]))
    assert e.shape == (2, 0, 2, 32)


@pytest.mark.parametrize("sep", [0, 1])
def test_semi_ar_forward(golden, sep):
    g = golden(f"semi_ar_sep{sep}")
    q, k, v, qd, kd = to_dev(g["q"], g["k"], g["v"], g.get("q_dec"), g.get("k_dec"))
    y, aux = cf.flare_semi_autoregressive_trition(q, k, v, block_size=32, chunk_size=16, Q_dec=qd, K_dec=kd)
    assert_close(y, g["y"], what="semi-AR y", **FWD32)
    assert_close(aux["LSE_dec"], g["lse_dec"], what="LSE_dec", **FWD32)
    assert_close(aux["LSE_enc"], g["lse_enc"], what="LSE_enc", **FWD32)
    y2, _ = cf.flare_semi_autoregressive_trition(q, k, v, block_size=32, chunk_size=32, Q_dec=qd, K_dec=kd)
    assert torch.equal(y, y2), "chunk_size must not change the result"


def test_semi_ar_bf16_long_and_segmented(monkeypatch):
    monkeypatch.setenv("FLARE_B200_PATH", "exact")  # the tensor path has its own test with its own LSE tolerance
    q, k, v = orc.make_inputs(1, 1024, 2, 64, 64, seed0=41, dtype=torch.bfloat16)
    ref, lse_dec, lse_enc = orc.semi_ar_forward(q, k, v, block_size=64)
    y, aux = cf.flare_semi_autoregressive_trition(*to_dev(q, k, v), block_size=64, chunk_size=64)
    assert_bf16_gate(y, ref, "semi-AR bf16")
    assert_close(aux["LSE_enc"], lse_enc, what="LSE_enc", atol=1e-4, rtol=1e-4)
    assert_close(aux["LSE_dec"], lse_dec, what="LSE_dec", atol=1e-4, rtol=1e-4)


def test_state_merge_kernel_matches_oracle():
    from causal_flare.autoregressive.inference import _merge_flare_stats

    q, k, v = orc.make_inputs(2, 30, 2, 32, 32, seed0=51)
    _, sa = orc.ar_forward(q, k[:, :13], v[:, :13], return_state=True)
    _, sb = orc.ar_forward(q, k[:, 13:], v[:, 13:], return_state=True)
    ref = orc.merge_states(sa, sb)
    a = {x: y.float().cuda() for x, y in sa.items()}
    b = {x: y.float().cuda() for x, y in sb.items()}
    m, d, u = _merge_flare_stats(a["m"], a["d"], a["u"], b["m"], b["d"], b["u"])
    assert_close(m, ref["m"], what="m", **ST32)
    assert_close(d, ref["d"], what="d", **ST32)
    assert_close(u, ref["u"], what="u", **ST32)
    empty = {x: y.cuda() for x, y in orc.init_state(2, 2, 32, 32).items()}
    m2, d2, u2 = _merge_flare_stats(empty["m"], empty["d"], empty["u"], a["m"], a["d"], a["u"])
    assert torch.equal(u2, a["u"]) and torch.equal(m2, a["m"])
    m3, d3, _ = _merge_flare_stats(empty["m"], empty["d"], empty["u"], empty["m"], empty["d"], empty["u"])
    assert bool(torch.isinf(m3).all()) and float(d3.abs().sum()) == 0.0


def test_profile_returns_timings(golden):
    g = golden("ar_sep00")
    q, k, v = to_dev(g["q"], g["k"], g["v"])
    y, prof = cf.flare_autoregressive_triton(q, k, v, profile=True)
    assert "forward" in prof and prof["forward_total_ms"] > 0 and "backward" in prof
    # one entry per kernel, as in the reference's profile dict; the entries add up to the total
    assert any(name.startswith("walk_exact_kernel") for name in prof["forward"]), prof["forward"]
    assert abs(sum(prof["forward"].values()) - prof["forward_total_ms"]) < 1e-6
    (y2, st), prof2 = cf.flare_autoregressive_prefill_triton(q, k, v, profile=True)
    assert prof2["forward_total_ms"] > 0
    # bf16 on the tensor path: the tcgen05 kernels show up by name, forward and backward
    qb, kb, vb = (t.bfloat16().requires_grad_(True) for t in (torch.randn(2, 64, 64, device="cuda"),
                                                                torch.randn(1, 256, 2, 64, device="cuda"),
                                                                torch.randn(1, 256, 2, 64, device="cuda")))
    yb, pb = cf.flare_autoregressive_triton(qb, kb, vb, profile=True)
    assert "prefill_tc_kernel" in pb["forward"]
    yb.backward(torch.ones_like(yb))
    assert {"bwd_tc_kernel", "bwd_tc_grads_kernel"} <= set(pb["backward"]) and pb["backward_total_ms"] > 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_semi_ar_block_granular_cached_prefill(dtype):
    # feeding whole blocks with a carried state equals the one-shot block-causal forward (exact path for fp32,
    # tensor path for bf16); a single block per call is block-granular decoding
    from causal_flare.semi_autoregressive.inference import flare_semi_autoregressive_block_prefill

    B, N, H, M, D, bs = 2, 384, 2, 64, 64, 32
    q, k, v = orc.make_inputs(B, N, H, M, D, seed0=81, dtype=dtype)
    ref, _, _ = orc.semi_ar_forward(q, k, v, block_size=bs)
    qc, kc, vc = to_dev(q, k, v)
    state, ys = None, []
    for lo, hi in ((0, 160), (160, 192), (192, 384)):
        y, state = flare_semi_autoregressive_block_prefill(qc, kc[:, lo:hi], vc[:, lo:hi], block_size=bs, state=state)
        ys.append(y)
    y = torch.cat(ys, 1)
    if dtype == torch.float32:
        assert_close(y, ref, what="block-granular prefill", **FWD32)
    else:
        assert_bf16_gate(y, ref, "block-granular prefill bf16")
    _, st_full = cf.flare_autoregressive_prefill_triton(qc, kc, vc, scale=D ** -0.5)
    assert_close(state["d"], st_full["d"], what="final state d", atol=1e-3, rtol=2e-3)
    with pytest.raises(ValueError):
        flare_semi_autoregressive_block_prefill(qc, kc[:, :40], vc[:, :40], block_size=bs)


def test_semi_ar_token_decode_releases_outputs_block_by_block():
    # token-by-token decoding of the block-causal operator: nothing is returned inside a block, the call that completes
    # a block returns the whole block's outputs, which equal the full-sequence operator's
    from causal_flare.semi_autoregressive.inference import (SemiAutoRegressiveTokenCache,
                                                            flare_semi_autoregressive_block_prefill,
                                                            flare_semi_autoregressive_token_decode)

    B, N, H, Ml, Dl, bs = 2, 96, 2, 32, 64, 32
    q, k, v = orc.make_inputs(B, N, H, Ml, Dl, seed0=41, dtype=torch.bfloat16)
    ref = orc.semi_ar_forward(q, k, v, block_size=bs)[0]
    qc, kc, vc = to_dev(q, k, v)
    # the first block through the block-granular prefill, the rest one token at a time on top of its state
    y0, st = flare_semi_autoregressive_block_prefill(qc, kc[:, :bs], vc[:, :bs], block_size=bs)
    cache = SemiAutoRegressiveTokenCache(st, bs)
    outs = [y0]
    for t in range(bs, N):
        y, cache = flare_semi_autoregressive_token_decode(qc, kc[:, t], vc[:, t:t + 1], cache, block_size=bs)
        if (t + 1) % bs == 0:
            assert y is not None and tuple(y.shape) == (B, bs, H, Dl) and cache.pending == 0
            outs.append(y)
        else:
            assert y is None and cache.pending == (t + 1) % bs
    assert_bf16_gate(torch.cat(outs, 1), ref, "token-granular block-causal decode")
    full = cf.flare_semi_autoregressive_trition(qc, kc, vc, block_size=bs, chunk_size=16)[0]
    assert orc.max_abs(torch.cat(outs, 1).float().cpu(), full.float().cpu()) <= 2e-2
    with pytest.raises(ValueError):
        flare_semi_autoregressive_token_decode(qc, kc[:, 0], vc[:, 0], cache, block_size=16)

