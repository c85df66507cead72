"""GPU parity of the wide (Dk, Dv) = (128, 128) prefill instance: one CTA carries all 128 value columns of a
(lane, latent group) instead of two CTAs with 64 each.  The library picks it when the two-slice grid would not fit
the SMs in one wave; here FLARE_B200_WIDE=1 forces it on small shapes, and every case is also compared with the
two-slice instance (FLARE_B200_WIDE=0) on the same inputs."""
import pytest
import torch

from causal_flare import _lib, _ops
from oracle import flare_oracle as orc
from util import assert_bf16_gate, assert_close, to_dev

pytestmark = pytest.mark.gpu

D = 128


def run(q, k, v, **kw):
    out = _ops.forward(q, k, v, scale=kw.pop("scale", D ** -0.5), path=_lib.PATH_TENSOR, **kw)
    assert _ops.device_status() == 0, "a tensor-core kernel gave up on a bounded wait"
    return out


@pytest.fixture(params=["on-chip merge", "merge kernel"])
def wide(monkeypatch, request):
    # two latent groups (M = 256): the two CTAs of a lane merge on chip as a thread-block cluster by default;
    # FLARE_B200_CLUSTER=0 keeps the partials in global memory and the merge kernel (the path M = 384 / 512 always take)
    monkeypatch.setenv("FLARE_B200_WIDE", "1")
    if request.param == "merge kernel":
        monkeypatch.setenv("FLARE_B200_CLUSTER", "0")
    return monkeypatch


@pytest.mark.parametrize("Ml, B, N, H", [(128, 1, 128, 1), (128, 2, 700, 2), (256, 1, 1000, 2), (512, 1, 384, 1),
                                         (128, 1, 4096, 1)])
def test_wide_matches_oracle_and_two_slice_instance(wide, Ml, B, N, H):
    q, k, v = orc.make_inputs(B, N, H, Ml, D, seed0=11, dtype=torch.bfloat16)
    ref, st_ref = orc.ar_forward(q, k, v, scale=D ** -0.5, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    y, st, ld, _ = run(qc, kc, vc, want_state=True, want_lse=True)
    assert_bf16_gate(y, ref, f"wide instance M={Ml} B={B} N={N} H={H}")
    assert_close(st["m"], st_ref["m"], what="m", atol=1e-4, rtol=1e-4)
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3
    wide.setenv("FLARE_B200_WIDE", "0")
    y2, st2, ld2, _ = run(qc, kc, vc, want_state=True, want_lse=True)
    assert_bf16_gate(y, y2.float(), "wide vs two-slice instance")
    assert_close(ld, ld2, what="LSE_dec", atol=5e-3, rtol=0)
    assert orc.rel_l2(st["u"].cpu(), st2["u"].cpu()) < 1e-3


def test_wide_is_deterministic(wide):
    q, k, v = orc.make_inputs(2, 900, 2, 256, D, seed0=12, dtype=torch.bfloat16)
    qc, kc, vc = to_dev(q, k, v)
    y1, _, _, _ = run(qc, kc, vc)
    y2, _, _, _ = run(qc, kc, vc)
    assert torch.equal(y1, y2)


@pytest.mark.parametrize("Ml", [128, 256])
def test_wide_state_in_and_state_only(wide, Ml):
    q, k, v = orc.make_inputs(2, 656, 2, Ml, D, seed0=13, dtype=torch.bfloat16)
    sc = D ** -0.5
    _, st0 = orc.ar_forward(q, k[:, :144], v[:, :144], scale=sc, return_state=True)
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    st_in = {a: b.float().cuda().contiguous() for a, b in st0.items()}
    y, st, _, _ = run(qc, kc[:, 144:], vc[:, 144:], state_in=st_in, want_state=True, scale=sc)
    assert_bf16_gate(y, ref[:, 144:], "wide carry-in y")
    assert_close(st["m"], st_ref["m"], what="m", atol=1e-4, rtol=1e-4)
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3
    # no read-out: state only
    y0, st2, _, _ = run(qc, kc, vc, want_state=True, want_y=False, scale=sc)
    assert y0 is None
    assert_close(st2["d"], st_ref["d"], what="d (state only)", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st2["u"].cpu(), st_ref["u"]) < 3e-3


@pytest.mark.parametrize("bs, Ml, B, N, H", [(16, 128, 2, 400, 2), (64, 256, 2, 576, 2), (128, 128, 1, 1024, 1),
                                             (32, 256, 1, 2048, 1)])
def test_wide_block_causal(wide, bs, Ml, B, N, H):
    q, k, v = orc.make_inputs(B, N, H, Ml, D, seed0=14, dtype=torch.bfloat16)
    sc = D ** -0.5
    ref, lse_dec, lse_enc = orc.semi_ar_forward(q, k, v, block_size=bs, scale=sc)
    qc, kc, vc = to_dev(q, k, v)
    y, _, ld, le = run(qc, kc, vc, block_size=bs, want_lse=True, scale=sc)
    assert_bf16_gate(y, ref, f"wide block-causal bs={bs} M={Ml}")
    assert_close(le, lse_enc, what="LSE_enc", atol=2e-4, rtol=2e-4)
    assert_close(ld, lse_dec, what="LSE_dec", atol=5e-3, rtol=0)


@pytest.mark.parametrize("power, Ml, B, N, H", [(2.0, 128, 2, 520, 2), (3.0, 256, 1, 700, 2)])
def test_wide_stablemax(wide, power, Ml, B, N, H):
    q, k, v = orc.make_inputs(B, N, H, Ml, D, seed0=15, dtype=torch.bfloat16)
    sc = D ** -0.5
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, variant="stablemax", power=power, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    y, st, _, _ = run(qc, kc, vc, variant=_lib.STABLEMAX, power=power, want_state=True, scale=sc)
    assert_bf16_gate(y, ref, f"wide stablemax p={power} M={Ml}")
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3


def test_wide_is_the_default_for_grids_beyond_one_wave():
    # 160 lanes x 2 value slices do not fit 148 SMs at once: the library takes the wide instance without being told
    q, k, v = orc.make_inputs(5, 384, 32, 128, D, seed0=16, dtype=torch.bfloat16)
    ref = orc.ar_forward(q, k, v, scale=D ** -0.5)
    y, _, _, _ = run(*to_dev(q, k, v))
    assert_bf16_gate(y, ref, "wide instance by default")


def test_wide_long_block_causal_lanes_at_full_length(wide):
    # C5's lanes at their full length (N = 65536, M = 256, D = 128, block 64; two of the 64 lanes): every token against
    # the oracle, 512 chunks of running frames, carried state and (by default) the on-chip merge of the two groups
    q, k, v = orc.make_inputs(1, 65536, 2, 256, D, seed0=17, dtype=torch.bfloat16)
    sc = D ** -0.5
    ref, lse_dec, lse_enc = orc.semi_ar_forward(q, k, v, block_size=64, scale=sc)
    qc, kc, vc = to_dev(q, k, v)
    y, _, ld, le = run(qc, kc, vc, block_size=64, want_lse=True, scale=sc)
    assert_bf16_gate(y, ref, "C5 lanes at full length, wide instance")
    assert_bf16_gate(y[:, -4096:], ref[:, -4096:], "C5 lanes, last 4096 tokens")
    assert_close(le, lse_enc, what="LSE_enc", atol=5e-4, rtol=5e-4)
    assert_close(ld, lse_dec, what="LSE_dec", atol=5e-3, rtol=0)


@pytest.mark.parametrize("bs, Ml", [(1, 128), (1, 256), (64, 256)])
def test_wide_training_forward_keeps_the_same_states_as_the_two_slice_instance(wide, bs, Ml):
    # the training forward leaves the per-chunk prefix states for the backward: gradients from the states kept by the
    # wide instance equal those from the two-slice instance's and pass the oracle's closed form
    q, k, v, dy = orc.make_inputs(2, 640, 2, Ml, D, seed0=18, dtype=torch.bfloat16, with_dy=True)
    sc = D ** -0.5
    qc, kc, vc, dyc = to_dev(q, k, v, dy)
    out = {}
    for w in ("1", "0"):
        wide.setenv("FLARE_B200_WIDE", w)
        kept = {}
        y, _, _, _ = _ops.forward(qc, kc, vc, scale=sc, block_size=bs, keep_for_backward=kept)
        out[w] = (y, _ops.backward(qc, kc, vc, dyc, scale=sc, block_size=bs, saved=kept)[:3])
        assert _ops.device_status() == 0
    assert_bf16_gate(out["1"][0], out["0"][0].float(), "y of the training forward, wide vs two-slice")
    for name, a, b in zip(("dQ", "dK", "dV"), out["1"][1], out["0"][1]):
        assert orc.rel_l2(a.float().cpu(), b.float().cpu()) < 2e-3, name
    ref = orc.ar_backward_closed_form(q, k, v, dy, scale=sc, block_size=bs)
    for name, got in zip(("dQ", "dK", "dV"), out["1"][1]):
        assert orc.rel_l2(got.float().cpu(), ref[name]) <= 6.5e-3, name
