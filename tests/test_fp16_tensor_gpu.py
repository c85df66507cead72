"""fp16 inputs on the tensor-core prefill: the library rounds q, k, v to bf16 copies in its workspace, runs the bf16
kernels on them and writes y back as fp16.  Every case is held to the oracle on the fp16 inputs with the bf16 gate
(the products inside the kernels are bf16 for every input type), and to the exact kernels, which read fp16 directly."""
import ctypes as C

import pytest
import torch

import causal_flare as cf
from causal_flare import _lib, _ops
from oracle import flare_oracle as orc
from util import assert_bf16_gate, assert_close, to_dev

pytestmark = pytest.mark.gpu

F16 = torch.float16


def run(q, k, v, **kw):
    out = _ops.forward(q, k, v, scale=kw.pop("scale", q.shape[-1] ** -0.5), **kw)
    assert _ops.device_status() == 0
    return out


def z_of(st):
    """The state without its frame: u / d, and the encoder log-sum-exp m + log d (rounding q and k moves the frame
    maximum m by a few 1e-3, which shifts d and u by that factor but neither of these)."""
    st = {a: b.float().cpu() for a, b in st.items()}
    return st["u"] / st["d"][..., None], st["m"] + st["d"].log()


def on_tensor_path(q, k, v, y, **kw):
    probe = _lib.make_fwd_args(q, k, v, None, None, y, scale=1.0, variant=kw.get("variant", _lib.SOFTMAX), power=2.0,
                               block_size=kw.get("block_size", 1), path=_lib.PATH_AUTO)
    return _lib.load().flare_forward_uses_tensor_path(C.byref(probe)) == 1


@pytest.mark.parametrize("B, N, H, M, Dk, Dv", [(2, 2048, 4, 64, 64, 64), (1, 129, 2, 32, 64, 128), (2, 1000, 2, 256, 128, 128),
                                                (1, 4096, 1, 128, 64, 64), (1, 700, 3, 512, 128, 128)])
def test_fp16_forward_matches_oracle_and_exact_kernels(B, N, H, M, Dk, Dv):
    q, k, v = orc.make_inputs(B, N, H, M, Dk, Dv, seed0=51, dtype=F16)
    ref, st_ref = orc.ar_forward(q, k, v, scale=Dk ** -0.5, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    y, st, ld, _ = run(qc, kc, vc, want_state=True, want_lse=True)
    assert y.dtype == F16 and on_tensor_path(qc, kc, vc, y)
    assert_bf16_gate(y, ref, f"fp16 on the tensor path {(B, N, H, M, Dk, Dv)}")
    z, lse = z_of(st)
    z_ref, lse_ref = z_of(st_ref)
    assert orc.rel_l2(z, z_ref) < 5e-3
    assert_close(lse, lse_ref, what="encoder log-sum-exp", atol=1e-2, rtol=0)
    ye, se, lde, _ = run(qc, kc, vc, want_state=True, want_lse=True, path=_lib.PATH_EXACT)
    assert_bf16_gate(y, ye.float(), "fp16: tensor path vs exact kernels")
    assert_close(ld, lde, what="LSE_dec", atol=2e-2, rtol=0)
    assert_close(lse, z_of(se)[1], what="encoder log-sum-exp vs exact kernels", atol=1e-2, rtol=0)


def test_fp16_public_api_strided_inputs_and_layouts():
    # k and v as slices of one fused projection (row stride 3 x H x D) and the [B, H, N, D] output layout
    B, N, H, M, D = 2, 640, 4, 64, 64
    q, k, v = orc.make_inputs(B, N, H, M, D, seed0=52, dtype=F16)
    ref = orc.ar_forward(q, k, v)
    fused = torch.empty(B, N, 3, H, D, dtype=F16, device="cuda")
    fused[:, :, 1], fused[:, :, 2] = k.cuda(), v.cuda()
    kc, vc = fused[:, :, 1], fused[:, :, 2]
    assert not kc.is_contiguous()
    y = cf.flare_autoregressive_triton(q.cuda(), kc, vc)
    assert y.dtype == F16
    assert_bf16_gate(y, ref, "fp16 strided k / v through the public entry point")
    yb, _, _, _ = run(q.cuda(), kc, vc, out_bhnd=True)
    assert tuple(yb.shape) == (B, H, N, D)
    assert torch.equal(yb.permute(0, 2, 1, 3), y)


def test_fp16_carried_state_block_causal_and_stablemax():
    B, N, H, M, D = 2, 1024, 2, 256, 128
    q, k, v = orc.make_inputs(B, N, H, M, D, seed0=53, dtype=F16)
    sc = D ** -0.5
    qc, kc, vc = to_dev(q, k, v)
    # carry: first 384 tokens, then the rest from the returned state
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, return_state=True)
    _, st0, _, _ = run(qc, kc[:, :384], vc[:, :384], want_state=True, want_y=False)
    y1, st1, _, _ = run(qc, kc[:, 384:], vc[:, 384:], state_in=st0, want_state=True)
    assert_bf16_gate(y1, ref[:, 384:], "fp16 carry-in")
    assert orc.rel_l2(z_of(st1)[0], z_of(st_ref)[0]) < 5e-3
    # block-causal read-out
    refb, lse_dec, lse_enc = orc.semi_ar_forward(q, k, v, block_size=64, scale=sc)
    yb, _, ld, le = run(qc, kc, vc, block_size=64, want_lse=True)
    assert yb.dtype == F16 and on_tensor_path(qc, kc, vc, yb, block_size=64)
    assert_bf16_gate(yb, refb, "fp16 block-causal")
    assert_close(le, lse_enc, what="LSE_enc", atol=1e-2, rtol=0)
    # stablemax encoder
    refs = orc.ar_forward(q, k, v, scale=sc, variant="stablemax", power=2.0)
    ys, _, _, _ = run(qc, kc, vc, variant=_lib.STABLEMAX, power=2.0)
    assert_bf16_gate(ys, refs, "fp16 stablemax")


def test_fp16_masked_rows_and_sharp_scores_keep_the_default_path_correct():
    B, N, H, M, D = 2, 512, 2, 64, 64
    q, k, v = orc.make_inputs(B, N, H, M, D, seed0=54, dtype=F16)
    # right-padded rows: served by compaction + per-row lengths on the tensor path
    mask = torch.ones(B, N, dtype=torch.int32)
    mask[0, 300:] = 0
    mask[1, 77:] = 0
    qc, kc, vc = to_dev(q, k, v)
    y, _, _, _ = run(qc, kc, vc, mask=mask.cuda())
    for b, n in ((0, 300), (1, 77)):
        ref = orc.ar_forward(q, k[b:b + 1, :n], v[b:b + 1, :n], scale=D ** -0.5)
        assert_bf16_gate(y[b:b + 1, :n], ref, f"fp16 masked row {b}")
        assert float(y[b, n:].abs().max()) == 0.0
    # score spreads of hundreds of nats: the kernels flag the lanes and the exact kernels recompute them from the fp16
    # tensors themselves (rounding q and k to bf16 would move such scores by more than a nat); a lane that stayed in
    # the kernels' domain is held to the oracle on the bf16 copies instead
    qs, ks = (q.float() * 8).to(F16), (k.float() * 8).to(F16)
    ref_h = orc.ar_forward(qs, ks, v, scale=D ** -0.5).float()
    ref_b = orc.ar_forward(qs.bfloat16(), ks.bfloat16(), v.bfloat16(), scale=D ** -0.5).float()
    ysh, _, _, _ = _ops.forward(qs.cuda(), ks.cuda(), vc, scale=D ** -0.5)
    status = _ops.device_status()
    assert status in (0, 2)  # 2: the exact kernels had to step in (informational)
    assert ysh.dtype == F16
    from_fp16 = 0
    for b in range(B):
        for h in range(H):
            got = ysh[b:b + 1, :, h:h + 1]
            bound = max(2e-2, 1e-2 * float(ref_h.abs().max()))
            try:
                assert_bf16_gate(got, ref_h[b:b + 1, :, h:h + 1], f"fp16 sharp scores, lane ({b}, {h})", max_abs=bound)
                from_fp16 += 1
            except AssertionError:
                assert_bf16_gate(got, ref_b[b:b + 1, :, h:h + 1], f"fp16 sharp scores, lane ({b}, {h}), bf16 copies", max_abs=bound)
    assert status == 0 or from_fp16 > 0, "flagged lanes must come from the fp16 tensors"


@pytest.mark.parametrize("B, N, H, M, Dk, Dv, bs, variant", [
    (2, 512, 2, 64, 128, 128, 1, "softmax"), (1, 300, 2, 64, 64, 64, 1, "softmax"), (1, 640, 2, 256, 128, 128, 64, "softmax"),
    (1, 384, 1, 48, 64, 128, 1, "stablemax")])
def test_fp16_backward_on_the_tensor_kernels(B, N, H, M, Dk, Dv, bs, variant):
    # gradients of fp16 inputs: bf16 copies of q, k, v, dY, the tensor-core backward, dK / dV back as fp16.  Against the
    # oracle on the bf16-rounded inputs the bound is the one of the bf16 shape sweep; against the oracle on the fp16
    # inputs the rounding of the four inputs adds to it.
    q, k, v, dy = orc.make_inputs(B, N, H, M, Dk, Dv, seed0=55, dtype=F16, with_dy=True)
    sc = Dk ** -0.5
    var = _lib.SOFTMAX if variant == "softmax" else _lib.STABLEMAX
    qc, kc, vc, dyc = to_dev(q, k, v, dy)
    a = _lib.BwdArgs()
    a.fwd = _lib.make_fwd_args(qc, kc, vc, None, None, None, scale=sc, variant=var, block_size=bs)
    a.dy = dyc.data_ptr()
    a.dy_stride_b, a.dy_stride_n, a.dy_stride_h = dyc.stride(0), dyc.stride(1), dyc.stride(2)
    dq0, dk0, dv0 = torch.empty(qc.shape, device="cuda"), torch.empty_like(kc), torch.empty_like(vc)
    a.dq, a.dk, a.dv = dq0.data_ptr(), dk0.data_ptr(), dv0.data_ptr()
    assert _lib.load().flare_backward_uses_tensor_path(C.byref(a)) == 1
    dq, dk, dv, _, _ = _ops.backward(qc, kc, vc, dyc, scale=sc, variant=var, power=2.0, block_size=bs)
    assert _ops.device_status() == 0
    assert dq.dtype == torch.float32 and dk.dtype == F16 and dv.dtype == F16
    got = dict(dQ=dq, dK=dk, dV=dv)
    kw = dict(scale=sc, block_size=bs, variant=variant, power=2.0)
    ref_b = orc.ar_backward_closed_form(q.bfloat16(), k.bfloat16(), v.bfloat16(), dy.bfloat16(), **kw)
    ref_h = orc.ar_backward_closed_form(q, k, v, dy, **kw)
    for key in ("dQ", "dK", "dV"):
        peak = float(ref_h[key].abs().max())
        assert_bf16_gate(got[key], ref_b[key], f"fp16 {key} vs oracle on the bf16 copies", max_abs=max(2e-2, peak * 2.0 ** -7),
                         rel_l2=6.5e-3)
        assert_bf16_gate(got[key], ref_h[key], f"fp16 {key} vs oracle on the fp16 inputs", max_abs=max(2e-2, peak * 2.0 ** -7),
                         rel_l2=8e-3)


def test_fp16_training_step_through_autograd():
    B, N, H, M, D = 2, 512, 2, 64, 64
    q, k, v, dy = orc.make_inputs(B, N, H, M, D, seed0=56, dtype=F16, with_dy=True)
    ref = orc.ar_backward_closed_form(q, k, v, dy)
    ql, kl, vl = (t.cuda().requires_grad_(True) for t in (q, k, v))
    y = cf.flare_autoregressive_triton(ql, kl, vl)
    assert y.dtype == F16
    assert_bf16_gate(y, orc.ar_forward(q, k, v), "fp16 y of the training forward")
    y.backward(dy.cuda())
    assert _ops.device_status() == 0
    for got, key in ((ql.grad, "dQ"), (kl.grad, "dK"), (vl.grad, "dV")):
        assert got.dtype == F16
        assert_bf16_gate(got, ref[key], f"fp16 autograd {key}", max_abs=max(2e-2, float(ref[key].abs().max()) * 2.0 ** -7),
                         rel_l2=8e-3)


def test_fp16_through_the_entry_point_that_allocates_nothing():
    # the bf16 copies live in the library's built-in scratch when they fit it (same bits as flare_forward with a
    # workspace); when they do not, the call runs on the exact kernels, which read fp16 directly
    lib = _lib.load()
    cap = lib.flare_noalloc_scratch_capacity()
    stream = torch.cuda.current_stream().cuda_stream
    for (B, N, H, M, D), fits in (((1, 1024, 2, 64, 64), True), ((2, 8192, 8, 64, 64), False)):
        q, k, v = to_dev(*orc.make_inputs(B, N, H, M, D, seed0=57, dtype=F16))
        y = torch.full_like(v, float("nan"))
        args = _lib.make_fwd_args(q, k, v, None, None, y, scale=D ** -0.5)
        need = lib.flare_forward_workspace_bytes(C.byref(args))
        assert (need <= cap) == fits
        assert lib.flare_forward_noalloc(C.byref(args), stream) == 0
        torch.cuda.synchronize()
        want = _ops.forward(q, k, v, scale=D ** -0.5, path=_lib.PATH_AUTO if fits else _lib.PATH_EXACT)[0]
        assert torch.equal(y, want)
    assert _ops.device_status() == 0
