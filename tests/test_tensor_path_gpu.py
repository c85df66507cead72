"""GPU parity of the tcgen05 tensor-core prefill path (bf16, M=128, D=64) against the CPU oracle, the exact
CUDA path, and size-independent properties at the full benchmark size."""
import ctypes as C

import pytest
import torch

import causal_flare as cf
from causal_flare import _lib, _ops
from oracle import flare_oracle as orc
from util import assert_bf16_gate, assert_close, to_dev

pytestmark = pytest.mark.gpu

M, D = 128, 64


def run(q, k, v, path, **kw):
    out = _ops.forward(q, k, v, scale=kw.pop("scale", D ** -0.5), path=path, **kw)
    assert _ops.device_status() == 0, "a tensor-core kernel gave up on a bounded wait"
    return out


def uses_tensor_path(q, k, v):
    args = _lib.make_fwd_args(q, k, v, None, None, torch.empty_like(v), scale=1.0)
    return _lib.load().flare_forward_uses_tensor_path(C.byref(args)) == 1


@pytest.mark.parametrize("B, N, H", [(1, 128, 1), (1, 256, 1), (2, 300, 2), (1, 1000, 3)])
def test_tensor_path_matches_oracle(B, N, H):
    q, k, v = orc.make_inputs(B, N, H, M, D, seed0=3, dtype=torch.bfloat16)
    ref = orc.ar_forward(q, k, v)
    qc, kc, vc = to_dev(q, k, v)
    assert uses_tensor_path(qc, kc, vc)
    y, _, _, _ = run(qc, kc, vc, _lib.PATH_TENSOR)
    assert_bf16_gate(y, ref, f"tensor path B={B} N={N} H={H}")


def test_tensor_path_state_in_and_out():
    q, k, v = orc.make_inputs(2, 400, 2, M, D, seed0=5, dtype=torch.bfloat16)
    sc = D ** -0.5
    _, st0 = orc.ar_forward(q, k[:, :144], v[:, :144], scale=sc, return_state=True)
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    st_in = {a: b.float().cuda().contiguous() for a, b in st0.items()}
    y, st, _, _ = run(qc, kc[:, 144:], vc[:, 144:], _lib.PATH_TENSOR, state_in=st_in, want_state=True, scale=sc)
    assert_bf16_gate(y, ref[:, 144:], "carry-in y")
    assert_close(st["m"], st_ref["m"], what="m", atol=1e-4, rtol=1e-4)
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3
    # the public prefill API takes the same route and continues correctly into the decode kernel
    y2, st2 = cf.flare_autoregressive_prefill_triton(qc, kc[:, :399], vc[:, :399], scale=sc)
    y3, _ = cf.flare_autoregressive_decode_triton(qc, kc[:, 399], vc[:, 399], st2, scale=sc)
    assert_bf16_gate(y3, ref[:, 399:], "decode after tensor-path prefill")


def test_tensor_path_segmented_small_batch():
    q, k, v = orc.make_inputs(1, 2048, 1, M, D, seed0=7, dtype=torch.bfloat16)
    ref = orc.ar_forward(q, k, v)
    y, _, _, _ = run(*to_dev(q, k, v), _lib.PATH_TENSOR)
    assert_bf16_gate(y, ref, "segmented tensor path")


def test_tensor_vs_exact_at_benchmark_size():
    # C2: B=8, N=8192, H=16, M=128, D=64.  The exact path is itself checked against the oracle on small
    # cases; here the two CUDA paths must agree at full size, and a prefix of one lane is checked on the CPU.
    B, N, H = 8, 8192, 16
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(H, M, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    y_t, _, _, _ = run(q, k, v, _lib.PATH_TENSOR)
    y_e, _, _, _ = run(q, k, v, _lib.PATH_EXACT)
    assert torch.isfinite(y_t.float()).all()
    assert_bf16_gate(y_t, y_e.float(), "tensor vs exact, C2")
    ref = orc.ar_forward(q[3:4].cpu(), k[5:6, :512, 3:4].cpu(), v[5:6, :512, 3:4].cpu())
    assert_bf16_gate(y_t[5:6, :512, 3:4], ref, "C2 lane prefix vs oracle")
    # causality: changing the last quarter of the sequence must not change earlier outputs
    k2, v2 = k.clone(), v.clone()
    k2[:, 3 * N // 4:] = 0
    v2[:, 3 * N // 4:] = 1
    y2, _, _, _ = run(q, k2, v2, _lib.PATH_TENSOR)
    assert torch.equal(y2[:, :3 * N // 4], y_t[:, :3 * N // 4])
    y3, _, _, _ = run(q, k, v, _lib.PATH_TENSOR)
    assert torch.equal(y3, y_t), "tensor path must be run-to-run deterministic"


def test_sharp_scores_forced_tensor_path_is_flagged_and_default_path_is_right():
    # scores with a standard deviation of ~64 nats: outside the tensor kernels' numeric domain.  Forcing that path
    # raises the device status; the default path (AUTO) reruns the flagged lanes on the exact kernels by itself.
    q, k, v = orc.make_inputs(1, 512, 2, M, D, seed0=13, dtype=torch.bfloat16)
    q, k = (q.float() * 8).bfloat16(), (k.float() * 8).bfloat16()
    ref = orc.ar_forward(q, k, v)
    qc, kc, vc = to_dev(q, k, v)
    _ops.device_status()
    y_t, _, _, _ = _ops.forward(qc, kc, vc, scale=D ** -0.5, path=_lib.PATH_TENSOR)
    status = _ops.device_status()
    assert status in (0, 2)
    if status == 0:
        assert_bf16_gate(y_t, ref, "sharp scores, tensor path")
    y_a = cf.flare_autoregressive_triton(qc, kc, vc)  # default environment
    assert_bf16_gate(y_a, ref, "sharp scores, default path")
    assert _ops.device_status() in (0, 2)  # the flag stays readable: it says that the exact kernels had to step in
    y_e, _, _, _ = _ops.forward(qc, kc, vc, scale=D ** -0.5, path=_lib.PATH_EXACT)
    assert _ops.device_status() == 0
    assert_bf16_gate(y_e, ref, "sharp scores, exact path")
    # in-domain inputs stay on the tensor kernels: same bits as the forced tensor path
    q2, k2, v2 = to_dev(*orc.make_inputs(1, 512, 2, M, D, seed0=14, dtype=torch.bfloat16))
    assert torch.equal(cf.flare_autoregressive_triton(q2, k2, v2),
                       _ops.forward(q2, k2, v2, scale=D ** -0.5, path=_lib.PATH_TENSOR)[0])
    assert _ops.device_status() == 0


@pytest.mark.parametrize("N", [512, 1024, 2048])
@pytest.mark.parametrize("qk_std", [4.0, 8.0])
def test_sharp_softmax_shapes_forward_and_backward_with_default_settings(N, qk_std):
    # the sharp-softmax regime (B=1, H=16, M=16, D=64; q and k scaled so that the scores have a standard deviation of
    # qk_std^2): results through the public operators with the default environment against the oracle.  The gradients
    # grow with the score scale, so their max-abs bound is taken relative to the largest reference entry.
    B, H, Ml, Dl = 1, 16, 16, 64
    q, k, v, dy = orc.make_inputs(B, N, H, Ml, Dl, seed0=31, dtype=torch.bfloat16, with_dy=True)
    q, k = (q.float() * qk_std).bfloat16(), (k.float() * qk_std).bfloat16()
    ref_y = orc.ar_forward(q, k, v)
    ref = orc.ar_backward_closed_form(q, k, v, dy)
    ql, kl, vl = (t.cuda().requires_grad_(True) for t in (q, k, v))
    y = cf.flare_autoregressive_triton(ql, kl, vl)
    # sharp decode weights pick single values: |y| reaches 4 and more, where one bf16 output step is 3.1e-2; the
    # max-abs bound is 1 % of the largest reference entry there
    assert_bf16_gate(y, ref_y, f"sharp y, std {qk_std}", max_abs=max(2e-2, 1e-2 * float(ref_y.abs().max())))
    y.backward(dy.cuda())
    for got, key in ((ql.grad, "dQ"), (kl.grad, "dK"), (vl.grad, "dV")):
        assert_bf16_gate(got, ref[key], f"sharp {key}, std {qk_std}", max_abs=2e-2 * max(1.0, float(ref[key].abs().max())))
    _ops.device_status()  # clear the informational flag for the tests that follow


@pytest.mark.parametrize("B, N, H, Ml, Dl, bs", [(2, 1024, 40, 256, 128, 1), (2, 1024, 40, 256, 128, 64),
                                                 (1, 512, 160, 128, 128, 1), (1, 1024, 16, 256, 128, 1)])
def test_sharp_scores_on_wide_heads_and_latent_groups_with_default_settings(B, N, H, Ml, Dl, bs):
    # Sharp scores (standard deviation 16) on the (128, 128) head shape, with one and two latent groups, on grids that
    # take the two-slice, the wide and the cluster-merged instance.  Three things went wrong here before the numeric
    # domain checks were tightened: a latent group whose weight mass was not a number passed as "empty" (NaN rows), a
    # read-out weight R = E a / D flushed to zero under a denominator that had grown by 2^43 inside one chunk (one
    # token off by 0.37), and the lane gates of such tokens were not raised.  Every entry is checked, per lane.
    g = torch.Generator().manual_seed(4 + N + H)
    q = (torch.randn(H, Ml, Dl, generator=g) * 4.0).bfloat16()
    k = (torch.randn(B, N, H, Dl, generator=g) * 4.0).bfloat16()
    v = torch.randn(B, N, H, Dl, generator=g).bfloat16()
    sc = Dl ** -0.5
    ref = orc.ar_forward(q, k, v, scale=sc) if bs == 1 else orc.semi_ar_forward(q, k, v, block_size=bs, scale=sc)[0]
    y = _ops.forward(*to_dev(q, k, v), scale=sc, block_size=bs)[0]  # default path
    assert torch.isfinite(y.float()).all()
    assert_bf16_gate(y, ref, "sharp scores, default path", max_abs=max(2e-2, 1e-2 * float(ref.abs().max())))
    d = y.float().cpu() - ref.float()
    assert float(d.abs().amax(dim=(1, 3)).max()) <= max(2e-2, 1e-2 * float(ref.abs().max())), "worst lane"
    _ops.device_status()  # clear the informational flag for the tests that follow


@pytest.mark.parametrize("Ml", [16, 64, 96])
def test_tensor_path_fewer_latents(Ml):
    q, k, v = orc.make_inputs(2, 333, 2, Ml, D, seed0=19, dtype=torch.bfloat16)
    sc = D ** -0.5
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    assert uses_tensor_path(qc, kc, vc)
    y, st, _, _ = run(qc, kc, vc, _lib.PATH_TENSOR, want_state=True, scale=sc)
    assert_bf16_gate(y, ref, f"tensor path M={Ml}")
    assert st["u"].shape == (2, 2, Ml, D)
    assert_close(st["m"], st_ref["m"], what="m", atol=1e-4, rtol=1e-4)
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=3e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3


@pytest.mark.parametrize("Ml, B, N, H", [(128, 1, 256, 1), (128, 2, 700, 2), (64, 2, 520, 3), (128, 1, 2048, 1)])
def test_tensor_path_wide_heads(Ml, B, N, H):
    # Dk = Dv = 128: two CTAs per lane, each with 64 value columns, latent bank in tensor memory
    Dw = 128
    q, k, v = orc.make_inputs(B, N, H, Ml, Dw, seed0=21, dtype=torch.bfloat16)
    sc = Dw ** -0.5
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    assert uses_tensor_path(qc, kc, vc)
    y, st, _, _ = run(qc, kc, vc, _lib.PATH_TENSOR, want_state=True, scale=sc)
    assert_bf16_gate(y, ref, f"tensor path D=128 M={Ml} N={N}")
    assert_close(st["m"], st_ref["m"], what="m", atol=1e-4, rtol=1e-4)
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3
    # carry-in: second half continued from the first half's state
    h = (N // 2) // 16 * 16
    _, st_a, _, _ = run(qc, kc[:, :h], vc[:, :h], _lib.PATH_TENSOR, want_state=True, scale=sc)
    y_b, _, _, _ = run(qc, kc[:, h:], vc[:, h:], _lib.PATH_TENSOR, state_in=st_a, scale=sc)
    assert_bf16_gate(y_b, ref[:, h:], "D=128 carry-in")


def test_wide_heads_training_shape_vs_exact():
    # B=4, N=4096, H=16, M=64, D=128 (training shape of the benchmark set): both CUDA paths must agree
    B, N, H, Ml, Dw = 4, 4096, 16, 64, 128
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(H, Ml, Dw, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, N, H, Dw, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, N, H, Dw, generator=g, device="cuda").bfloat16()
    y_t, _, _, _ = run(q, k, v, _lib.PATH_TENSOR, scale=Dw ** -0.5)
    y_e, _, _, _ = run(q, k, v, _lib.PATH_EXACT, scale=Dw ** -0.5)
    assert_bf16_gate(y_t, y_e.float(), "tensor vs exact, D=128 training shape")


@pytest.mark.parametrize("Ml, Dw, B, N, H", [(256, 64, 1, 256, 1), (256, 128, 2, 600, 2), (192, 64, 1, 900, 2),
                                             (512, 128, 1, 384, 1), (256, 128, 1, 4096, 1)])
def test_tensor_path_latent_groups(Ml, Dw, B, N, H):
    # more than 128 latents: one CTA per group of 128, partial read-outs merged by a second kernel
    q, k, v = orc.make_inputs(B, N, H, Ml, Dw, seed0=31, dtype=torch.bfloat16)
    sc = Dw ** -0.5
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    assert uses_tensor_path(qc, kc, vc)
    y, st, _, _ = run(qc, kc, vc, _lib.PATH_TENSOR, want_state=True, scale=sc)
    assert_bf16_gate(y, ref, f"tensor path M={Ml} D={Dw} N={N}")
    assert_close(st["m"], st_ref["m"], what="m", atol=1e-4, rtol=1e-4)
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3
    h = (N // 2) // 16 * 16
    _, st_a, _, _ = run(qc, kc[:, :h], vc[:, :h], _lib.PATH_TENSOR, want_state=True, scale=sc)
    y_b, _, _, _ = run(qc, kc[:, h:], vc[:, h:], _lib.PATH_TENSOR, state_in=st_a, scale=sc)
    assert_bf16_gate(y_b, ref[:, h:], "latent groups, carry-in")


@pytest.mark.parametrize("bs, Ml", [(32, 192), (64, 192), (32, 256), (1, 192)])
def test_latent_groups_every_lane_holds_the_gate_over_many_chunks(bs, Ml):
    # Several lanes per SM-sized grid, 20 chunks, a padded second latent group: every token's weight masses for the
    # merge of the groups come from that token's own chunk (the token group once read the decode frame of a LATER
    # chunk here, which showed as 1-2 % errors in single lanes while the whole tensor stayed near the gate)
    B, N, H, Dw = 3, 2496, 5, 128
    q, k, v = orc.make_inputs(B, N, H, Ml, Dw, seed0=33, dtype=torch.bfloat16)
    sc = Dw ** -0.5
    if bs == 1:
        ref, ld_ref = orc.ar_forward(q, k, v, scale=sc), None
    else:
        ref, ld_ref, _ = orc.semi_ar_forward(q, k, v, block_size=bs, scale=sc)
    y, _, ld, _ = run(*to_dev(q, k, v), _lib.PATH_TENSOR, block_size=bs, want_lse=True, scale=sc)
    assert_bf16_gate(y, ref, f"latent groups bs={bs} M={Ml}")
    d = y.float().cpu() - ref
    lane = (d.pow(2).sum(dim=(1, 3)) / ref.pow(2).sum(dim=(1, 3))).sqrt()
    assert float(lane.max()) <= 5e-3, f"worst lane rel-L2 {float(lane.max()):.2e}"
    if ld_ref is not None:
        assert_close(ld, ld_ref, what="LSE_dec", atol=5e-3, rtol=0)


def test_latent_groups_decode_cache_shape_vs_exact():
    # B=64, H=32, M=256, D=128 (decode benchmark's cache shape), prefix of 512 tokens, then decode continues
    B, N, H, Ml, Dw = 64, 512, 32, 256, 128
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(H, Ml, Dw, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, N + 1, H, Dw, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, N + 1, H, Dw, generator=g, device="cuda").bfloat16()
    sc = Dw ** -0.5
    y_t, st_t, _, _ = run(q, k[:, :N], v[:, :N], _lib.PATH_TENSOR, want_state=True, scale=sc)
    y_e, st_e, _, _ = run(q, k[:, :N], v[:, :N], _lib.PATH_EXACT, want_state=True, scale=sc)
    assert_bf16_gate(y_t, y_e.float(), "tensor vs exact, M=256 D=128")
    assert orc.rel_l2(st_t["u"], st_e["u"]) < 3e-3
    y1, _ = cf.flare_autoregressive_decode_triton(q, k[:, N], v[:, N], st_t, scale=sc)
    y2, _ = cf.flare_autoregressive_decode_triton(q, k[:, N], v[:, N], st_e, scale=sc)
    assert_bf16_gate(y1, y2.float(), "decode after M=256 prefill")


@pytest.mark.parametrize("bs, Ml, Dw, B, N, H", [(64, 128, 64, 1, 256, 1), (16, 128, 64, 2, 400, 2), (32, 64, 128, 1, 672, 2),
                                                 (128, 128, 64, 1, 1024, 1), (64, 256, 128, 2, 576, 2),
                                                 (32, 192, 64, 1, 4096, 1)])
def test_tensor_path_block_causal(bs, Ml, Dw, B, N, H):
    # semi-autoregressive read-out on the tensor path: y and both log normalisers against the oracle
    q, k, v = orc.make_inputs(B, N, H, Ml, Dw, seed0=41, dtype=torch.bfloat16)
    sc = Dw ** -0.5
    ref, lse_dec, lse_enc = orc.semi_ar_forward(q, k, v, block_size=bs, scale=sc)
    qc, kc, vc = to_dev(q, k, v)
    y, _, ld, le = run(qc, kc, vc, _lib.PATH_TENSOR, block_size=bs, want_lse=True, scale=sc)
    assert_bf16_gate(y, ref, f"block-causal tensor path bs={bs} M={Ml} D={Dw}")
    assert_close(le, lse_enc, what="LSE_enc", atol=2e-4, rtol=2e-4)
    assert_close(ld, lse_dec, what="LSE_dec", atol=5e-3, rtol=0)  # from bf16 operands of the read-out
    # the public API takes the same kernel
    y2, aux = cf.flare_semi_autoregressive_trition(qc, kc, vc, block_size=bs, chunk_size=16, scale=sc)
    assert torch.equal(y2, y) and torch.equal(aux["LSE_enc"], le)


@pytest.mark.parametrize("Ml, Dw", [(128, 64), (256, 128), (64, 128)])
def test_tensor_path_state_only(Ml, Dw):
    # no read-out wanted: the kernel skips R, W and the read-out MMAs and must still deliver the exact state
    q, k, v = orc.make_inputs(2, 700, 2, Ml, Dw, seed0=51, dtype=torch.bfloat16)
    sc = Dw ** -0.5
    _, st_ref = orc.ar_forward(q, k, v, scale=sc, return_state=True)
    y, st, _, _ = run(*to_dev(q, k, v), _lib.PATH_TENSOR, want_state=True, want_y=False, scale=sc)
    assert y is None
    assert_close(st["m"], st_ref["m"], what="m", atol=1e-4, rtol=1e-4)
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3


@pytest.mark.parametrize("power, Ml, Dw, B, N, H", [(2.0, 128, 64, 1, 256, 1), (1.0, 64, 128, 2, 520, 2), (3.0, 256, 128, 1, 700, 2),
                                                    (2.5, 128, 64, 2, 384, 1), (2.0, 128, 64, 1, 4096, 1)])
def test_tensor_path_stablemax(power, Ml, Dw, B, N, H):
    # stablemax encoder weights on the tensor path: no frames on the encoder side, softmax decode weights
    q, k, v = orc.make_inputs(B, N, H, Ml, Dw, seed0=61, dtype=torch.bfloat16)
    sc = Dw ** -0.5
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, variant="stablemax", power=power, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    y, st, _, _ = run(qc, kc, vc, _lib.PATH_TENSOR, variant=_lib.STABLEMAX, power=power, want_state=True, scale=sc)
    assert_bf16_gate(y, ref, f"stablemax tensor path p={power} M={Ml} D={Dw}")
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3
    y_e, _, _, _ = run(qc, kc, vc, _lib.PATH_EXACT, variant=_lib.STABLEMAX, power=power, scale=sc)
    assert_bf16_gate(y, y_e.float(), "stablemax tensor vs exact")
    h = (N // 2) // 16 * 16
    _, st_a, _, _ = run(qc, kc[:, :h], vc[:, :h], _lib.PATH_TENSOR, variant=_lib.STABLEMAX, power=power, want_state=True,
                        scale=sc)
    y_b, _, _, _ = run(qc, kc[:, h:], vc[:, h:], _lib.PATH_TENSOR, variant=_lib.STABLEMAX, power=power, state_in=st_a,
                       scale=sc)
    assert_bf16_gate(y_b, ref[:, h:], "stablemax carry-in")


@pytest.mark.parametrize("Ml, Dw", [(128, 64), (256, 128)])
def test_tensor_path_masked_prefill(Ml, Dw):
    # attention masks on the tensor path: valid tokens are compacted to the front of every row, the kernel walks
    # per-row lengths, outputs are scattered back (masked positions: y = 0, state untouched)
    B, N, H = 3, 600, 2
    q, k, v = orc.make_inputs(B, N, H, Ml, Dw, seed0=71, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(3)
    mask = torch.ones(B, N, dtype=torch.int32)
    mask[0, :137] = 0                                   # left padding
    mask[1, 400:] = 0                                   # right padding
    mask[2] = (torch.rand(N, generator=g) > 0.3).int()  # holes
    sc = Dw ** -0.5
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, attention_mask=mask, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    y, st, _, _ = run(qc, kc, vc, _lib.PATH_TENSOR, mask=mask.cuda(), want_state=True, scale=sc)
    assert_bf16_gate(y, ref, f"masked tensor prefill M={Ml}")
    assert float(y[mask.cuda() == 0].float().abs().max()) == 0.0
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3
    y_e, _, _, _ = run(qc, kc, vc, _lib.PATH_EXACT, mask=mask.cuda(), scale=sc)
    assert_bf16_gate(y, y_e.float(), "masked: tensor vs exact")
    # public API: masked prefill, then a decode step
    y2, st2 = cf.flare_autoregressive_prefill_triton(qc, kc[:, :599], vc[:, :599], scale=sc, attention_mask=mask[:, :599].cuda())
    y3, _ = cf.flare_autoregressive_decode_triton(qc, kc[:, 599], vc[:, 599], st2, scale=sc, attention_mask=mask[:, 599].cuda())
    assert_bf16_gate(y3, ref[:, 599:], "decode after masked tensor prefill")


def test_block_causal_long_context_shape_vs_exact():
    # B=2, N=65536, H=32, M=256, D=128, block 64 (the long-context benchmark shape) on one GPU: both CUDA paths must
    # agree over the whole output, a prefix of one lane is checked on the CPU, and later blocks must not leak back
    B, N, H, Ml, Dw, bs = 2, 65536, 32, 256, 128, 64
    g = torch.Generator(device="cuda").manual_seed(4)
    q = torch.randn(H, Ml, Dw, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, N, H, Dw, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, N, H, Dw, generator=g, device="cuda").bfloat16()
    sc = Dw ** -0.5
    y_t, _, ld_t, le_t = run(q, k, v, _lib.PATH_TENSOR, block_size=bs, want_lse=True, scale=sc)
    y_e, _, ld_e, le_e = run(q, k, v, _lib.PATH_EXACT, block_size=bs, want_lse=True, scale=sc)
    assert torch.isfinite(y_t.float()).all()
    assert_bf16_gate(y_t, y_e.float(), "tensor vs exact, long block-causal shape")
    assert_close(le_t, le_e, what="LSE_enc", atol=5e-4, rtol=5e-4)
    assert_close(ld_t, ld_e, what="LSE_dec", atol=5e-3, rtol=0)
    ref, _, _ = orc.semi_ar_forward(q[7:8].cpu(), k[1:2, :256, 7:8].cpu(), v[1:2, :256, 7:8].cpu(), block_size=bs, scale=sc)
    assert_bf16_gate(y_t[1:2, :256, 7:8], ref, "lane prefix vs oracle")
    k2, v2 = k.clone(), v.clone()
    k2[:, N // 2:] = 0
    v2[:, N // 2:] = 1
    y2, _, _, _ = run(q, k2, v2, _lib.PATH_TENSOR, block_size=bs, scale=sc)
    assert torch.equal(y2[:, :N // 2], y_t[:, :N // 2]), "tokens of later blocks changed earlier outputs"


@pytest.mark.parametrize("N", [1, 5, 16, 17, 127, 129])
def test_tensor_path_tiny_and_ragged_lengths(N):
    # one partial chunk, a chunk boundary, and one token past it, for the three read-out modes
    Ml, Dw = 64, 64
    q, k, v = orc.make_inputs(2, N, 2, Ml, Dw, seed0=91, dtype=torch.bfloat16)
    sc = Dw ** -0.5
    qc, kc, vc = to_dev(q, k, v)
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, return_state=True)
    y, st, _, _ = run(qc, kc, vc, _lib.PATH_TENSOR, want_state=True, scale=sc)
    assert_bf16_gate(y, ref, f"softmax N={N}")
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3
    ref_s = orc.ar_forward(q, k, v, scale=sc, variant="stablemax", power=2.0)
    y_s, _, _, _ = run(qc, kc, vc, _lib.PATH_TENSOR, variant=_lib.STABLEMAX, power=2.0, scale=sc)
    assert_bf16_gate(y_s, ref_s, f"stablemax N={N}")
    if N % 16 == 0:
        ref_b, _, _ = orc.semi_ar_forward(q, k, v, block_size=16, scale=sc)
        y_b, _, _, _ = run(qc, kc, vc, _lib.PATH_TENSOR, block_size=16, scale=sc)
        assert_bf16_gate(y_b, ref_b, f"block-causal N={N}")


@pytest.mark.parametrize("Ml, B, N, H", [(128, 2, 520, 2), (256, 1, 700, 2), (64, 1, 4096, 1)])
def test_tensor_path_mixed_head_widths(Ml, B, N, H):
    # Dk = 64 with Dv = 128: score work of the narrow instance, two value slices per lane
    Dk, Dv = 64, 128
    q, k, v = orc.make_inputs(B, N, H, Ml, Dk, Dv, seed0=101, dtype=torch.bfloat16)
    sc = Dk ** -0.5
    ref, st_ref = orc.ar_forward(q, k, v, scale=sc, return_state=True)
    qc, kc, vc = to_dev(q, k, v)
    assert uses_tensor_path(qc, kc, vc)
    y, st, _, _ = run(qc, kc, vc, _lib.PATH_TENSOR, want_state=True, scale=sc)
    assert_bf16_gate(y, ref, f"Dk=64 Dv=128 M={Ml}")
    assert_close(st["d"], st_ref["d"], what="d", atol=1e-3, rtol=2e-3)
    assert orc.rel_l2(st["u"].cpu(), st_ref["u"]) < 3e-3
    h = (N // 2) // 16 * 16
    _, st_a, _, _ = run(qc, kc[:, :h], vc[:, :h], _lib.PATH_TENSOR, want_state=True, scale=sc)
    y_b, _, _, _ = run(qc, kc[:, h:], vc[:, h:], _lib.PATH_TENSOR, state_in=st_a, scale=sc)
    assert_bf16_gate(y_b, ref[:, h:], "mixed widths carry-in")
    ref_b, _, _ = orc.semi_ar_forward(q, k[:, :512], v[:, :512], block_size=32, scale=sc)
    y_blk, _, _, _ = run(qc, kc[:, :512], vc[:, :512], _lib.PATH_TENSOR, block_size=32, scale=sc)
    assert_bf16_gate(y_blk, ref_b, "mixed widths block-causal")
