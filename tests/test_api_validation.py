"""CPU: argument validation of the public operators (same exception types and message fragments as the
operator API they replace; the reference pins these in testing/autoregressive/test_flare.py:493-517 and
testing/semi_autoregressive/test_block_causal.py:18-41, :260-275)."""
import pytest
import torch

import causal_flare as cf
from causal_flare._common import _normalize_input_precision, _resolve_attn_scale
from causal_flare._reference_utils import resolve_flare_causal_decode_inputs, validate_flare_qkv_layouts
from causal_flare.autoregressive import flare_autoregressive_stablemax_triton
from causal_flare.autoregressive.inference import _canonicalize_flare_state
from causal_flare.semi_autoregressive.reference import _validate_block_causal_config


def qkv(B=1, N=32, H=2, M=16, D=16):
    return torch.randn(H, M, D), torch.randn(B, N, H, D), torch.randn(B, N, H, D)


def test_scale_default():
    assert _resolve_attn_scale(None, 8) == 1.0
    assert _resolve_attn_scale(None, 64) == 64 ** -0.5
    assert _resolve_attn_scale(0.3, 64) == pytest.approx(0.3)


def test_input_precision_values():
    for ok in ("ieee", "tf32", "TF32x3", None, True, False):
        _normalize_input_precision(ok)
    with pytest.raises(ValueError, match="Unsupported input_precision"):
        _normalize_input_precision("fp8")


def test_layout_validation_messages():
    q, k, v = qkv()
    assert validate_flare_qkv_layouts(q, k, v, name="x") == (1, 32, 2, 16, 16, 16)
    with pytest.raises(ValueError, match="expects Q \\[H, M, D_k\\]"):
        validate_flare_qkv_layouts(q[0], k, v, name="x")
    with pytest.raises(ValueError, match="agree on \\[B, N, H\\]"):
        validate_flare_qkv_layouts(q, k, v[:, :5], name="x")
    with pytest.raises(ValueError, match="matching H,D_k"):
        validate_flare_qkv_layouts(q[:1], k, v, name="x")


def test_decode_alias_rule_is_by_identity():
    q, k, v = qkv()
    assert resolve_flare_causal_decode_inputs(q, k)[2:] == (False, False, True)
    assert resolve_flare_causal_decode_inputs(q, k, k, q)[2:] == (True, True, True)
    assert resolve_flare_causal_decode_inputs(q, k, k.clone(), None)[2:] == (True, False, False)
    assert resolve_flare_causal_decode_inputs(q, k, None, q.clone())[2:] == (False, True, False)
    with pytest.raises(ValueError, match="Q_dec and K_enc must have the same shape"):
        resolve_flare_causal_decode_inputs(q, k, k[:, :3], None)
    with pytest.raises(ValueError, match="Expected K_dec \\[H, M, D\\]"):
        resolve_flare_causal_decode_inputs(q, k, None, q[0])


def test_ar_forward_asserts():
    q, k, v = qkv()
    with pytest.raises(AssertionError, match="3D and 4D"):
        cf.flare_autoregressive_triton(q[0], k, v)
    with pytest.raises(AssertionError, match="agree on \\[B, N, H\\]"):
        cf.flare_autoregressive_triton(q, k, v[:, :3])
    with pytest.raises(AssertionError, match="M must be divisible by 16"):
        cf.flare_autoregressive_triton(q[:, :8], k, v)
    with pytest.raises(AssertionError, match="CHUNK_SIZE must be divisible by 16"):
        cf.flare_autoregressive_triton(q, k, v, chunk_size=24)


def test_block_causal_config_messages():
    ok = _validate_block_causal_config(N=128, block_size=32, chunk_size=16, name="x")
    assert ok == (32, 16, 4, 8, 2)
    cases = [
        (dict(N=128, block_size=None, chunk_size=16), "requires block_size to be specified explicitly"),
        (dict(N=128, block_size=32, chunk_size=None), "requires chunk_size to be specified explicitly"),
        (dict(N=128, block_size=0, chunk_size=16), "requires block_size > 0"),
        (dict(N=128, block_size=24, chunk_size=16), "positive multiple of 16"),
        (dict(N=128, block_size=32, chunk_size=48), "currently supports chunk_size in"),
        (dict(N=100, block_size=32, chunk_size=16), "exact multiple of block_size"),
        (dict(N=128, block_size=32, chunk_size=64), "integer multiple of chunk_size"),
    ]
    for kw, msg in cases:
        with pytest.raises(ValueError, match=msg):
            _validate_block_causal_config(name="x", **kw)
    q, k, v = qkv(N=100)
    with pytest.raises(ValueError, match="exact multiple of block_size"):
        cf.flare_semi_autoregressive_trition(q, k, v, block_size=32, chunk_size=16)
    with pytest.raises(TypeError):
        cf.flare_semi_autoregressive_trition(q, k, v)  # block_size / chunk_size are required keywords


def test_semi_ar_inference_entry_points_raise():
    # same calls and messages as the reference's own tests (testing/semi_autoregressive/test_block_causal.py:260-275)
    q, k, v = torch.randn(2, 4, 16), torch.randn(1, 8, 2, 16), torch.randn(1, 8, 2, 16)
    with pytest.raises(NotImplementedError, match="not implemented yet"):
        cf.flare_semi_autoregressive_prefill_trition(q, k, v)
    with pytest.raises(NotImplementedError, match="not implemented yet"):
        cf.flare_semi_autoregressive_decode_trition(q, k[:, 0], v[:, 0])
    with pytest.raises(TypeError):
        cf.flare_semi_autoregressive_prefill_trition(q, k, v, None)  # the options are keyword-only, as in the reference


def test_stablemax_unsupported_options():
    q, k, v = qkv()
    for kw in (dict(eps=1e-6), dict(profile=True), dict(state={}), dict(attention_mask=torch.ones(1, 32)),
               dict(return_state=True), dict(write_gate=True)):
        with pytest.raises(NotImplementedError):
            flare_autoregressive_stablemax_triton(q, k, v, **kw)


def test_state_validation():
    dev = torch.device("cpu")
    st = _canonicalize_flare_state(None, 2, 3, 16, 32, dev)
    assert st["m"].shape == (2, 3, 16) and bool(torch.isinf(st["m"]).all()) and st["u"].shape == (2, 3, 16, 32)
    with pytest.raises(ValueError, match="must be a dict"):
        _canonicalize_flare_state([1], 2, 3, 16, 32, dev)
    with pytest.raises(ValueError, match="Invalid FLARE recurrent state keys"):
        _canonicalize_flare_state({"m": st["m"]}, 2, 3, 16, 32, dev)
    with pytest.raises(ValueError, match="Invalid FLARE recurrent state shapes"):
        _canonicalize_flare_state(st, 2, 3, 16, 16, dev)
    same = _canonicalize_flare_state(st, 2, 3, 16, 32, dev)
    assert same["u"].data_ptr() == st["u"].data_ptr()  # fp32 state is used in place


def test_recurrent_requires_equal_kv_shapes():
    q, k, v = qkv()
    with pytest.raises(ValueError, match="K and V must have the same shape"):
        cf.flare_recurrent_triton(q, k, torch.randn(1, 32, 2, 32))
