"""CPU: the shared library loads, exports every symbol the public header declares, agrees with the
ctypes struct layouts, and rejects malformed problems with the documented status codes.  No kernel runs."""
import ctypes as C
import os
import re

import pytest
import torch

from causal_flare import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names.update(re.findall(r"\b(flare_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_declares_the_bound_entry_points():
    decl = declared_functions()
    for name in _lib.EXPORTS:
        assert name in decl, f"{name} is bound by the Python shim but not declared in include/"


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"libflare_b200.so does not export {name}"
    assert lib.flare_abi_version() >= 1


def test_struct_layouts_match():
    lib = _lib.load()
    for which, struct in enumerate((_lib.FwdArgs, _lib.BwdArgs, _lib.DecodeArgs, _lib.State)):
        assert lib.flare_abi_sizeof(which) == C.sizeof(struct)
    assert lib.flare_abi_sizeof(99) == 0


def _fake_args(B=2, N=64, H=2, M=32, Dk=32, Dv=32, **kw):
    a = _lib.FwdArgs()
    a.q = a.k = a.v = a.y = 0x1000  # never dereferenced: validation and planning only
    a.B, a.N, a.H, a.M, a.Dk, a.Dv = B, N, H, M, Dk, Dv
    a.q_stride_h, a.q_stride_m = M * Dk, Dk
    a.k_stride_b, a.k_stride_n, a.k_stride_h = N * H * Dk, H * Dk, Dk
    a.v_stride_b, a.v_stride_n, a.v_stride_h = N * H * Dv, H * Dv, Dv
    a.y_stride_b, a.y_stride_n, a.y_stride_h = N * H * Dv, H * Dv, Dv
    a.scale, a.power, a.dtype, a.variant, a.block_size = 1.0, 2.0, _lib.BF16, _lib.SOFTMAX, 1
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_status_strings():
    lib = _lib.load()
    assert lib.flare_status_string(0) == b"ok"
    seen = {lib.flare_status_string(i) for i in range(9)}
    assert len(seen) == 9
    assert b"unknown" in lib.flare_status_string(1234)


@pytest.mark.parametrize(
    "kw, status",
    [
        (dict(M=24), 1),            # not a multiple of 16
        (dict(Dk=0), 1),
        (dict(dtype=7), 5),
        (dict(variant=3), 6),
        (dict(block_size=0), 6),
        (dict(block_size=48), 6),   # does not divide N=64
        (dict(block_size=32, variant=_lib.STABLEMAX), 6),
        (dict(q=None), 3),
        (dict(k=0x1004), 3),        # misaligned
        (dict(k_stride_n=33), 3),
        (dict(M=1024), 2),
    ],
)
def test_forward_rejects_bad_problems(kw, status):
    lib = _lib.load()
    a = _fake_args(**kw)
    assert lib.flare_forward(C.byref(a), None) == status
    assert lib.flare_forward_workspace_bytes(C.byref(a)) == 0


def test_workspace_plan_small_batch_is_segmented():
    lib = _lib.load()
    few = _fake_args(B=1, N=8192, H=2, M=64, Dk=64, Dv=64)
    many = _fake_args(B=8, N=8192, H=64, M=64, Dk=64, Dv=64)
    assert lib.flare_forward_workspace_bytes(C.byref(few)) > 0
    # many lanes: no segment states; the default path only asks for its gate words (1 + lanes ints, rounded to 256 B)
    assert lib.flare_forward_workspace_bytes(C.byref(many)) == (4 * (1 + 8 * 64) + 255) // 256 * 256
    many.path = _lib.PATH_TENSOR
    assert lib.flare_forward_workspace_bytes(C.byref(many)) == 0
    many.path = _lib.PATH_EXACT
    assert lib.flare_forward_workspace_bytes(C.byref(many)) == 0
    # too-small workspace is refused before anything is launched
    few.workspace, few.workspace_bytes = 0x2000, 16
    assert lib.flare_forward(C.byref(few), None) == 4


def test_fp16_plan_takes_the_tensor_path_through_bf16_copies():
    lib = _lib.load()
    B, N, H, M, D = 8, 8192, 64, 64, 64
    bf = _fake_args(B=B, N=N, H=H, M=M, Dk=D, Dv=D, path=_lib.PATH_TENSOR)
    hf = _fake_args(B=B, N=N, H=H, M=M, Dk=D, Dv=D, path=_lib.PATH_TENSOR, dtype=_lib.F16)
    assert lib.flare_forward_uses_tensor_path(C.byref(bf)) == 1
    assert lib.flare_forward_uses_tensor_path(C.byref(hf)) == 1
    # bf16 copies of q, k, v and a bf16 y (each rounded up to 256 bytes) on top of the bf16 plan
    copies = (H * M * D * 2 + 255) // 256 * 256 + 3 * (B * N * H * D * 2)
    assert lib.flare_forward_workspace_bytes(C.byref(hf)) == lib.flare_forward_workspace_bytes(C.byref(bf)) + copies
    hf.workspace, hf.workspace_bytes = 0x2000, copies - 256
    assert lib.flare_forward(C.byref(hf), None) == 4  # too small: refused before any launch
    # the exact kernels read fp16 directly; the training forward and separate decode weights stay on them
    assert lib.flare_forward_keep_bytes(C.byref(hf)) == 0
    for kw in (dict(path=_lib.PATH_EXACT), dict(q_dec=0x1000, qd_stride_b=N * H * D, qd_stride_n=H * D, qd_stride_h=D),
               dict(Dk=32, Dv=32)):
        other = _fake_args(B=B, N=N, H=H, M=M, **{"Dk": D, "Dv": D, "dtype": _lib.F16, **kw})
        assert lib.flare_forward_uses_tensor_path(C.byref(other)) == 0


def test_decode_and_merge_reject_bad_problems():
    lib = _lib.load()
    d = _lib.DecodeArgs()
    assert lib.flare_decode_step(C.byref(d), None) == 1
    d.B, d.H, d.M, d.Dk, d.Dv, d.dtype = 2, 2, 32, 32, 32, _lib.BF16
    assert lib.flare_decode_step(C.byref(d), None) == 3
    s = _lib.State(None, None, None)
    assert lib.flare_state_merge(C.byref(s), C.byref(s), C.byref(s), 4, 32, 32, 1, None) == 3


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_cpu_tensors_are_refused():
    import causal_flare as cf

    q, k, v = torch.randn(2, 16, 16), torch.randn(1, 8, 2, 16), torch.randn(1, 8, 2, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        cf.flare_autoregressive_triton(q, k, v)
    with pytest.raises(RuntimeError, match="CUDA"):
        cf.flare_autoregressive_prefill_triton(q, k, v)
    with pytest.raises(RuntimeError, match="CUDA"):
        cf.flare_autoregressive_decode_triton(q, k[:, 0], v[:, 0])
    with pytest.raises(RuntimeError, match="CUDA"):
        cf.flare_recurrent_triton(q, k, v)
    with pytest.raises(RuntimeError, match="CUDA"):
        cf.flare_semi_autoregressive_trition(q, torch.randn(1, 16, 2, 16), torch.randn(1, 16, 2, 16), block_size=16, chunk_size=16)
