"""GPU: flare_forward_noalloc, the forward entry point for callers that must not allocate device memory (a serving
loop that owns all GPU memory through its own pool, a plugin running inside another framework's allocator hook, a
binding without an allocator for workspaces).  It must give exactly what flare_forward gives with a caller-provided
workspace - here on problems that really use the scratch (few lanes, long sequence: segment-state scan) - on two
calls in a row, because every call reuses the same built-in scratch array."""
import ctypes as C

import pytest
import torch

from causal_flare import _lib
from oracle import flare_oracle as orc

pytestmark = pytest.mark.gpu


def _problem(dtype, B, N, H, M, D):
    q, k, v = orc.make_inputs(B, N, H, M, D, seed0=77, dtype=dtype)
    return q.cuda(), k.cuda(), v.cuda()


def _run(entry, q, k, v, with_workspace, check_free=False):
    lib = _lib.load()
    y = torch.full_like(v, float("nan"))
    st = {"m": torch.empty(v.shape[0], v.shape[2], q.shape[1], device="cuda"),
          "d": torch.empty(v.shape[0], v.shape[2], q.shape[1], device="cuda"),
          "u": torch.empty(v.shape[0], v.shape[2], q.shape[1], v.shape[3], device="cuda")}
    args = _lib.make_fwd_args(q, k, v, None, None, y, scale=q.shape[-1] ** -0.5, state_out=st)
    need = lib.flare_forward_workspace_bytes(C.byref(args))
    assert need > 0, "the test problem must be one that uses scratch memory"
    ws = None
    if with_workspace:
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        args.workspace, args.workspace_bytes = ws.data_ptr(), need
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]  # what the driver reports: sees any allocation, not just torch's
    rc = getattr(lib, entry)(C.byref(args), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.flare_status_string(rc)
    torch.cuda.synchronize()
    if check_free:
        assert torch.cuda.mem_get_info()[0] >= free_before, "the call allocated device memory"
    return y, st


@pytest.mark.parametrize("dtype, shape", [(torch.float32, (1, 2048, 1, 32, 32)),      # exact path, segmented
                                          (torch.bfloat16, (1, 4096, 2, 128, 64))])   # tensor-core path, segmented
def test_noalloc_matches_flare_forward_twice(dtype, shape):
    q, k, v = _problem(dtype, *shape)
    y_ref, st_ref = _run("flare_forward", q, k, v, with_workspace=True)
    assert torch.isfinite(y_ref.float()).all()
    for call in range(2):
        before = torch.cuda.memory_allocated()
        # free device memory as the driver reports it is compared around the second call: the first one may still
        # load the library's code and its built-in scratch array onto the device (lazy module loading)
        y, st = _run("flare_forward_noalloc", q, k, v, with_workspace=False, check_free=call > 0)
        assert torch.equal(y, y_ref), f"call {call}: output differs from flare_forward"
        for key in "mdu":
            assert torch.equal(st[key], st_ref[key]), f"call {call}: state {key} differs"
        del y, st
        assert torch.cuda.memory_allocated() == before
    # a different problem in between must not disturb the next call (the scratch keeps stale contents)
    q2, k2, v2 = _problem(torch.float32, 1, 1024, 2, 16, 16)
    _run("flare_forward_noalloc", q2, k2, v2, with_workspace=False)
    y3, _ = _run("flare_forward_noalloc", q, k, v, with_workspace=False)
    assert torch.equal(y3, y_ref)


def test_noalloc_rejects_problems_beyond_its_capacity():
    lib = _lib.load()
    cap = lib.flare_noalloc_scratch_capacity()
    assert cap == 8 << 20
    q, k, v = _problem(torch.bfloat16, 1, 65536, 4, 512, 16)
    vbig = torch.zeros(1, 65536, 4, 512, dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(vbig)
    args = _lib.make_fwd_args(q, k, vbig, None, None, y, scale=0.25)
    need = lib.flare_forward_workspace_bytes(C.byref(args))
    assert need > cap
    y.fill_(7.0)
    assert lib.flare_forward_noalloc(C.byref(args), torch.cuda.current_stream().cuda_stream) == 8  # FLARE_ERR_TOO_LARGE
    torch.cuda.synchronize()
    assert bool((y == 7.0).all()), "a rejected call must not launch anything"
    assert b"capacity" in lib.flare_status_string(8)
