"""ctypes binding of libflare_b200.so (the C ABI declared in include/flare_b200.h).

There is no fallback: if the shared library is missing or a kernel reports an error the
call raises.  Build the library with ``python causal-flare_b200/build.py``.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FLARE_B200_LIB") or os.path.join(os.path.dirname(_HERE), "libflare_b200.so")

F32, BF16, F16 = 0, 1, 2
SOFTMAX, STABLEMAX = 0, 1
PATH_AUTO, PATH_EXACT, PATH_TENSOR = 0, 1, 2

_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


class State(C.Structure):
    _fields_ = [("m", C.c_void_p), ("d", C.c_void_p), ("u", C.c_void_p)]


class FwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("q_dec", C.c_void_p), ("k_dec", C.c_void_p),
        ("y", C.c_void_p), ("mask", C.c_void_p), ("lengths", C.c_void_p),
        ("state_in", State), ("state_out", State),
        ("lse_dec", C.c_void_p), ("lse_enc", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("B", C.c_int32), ("N", C.c_int32), ("H", C.c_int32), ("M", C.c_int32), ("Dk", C.c_int32), ("Dv", C.c_int32),
        ("q_stride_h", C.c_int64), ("q_stride_m", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_n", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_n", C.c_int64), ("v_stride_h", C.c_int64),
        ("qd_stride_b", C.c_int64), ("qd_stride_n", C.c_int64), ("qd_stride_h", C.c_int64),
        ("kd_stride_h", C.c_int64), ("kd_stride_m", C.c_int64),
        ("y_stride_b", C.c_int64), ("y_stride_n", C.c_int64), ("y_stride_h", C.c_int64),
        ("scale", C.c_float), ("power", C.c_float),
        ("dtype", C.c_int32), ("variant", C.c_int32), ("block_size", C.c_int32), ("path", C.c_int32),
        ("keep", C.c_void_p), ("keep_bytes", C.c_size_t),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("fwd", FwdArgs),
        ("dy", C.c_void_p),
        ("dy_stride_b", C.c_int64), ("dy_stride_n", C.c_int64), ("dy_stride_h", C.c_int64),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("dq_dec", C.c_void_p), ("dk_dec", C.c_void_p),
        ("carry_b", C.c_void_p), ("carry_c", C.c_void_p), ("carry_rho", C.c_void_p),
        ("span_b0", C.c_void_p), ("span_c0", C.c_void_p), ("span_gam", C.c_void_p), ("span_rho_first", C.c_void_p),
        ("phase", C.c_int32),
        ("y", C.c_void_p), ("y_stride_b", C.c_int64), ("y_stride_n", C.c_int64), ("y_stride_h", C.c_int64),
        ("lse_dec", C.c_void_p),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("q_dec", C.c_void_p), ("k_dec", C.c_void_p),
        ("y", C.c_void_p), ("mask", C.c_void_p), ("state", State),
        ("B", C.c_int32), ("H", C.c_int32), ("M", C.c_int32), ("Dk", C.c_int32), ("Dv", C.c_int32),
        ("q_stride_h", C.c_int64), ("q_stride_m", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_h", C.c_int64),
        ("qd_stride_b", C.c_int64), ("qd_stride_h", C.c_int64),
        ("kd_stride_h", C.c_int64), ("kd_stride_m", C.c_int64),
        ("scale", C.c_float), ("dtype", C.c_int32),
    ]


EXPORTS = (
    "flare_forward_workspace_bytes", "flare_forward", "flare_forward_keep_bytes", "flare_backward_workspace_bytes",
    "flare_backward",
    "flare_decode_step", "flare_state_merge", "flare_status_string", "flare_last_cuda_error",
    "flare_abi_version", "flare_abi_sizeof", "flare_set_kernel_events", "flare_last_launch_count",
    "flare_forward_uses_tensor_path", "flare_backward_uses_tensor_path", "flare_device_status", "flare_set_trace_buffer",
    "flare_forward_noalloc", "flare_noalloc_scratch_capacity",
    "flare_profile_enable", "flare_profile_count", "flare_profile_entry",
)

_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it is absent or its struct layouts differ from ours."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"libflare_b200.so not found at {LIB_PATH}. Build it with `python causal-flare_b200/build.py` "
            "(needs nvcc with sm_100a support). There is no fallback implementation."
        )
    lib = C.CDLL(LIB_PATH)
    lib.flare_forward_workspace_bytes.restype = C.c_size_t
    lib.flare_forward_workspace_bytes.argtypes = [C.POINTER(FwdArgs)]
    lib.flare_forward_keep_bytes.restype = C.c_size_t
    lib.flare_forward_keep_bytes.argtypes = [C.POINTER(FwdArgs)]
    lib.flare_forward.restype = C.c_int
    lib.flare_forward.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
    lib.flare_backward_workspace_bytes.restype = C.c_size_t
    lib.flare_backward_workspace_bytes.argtypes = [C.POINTER(BwdArgs)]
    lib.flare_backward.restype = C.c_int
    lib.flare_backward.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
    lib.flare_decode_step.restype = C.c_int
    lib.flare_decode_step.argtypes = [C.POINTER(DecodeArgs), C.c_void_p]
    lib.flare_state_merge.restype = C.c_int
    lib.flare_state_merge.argtypes = [C.POINTER(State), C.POINTER(State), C.POINTER(State), C.c_int64, C.c_int32,
                                      C.c_int32, C.c_int32, C.c_void_p]
    lib.flare_status_string.restype = C.c_char_p
    lib.flare_status_string.argtypes = [C.c_int]
    lib.flare_last_cuda_error.restype = C.c_char_p
    lib.flare_abi_version.restype = C.c_int
    lib.flare_set_kernel_events.restype = None
    lib.flare_set_kernel_events.argtypes = [C.c_void_p, C.c_void_p]
    lib.flare_last_launch_count.restype = C.c_int
    lib.flare_forward_uses_tensor_path.restype = C.c_int
    lib.flare_forward_uses_tensor_path.argtypes = [C.POINTER(FwdArgs)]
    lib.flare_backward_uses_tensor_path.restype = C.c_int
    lib.flare_backward_uses_tensor_path.argtypes = [C.POINTER(BwdArgs)]
    lib.flare_device_status.restype = C.c_int
    lib.flare_forward_noalloc.restype = C.c_int
    lib.flare_forward_noalloc.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
    lib.flare_noalloc_scratch_capacity.restype = C.c_size_t
    lib.flare_profile_enable.restype = None
    lib.flare_profile_enable.argtypes = [C.c_int]
    lib.flare_profile_count.restype = C.c_int
    lib.flare_profile_entry.restype = C.c_int
    lib.flare_profile_entry.argtypes = [C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_float)]
    lib.flare_set_trace_buffer.restype = None
    lib.flare_set_trace_buffer.argtypes = [C.c_void_p]
    lib.flare_device_status.argtypes = [C.c_int]
    lib.flare_abi_sizeof.restype = C.c_size_t
    lib.flare_abi_sizeof.argtypes = [C.c_int]
    for which, struct in enumerate((FwdArgs, BwdArgs, DecodeArgs, State)):
        if lib.flare_abi_sizeof(which) != C.sizeof(struct):
            raise RuntimeError(
                f"ABI mismatch for {struct.__name__}: library {lib.flare_abi_sizeof(which)} bytes, "
                f"binding {C.sizeof(struct)} bytes"
            )
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status == 0:
        return
    lib = load()
    msg = lib.flare_status_string(status).decode()
    if status == 7:
        msg += ": " + lib.flare_last_cuda_error().decode()
    exc = RuntimeError if status in (4, 7) else ValueError
    raise exc(f"{what} failed: {msg} (status {status})")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"FLARE kernels support float32, bfloat16 and float16 inputs. Got {dtype}.") from None


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_handle(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def kernel_ready(t: torch.Tensor) -> torch.Tensor:
    """Return ``t`` if the kernels can read it in place (inner dim contiguous, 16-byte aligned rows), else a dense copy."""
    if t.numel() == 0:
        return t
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def state_struct(st) -> State:
    if st is None:
        return State(None, None, None)
    return State(st["m"].data_ptr(), st["d"].data_ptr(), st["u"].data_ptr())


def make_fwd_args(q, k, v, q_dec, k_dec, y, *, scale, variant=SOFTMAX, power=2.0, block_size=1, mask=None,
                  state_in=None, state_out=None, lse_dec=None, lse_enc=None, path=PATH_AUTO, lengths=None) -> FwdArgs:
    """q [H,M,Dk]; k, v, q_dec, y given as [B,N,H,D] views (any b/n/h strides)."""
    B, N, H, Dk = k.shape
    a = FwdArgs()
    a.q, a.k, a.v, a.q_dec, a.k_dec, a.y = ptr(q), ptr(k), ptr(v), ptr(q_dec), ptr(k_dec), ptr(y)
    a.mask = ptr(mask)
    a.lengths = ptr(lengths)
    a.state_in = state_struct(state_in)
    a.state_out = state_struct(state_out)
    a.lse_dec, a.lse_enc = ptr(lse_dec), ptr(lse_enc)
    a.B, a.N, a.H, a.M, a.Dk, a.Dv = B, N, H, q.shape[1], Dk, v.shape[-1]
    a.q_stride_h, a.q_stride_m = q.stride(0), q.stride(1)
    a.k_stride_b, a.k_stride_n, a.k_stride_h = k.stride(0), k.stride(1), k.stride(2)
    a.v_stride_b, a.v_stride_n, a.v_stride_h = v.stride(0), v.stride(1), v.stride(2)
    if q_dec is not None:
        a.qd_stride_b, a.qd_stride_n, a.qd_stride_h = q_dec.stride(0), q_dec.stride(1), q_dec.stride(2)
    if k_dec is not None:
        a.kd_stride_h, a.kd_stride_m = k_dec.stride(0), k_dec.stride(1)
    if y is not None:
        a.y_stride_b, a.y_stride_n, a.y_stride_h = y.stride(0), y.stride(1), y.stride(2)
    a.scale, a.power = float(scale), float(power)
    a.dtype = dtype_code(k.dtype)
    a.variant, a.block_size, a.path = int(variant), int(block_size), int(path)
    return a


def run_forward(args: FwdArgs, device) -> None:
    lib = load()
    need = lib.flare_forward_workspace_bytes(C.byref(args))
    ws = None
    if need:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        args.workspace, args.workspace_bytes = ws.data_ptr(), need
    check(lib.flare_forward(C.byref(args), stream_handle(device)), "flare_forward")
    # `ws` is stream-ordered torch memory: safe to release after the launches are enqueued.


def run_backward(args: BwdArgs, device) -> None:
    lib = load()
    need = lib.flare_backward_workspace_bytes(C.byref(args))
    ws = None
    if need:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        args.fwd.workspace, args.fwd.workspace_bytes = ws.data_ptr(), need
    check(lib.flare_backward(C.byref(args), stream_handle(device)), "flare_backward")
