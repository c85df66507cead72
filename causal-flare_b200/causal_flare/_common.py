"""Helpers shared by the operator wrappers: scale default, precision-mode validation, error metrics,
CUDA-event timing for ``profile=True``."""

from __future__ import annotations

import torch

__all__ = [
    "_resolve_attn_scale", "_normalize_input_precision", "_rel_l2_err", "_max_abs_err", "_check_finite",
    "_timed", "_refresh_profile_totals",
]


def _resolve_attn_scale(scale, head_dim: int) -> float:
    """Default softmax scale: 1 for tiny heads (<= 8), else head_dim ** -0.5."""
    if scale is not None:
        return float(scale)
    return 1.0 if head_dim <= 8 else head_dim ** -0.5


def _normalize_input_precision(input_precision, allow_tf32=None) -> str:
    """Validate the Triton-era precision knob.  The B200 kernels have one numeric mode per path
    (fp32 FMAs on the exact path, bf16 operands with fp32 accumulation on the tensor path), so the
    value is checked for validity and otherwise ignored."""
    if input_precision is None:
        mode = "tf32x3" if allow_tf32 is None else ("tf32" if allow_tf32 else "ieee")
    elif isinstance(input_precision, bool):
        mode = "tf32" if input_precision else "ieee"
    else:
        mode = str(input_precision).strip().lower()
    if mode not in ("tf32", "tf32x3", "ieee"):
        raise ValueError(
            f"Unsupported input_precision={input_precision!r}. "
            "Expected one of {'tf32','tf32x3','ieee'}."
        )
    return mode


def _rel_l2_err(a: torch.Tensor, b: torch.Tensor) -> float:
    num = torch.linalg.norm((a - b).float())
    den = torch.linalg.norm(b.float())
    return (num / (den + 1e-12)).item()


def _max_abs_err(a: torch.Tensor, b: torch.Tensor) -> float:
    return (a.float() - b.float()).abs().max().item() if a.numel() else 0.0


def _check_finite(name: str, tensor: torch.Tensor) -> None:
    if not torch.isfinite(tensor).all():
        raise RuntimeError(f"FLARE numerical issue in {name}")


def _timed(device, timings, name, fn):
    """Run fn(); when ``timings`` is a dict, record one entry per kernel launch (milliseconds of device time, summed
    over repeated launches of the same kernel) and, under ``name + " (launch gaps, memsets)"``, what the CUDA events
    around the whole call measured beyond the kernels, so that the entries add up to the call's device time."""
    if timings is None:
        return fn()
    import ctypes as C

    from . import _lib

    lib = _lib.load()
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    lib.flare_profile_enable(1)
    start.record(torch.cuda.current_stream(device))
    try:
        out = fn()
    finally:
        lib.flare_profile_enable(0)
    end.record(torch.cuda.current_stream(device))
    end.synchronize()
    total = start.elapsed_time(end)
    kernels = 0.0
    kname, ms = C.c_char_p(), C.c_float()
    for i in range(lib.flare_profile_count()):
        if lib.flare_profile_entry(i, C.byref(kname), C.byref(ms)) == 0:
            key = kname.value.decode()
            timings[key] = timings.get(key, 0.0) + ms.value
            kernels += ms.value
    rest = name + " (launch gaps, memsets)"
    timings[rest] = timings.get(rest, 0.0) + max(0.0, total - kernels)
    return out


def _refresh_profile_totals(profile_data: dict) -> None:
    fwd = sum(v for v in profile_data.get("forward", {}).values() if isinstance(v, (int, float)))
    bwd = sum(v for v in profile_data.get("backward", {}).values() if isinstance(v, (int, float)))
    profile_data["forward_total_ms"] = fwd
    profile_data["backward_total_ms"] = bwd
    profile_data["total_ms"] = fwd + bwd
