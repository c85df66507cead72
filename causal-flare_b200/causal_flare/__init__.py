"""Causal FLARE attention for NVIDIA B200: drop-in for the `causal_flare` operator API.

Same function names, argument shapes, return values and autograd behaviour as the Triton package
it replaces; the work is done by hand-written sm_100a CUDA kernels in libflare_b200.so, reached
through a C ABI.  There is no Triton, no alternative backend and no CPU fallback.
"""

from . import autoregressive, semi_autoregressive
from .autoregressive.training import flare_autoregressive_triton
from .autoregressive.inference import (
    flare_autoregressive_decode_triton,
    flare_autoregressive_prefill_triton,
)
from .autoregressive.recurrent import flare_recurrent_triton
from .semi_autoregressive.training import flare_semi_autoregressive_trition
from .semi_autoregressive.inference import (
    flare_semi_autoregressive_decode_trition,
    flare_semi_autoregressive_prefill_trition,
)

__version__ = "0.0.1"

__all__ = [
    "autoregressive",
    "semi_autoregressive",
    "flare_autoregressive_triton",
    "flare_autoregressive_decode_triton",
    "flare_autoregressive_prefill_triton",
    "flare_recurrent_triton",
    "flare_semi_autoregressive_decode_trition",
    "flare_semi_autoregressive_prefill_trition",
    "flare_semi_autoregressive_trition",
    "__version__",
]
