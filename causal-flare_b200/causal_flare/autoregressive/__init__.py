from .training import AutoRegressiveFLARE, flare_autoregressive_triton
from .inference import flare_autoregressive_decode_triton, flare_autoregressive_prefill_triton
from .stablemax_triton import FLAREAutoregressiveStablemaxTriton, flare_autoregressive_stablemax_triton

__all__ = [
    "AutoRegressiveFLARE",
    "FLAREAutoregressiveStablemaxTriton",
    "flare_autoregressive_triton",
    "flare_autoregressive_decode_triton",
    "flare_autoregressive_prefill_triton",
    "flare_autoregressive_stablemax_triton",
]
