from .training import SemiAutoRegressiveFLARE, flare_semi_autoregressive_trition
from .inference import (
    SemiAutoRegressiveDecodeFLARE,
    SemiAutoRegressivePrefillFLARE,
    flare_semi_autoregressive_decode_trition,
    flare_semi_autoregressive_prefill_trition,
)

__all__ = [
    "SemiAutoRegressiveDecodeFLARE",
    "SemiAutoRegressiveFLARE",
    "SemiAutoRegressivePrefillFLARE",
    "flare_semi_autoregressive_decode_trition",
    "flare_semi_autoregressive_prefill_trition",
    "flare_semi_autoregressive_trition",
]
