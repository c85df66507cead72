"""Cached inference for the block-causal operator is not defined by the operator API this package
mirrors (reference: causal_flare/semi_autoregressive/inference.py:1-36): both entry points raise."""

from torch import autograd


class SemiAutoRegressivePrefillFLARE(autograd.Function):
    @staticmethod
    def forward(ctx, *args, **kwargs):
        raise NotImplementedError("SemiAutoRegressivePrefillFLARE is not implemented yet.")


class SemiAutoRegressiveDecodeFLARE(autograd.Function):
    @staticmethod
    def forward(ctx, *args, **kwargs):
        raise NotImplementedError("SemiAutoRegressiveDecodeFLARE is not implemented yet.")


def flare_semi_autoregressive_prefill_trition(*args, **kwargs):
    raise NotImplementedError("flare_semi_autoregressive_prefill_trition is not implemented yet.")


def flare_semi_autoregressive_decode_trition(*args, **kwargs):
    raise NotImplementedError("flare_semi_autoregressive_decode_trition is not implemented yet.")
