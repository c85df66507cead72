"""Configuration rules of the block-causal operator (reference: causal_flare/semi_autoregressive/reference.py:17-51)."""

from __future__ import annotations

import math

_SUPPORTED_BLOCK_CAUSAL_CHUNK_SIZES = (16, 32, 64, 128)


def _validate_block_causal_config(*, N: int, block_size, chunk_size, name: str):
    if block_size is None:
        raise ValueError(f"{name} requires block_size to be specified explicitly.")
    if chunk_size is None:
        raise ValueError(f"{name} requires chunk_size to be specified explicitly.")
    block_size = int(block_size)
    chunk_size = int(chunk_size)
    if block_size <= 0:
        raise ValueError(f"{name} requires block_size > 0. Got block_size={block_size}.")
    if block_size % 16 != 0:
        raise ValueError(f"{name} requires block_size to be a positive multiple of 16. Got block_size={block_size}.")
    if chunk_size not in _SUPPORTED_BLOCK_CAUSAL_CHUNK_SIZES:
        raise ValueError(
            f"{name} currently supports chunk_size in {_SUPPORTED_BLOCK_CAUSAL_CHUNK_SIZES}. "
            f"Got chunk_size={chunk_size}."
        )
    if N % block_size != 0:
        raise ValueError(
            f"{name} requires sequence length N to be an exact multiple of block_size. "
            f"Got N={N}, block_size={block_size}."
        )
    if block_size % chunk_size != 0:
        raise ValueError(
            f"{name} requires block_size to be an integer multiple of chunk_size so blocks align with chunk summaries. "
            f"Got block_size={block_size}, chunk_size={chunk_size}."
        )
    num_blocks = math.ceil(N / block_size) if N > 0 else 0
    num_chunks = math.ceil(N / chunk_size) if N > 0 else 0
    return block_size, chunk_size, num_blocks, num_chunks, block_size // chunk_size
