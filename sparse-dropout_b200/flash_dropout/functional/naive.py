"""Masked-dense blockwise dropout + matmul in plain PyTorch (the reference's ``blockwise[naive]`` variant,
flash_dropout/functional/naive.py).  It is selected only by name; the sm_100a path never falls back to it.
"""
from __future__ import annotations

from math import ceil

import torch
import torch.nn.functional as F

from .utils import blockwise_dropout_mask


def blockwise_dropout_matmul_mask(input: torch.Tensor, mask: torch.Tensor, block_size: int, p: float,
                                  weight: torch.Tensor) -> torch.Tensor:
    """``F.linear(keep o input / (1 - p), weight)`` with ``mask`` True = dropped (naive.py:8-25)."""
    assert 0 <= p < 1, "Dropout probability must be in [0, 1)"
    M, K = input.shape
    bm, bk = block_size if isinstance(block_size, (tuple, list)) else (block_size, block_size)
    if tuple(mask.shape) != (ceil(M / bm), ceil(K / bk)):
        raise RuntimeError(f"mask shape {tuple(mask.shape)} does not match input {tuple(input.shape)}")
    keep = (~mask).to(input.dtype) / (1 - p)
    keep = keep.repeat_interleave(bm, 0).repeat_interleave(bk, 1)[:M, :K]
    return F.linear(input * keep, weight)


def blockwise_dropout_matmul(input: torch.Tensor, weight: torch.Tensor, block_size: int, p: float):
    mask = blockwise_dropout_mask(input, block_size, p)
    return blockwise_dropout_matmul_mask(input, mask, block_size, p, weight)
