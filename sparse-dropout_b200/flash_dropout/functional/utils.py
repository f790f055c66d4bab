"""Mask and index-list helpers of the operator API (reference: flash_dropout/functional/utils.py)."""
from __future__ import annotations

from math import ceil

import torch


def blockwise_dropout_mask(x: torch.Tensor, block_size: int, p: float) -> torch.Tensor:
    """Bernoulli(p) drop mask (True = dropped) per ``block_size`` x ``block_size`` block of the last two dims
    (``block_size`` may also be an ``(m, k)`` pair, the form of eval/mlp/config.py:23-27).

    Same shape rule and polarity as flash_dropout/functional/utils.py:11-16.  For a 2-D CUDA tensor the
    mask is drawn on the device by the Philox plan kernel; otherwise by ``torch.rand`` as in the reference.
    """
    *b, m, k = x.shape
    bm, bk = block_size if isinstance(block_size, (tuple, list)) else (block_size, block_size)
    if x.is_cuda and not b and bm % 128 == 0 and bk % 128 == 0:
        from flash_dropout.cuda.binding_gemm import BlockPlan
        # the next mask of the stream (host- or device-side counter, so that a captured step draws afresh on replay)
        return BlockPlan.draw(m, k, block_size, p, x.device).mask
    shape = (*b, ceil(m / bm), ceil(k / bk))
    return torch.rand(shape, device=x.device) < p


def mask_to_increment_table(mask: torch.Tensor, BLOCK_K: int):
    """CSR-style pointer-increment table of the kept blocks (flash_dropout/functional/utils.py:19-69).

    Returns ``(table, row_indices, row_widths)``: ``row_widths[r]`` kept blocks in row r,
    ``row_indices[r]`` where row r starts in ``table``, and ``table`` the element offset of each kept
    block relative to the previous kept block of its row (absolute for the first one of a row).
    """
    keep = ~mask
    row_widths = keep.sum(dim=1)
    row_indices = torch.cumsum(row_widths, dim=0) - row_widths
    cols = torch.nonzero(keep, as_tuple=True)[1]
    offsets = cols * BLOCK_K
    table = offsets.clone()
    if table.numel() > 1:
        table[1:] = offsets[1:] - offsets[:-1]
    starts = row_indices[row_indices < table.numel()]
    table[starts] = offsets[starts]
    return table, row_indices, row_widths
