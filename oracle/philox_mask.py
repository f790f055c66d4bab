"""NumPy restatement of the block-mask draw and of every kept-block index format.  TEST INFRASTRUCTURE.

What it follows in andylolu2/sparse-dropout (paths relative to that project):
  * mask shape and polarity  — flash_dropout/functional/utils.py:11-16
        mask_shape = (ceil(m / block_size), ceil(k / block_size));  mask = rand(...) < p;  True = dropped
  * kept (row, col) list     — flash_dropout/functional/blockwise_dropout_matmul_triton.py:48
        torch.nonzero(~mask): row-major order
  * transposed view          — flash_dropout/functional/blockwise_dropout_matmul_cuda.py:50  (mask.T -> CSC)
  * CSR lists                — flash_dropout/functional/utils.py:57-69 (row_widths, row_indices)

PARITY OF MASK VALUES IS UNPINNED against the reference: the reference draws with ``torch.rand``
and none of its tests fixes the values (test/test_cuda.py:34 shares one drawn mask between both
implementations).  The draw is therefore specified here — Philox4x32-10 (Salmon et al., SC'11),
key = seed, counter = (block index lo, block index hi, offset lo, offset hi), first output word,
u = (x >> 8) * 2^-24 in fp32, dropped iff u < fp32(p) — and the Philox rounds themselves are pinned
by the generator's published known-answer vectors (tests/test_oracle.py).  The index formats ARE
pinned: against the reference's own functions run in this container (tests/golden/).
"""
from __future__ import annotations

from math import ceil

import numpy as np

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(counter: np.ndarray, key: np.ndarray) -> np.ndarray:
    """Philox4x32-10.  counter: (..., 4) uint32, key: (..., 2) uint32 -> (..., 4) uint32."""
    c = [np.asarray(counter[..., i], dtype=np.uint64) for i in range(4)]
    k0 = np.asarray(key[..., 0], dtype=np.uint64)
    k1 = np.asarray(key[..., 1], dtype=np.uint64)
    for _ in range(10):
        p0 = _M0 * c[0]
        p1 = _M1 * c[2]
        n0 = ((p1 >> np.uint64(32)) ^ c[1] ^ k0) & _MASK32
        n1 = p1 & _MASK32
        n2 = ((p0 >> np.uint64(32)) ^ c[3] ^ k1) & _MASK32
        n3 = p0 & _MASK32
        c = [n0, n1, n2, n3]
        k0 = (k0 + np.uint64(_W0)) & _MASK32
        k1 = (k1 + np.uint64(_W1)) & _MASK32
    return np.stack(c, axis=-1).astype(np.uint32)


def uniform24(seed: int, offset: int, n: int) -> np.ndarray:
    """u_i in [0, 1) for block indices i = 0..n-1 (fp32, 24 random bits)."""
    idx = np.arange(n, dtype=np.uint64)
    counter = np.stack([idx & _MASK32, idx >> np.uint64(32),
                        np.full(n, offset & 0xFFFFFFFF, dtype=np.uint64),
                        np.full(n, (offset >> 32) & 0xFFFFFFFF, dtype=np.uint64)], axis=-1)
    key = np.array([seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF], dtype=np.uint64)
    x = philox4x32_10(counter, np.broadcast_to(key, (n, 2)))[..., 0]
    return (x >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -24)


def block_pair(block_size) -> tuple:
    """(rows, columns) of a logical block: an int, or an (m, k) pair as in eval/mlp/config.py:23-27."""
    if isinstance(block_size, (tuple, list)):
        return int(block_size[0]), int(block_size[1])
    return int(block_size), int(block_size)


def block_mask(M: int, K: int, block_size, p: float, seed: int, offset: int = 0) -> np.ndarray:
    """Drop mask (True = dropped) of shape (ceil(M/bm), ceil(K/bk)) — utils.py:11-16 with the Philox draw."""
    assert 0 <= p < 1, "Dropout probability must be in [0, 1)"
    bm, bk = block_pair(block_size)
    R, C = ceil(M / bm), ceil(K / bk)
    u = uniform24(seed, offset, R * C).reshape(R, C)
    return u < np.float32(p)


def expand_to_tiles(mask: np.ndarray, M: int, K: int, block_size, tile: int = 128) -> np.ndarray:
    """Mask at `tile` granularity: tile (r, c) inherits logical block (r // rep_r, c // rep_c)."""
    bm, bk = block_pair(block_size)
    R, C = ceil(M / tile), ceil(K / tile)
    return np.repeat(np.repeat(mask, bm // tile, axis=0), bk // tile, axis=1)[:R, :C]


def kept_pairs(mask: np.ndarray) -> np.ndarray:
    """(row, col) of kept blocks, row-major order == torch.nonzero(~mask)."""
    return np.argwhere(~mask).astype(np.int32)


def csr(mask: np.ndarray):
    """row_ptr (R+1), col_idx (nnz): kept column indices of each row, ascending."""
    widths = (~mask).sum(axis=1)
    row_ptr = np.concatenate([[0], np.cumsum(widths)]).astype(np.int32)
    return row_ptr, kept_pairs(mask)[:, 1].copy()


def csc(mask: np.ndarray):
    """col_ptr (C+1), row_idx (nnz): kept row indices of each column, ascending (CSR of mask.T)."""
    return csr(mask.T)


def sdd_items(mask: np.ndarray) -> np.ndarray:
    """Kept blocks of each row paired up in ascending order: (row, col0, col1 or -1)."""
    out = []
    for r in range(mask.shape[0]):
        cols = np.flatnonzero(~mask[r])
        for i in range(0, len(cols), 2):
            out.append((r, cols[i], cols[i + 1] if i + 1 < len(cols) else -1))
    return np.array(out, dtype=np.int32).reshape(-1, 3)


def increment_table(mask: np.ndarray, BLOCK_K: int):
    """Restatement of mask_to_increment_table (flash_dropout/functional/utils.py:57-69).

    table: per kept block the element offset delta to the previous kept block of its row (the
    first kept block of a row holds its absolute offset); row_indices: exclusive prefix sum of
    kept-per-row; row_widths: kept-per-row.
    """
    row_widths = (~mask).sum(axis=1).astype(np.int64)
    row_indices = np.concatenate([[0], np.cumsum(row_widths[:-1])]).astype(np.int64)
    offsets = np.argwhere(~mask)[:, 1].astype(np.int64) * BLOCK_K
    table = np.diff(offsets, prepend=0)
    in_range = row_indices[row_indices < len(table)]
    table[in_range] = offsets[in_range]
    return table, row_indices, row_widths
