"""Conv2d with blockwise dropout on its im2col matrix, on the sm_100a DSD/SDD kernels.

The reference has no such op (its blockwise conv variants are commented out,
flash_dropout/layers/dropout_conv.py:86-99).  Semantics defined here: the im2col matrix of
flash_dropout/functional/im2col_conv2d.py:17-20 — M = N*P*Q rows, K = C*R*S columns in unfold order
k = c*R*S + r*S + s — gets one Bernoulli(p) drop decision per block_size x block_size block
(K zero-padded to the next multiple of the block), then the linear with the kernel viewed (Kout, CRS).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .blockwise_dropout_matmul_cuda import blockwise_dropout_matmul
from .im2col_conv2d import conv_output_size, im2col_matrix


def blockwise_dropout_conv2d(input: torch.Tensor, kernel: torch.Tensor, block_size: int, p: float,
                             padding=(0, 0), stride=(1, 1), dilation=(1, 1), plan=None) -> torch.Tensor:
    N, C, H, W = input.shape
    Ko, _, R, S = kernel.shape
    P, Q = conv_output_size(H, W, R, S, padding, stride, dilation)
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        input, kernel = input.to(dt), kernel.to(dt)
    a = im2col_matrix(input, (R, S), padding, stride, dilation).reshape(N * P * Q, C * R * S)
    w = kernel.reshape(Ko, C * R * S)
    pad_k = (-a.size(1)) % 8
    pad_n = (-Ko) % 8
    if pad_k:   # 16-byte rows for TMA; zero columns change nothing
        a, w = F.pad(a, (0, pad_k)), F.pad(w, (0, pad_k))
    if pad_n:
        w = F.pad(w, (0, 0, 0, pad_n))
    out = blockwise_dropout_matmul(a, w, block_size, p, plan)      # (N PQ, Ko)
    if pad_n:
        out = out[:, :Ko]
    return out.reshape(N, P * Q, Ko).transpose(1, 2).reshape(N, Ko, P, Q)
