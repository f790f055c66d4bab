"""fp32 CPU restatement of the masked-dense SparseDrop products.  TEST INFRASTRUCTURE.

Follows andylolu2/sparse-dropout (paths relative to that project):
  * forward  — flash_dropout/functional/naive.py:8-25 (blockwise_dropout_matmul_mask):
        clone x; view as (M/bs, bs, K/bs, bs); dropped blocks = 0, kept blocks /= (1 - p); F.linear(x, W)
  * backward — what autograd derives from those lines, written out:
        dx = keep o (dy . W) / (1 - p),      dW = dy^T . (keep o x) / (1 - p)
    which are the two products flash_dropout/functional/blockwise_dropout_matmul_cuda.py:44-51 computes
  * conv     — flash_dropout/functional/im2col_conv2d.py:12-27: unfold -> (N, PQ, CRS) -> linear with the
        kernel viewed (K, CRS) -> (N, K, P, Q); K order of the im2col matrix is k = c*R*S + r*S + s

The arithmetic library is PyTorch on the CPU, as in the reference.  Shapes that are not multiples of the
block size are zero-padded to the next multiple (the reference raises instead, naive.py:19-21).
Pinned against outputs of the reference's own functions run in this container: tests/golden/.
Blockwise dropout on the conv im2col matrix has no counterpart in the reference
(flash_dropout/layers/dropout_conv.py:86-99 is commented out): PARITY UNPINNED for that composition; its
two building blocks (im2col_conv2d and the masked-dense product) are each pinned.
"""
from __future__ import annotations

from math import ceil

import numpy as np
import torch
import torch.nn.functional as F


def _keep_matrix(mask, M: int, K: int, block_size) -> torch.Tensor:
    """fp32 (M, K) matrix: 0 in dropped blocks, 1 elsewhere.  ``block_size``: an int or an (m, k) pair."""
    bm, bk = (block_size if isinstance(block_size, (tuple, list)) else (block_size, block_size))
    m = torch.as_tensor(np.asarray(mask), dtype=torch.bool)
    assert tuple(m.shape) == (ceil(M / bm), ceil(K / bk)), (m.shape, M, K, block_size)
    keep = (~m).to(torch.float32)
    keep = keep.repeat_interleave(bm, 0).repeat_interleave(bk, 1)
    return keep[:M, :K]


def forward(x: torch.Tensor, mask, block_size: int, p: float, weight: torch.Tensor) -> torch.Tensor:
    """y = (keep o x / (1-p)) . W^T — naive.py:8-25."""
    assert 0 <= p < 1, "Dropout probability must be in [0, 1)"
    x = x.detach().to(torch.float32)
    M, K = x.shape
    keep = _keep_matrix(mask, M, K, block_size)
    return F.linear(x * keep / (1 - p), weight.detach().to(torch.float32))


def backward(x: torch.Tensor, mask, block_size: int, p: float, weight: torch.Tensor, dy: torch.Tensor):
    """(dx, dW) of `forward` for upstream gradient dy."""
    x = x.detach().to(torch.float32)
    w = weight.detach().to(torch.float32)
    dy = dy.detach().to(torch.float32)
    M, K = x.shape
    keep = _keep_matrix(mask, M, K, block_size)
    dx = (dy @ w) * keep / (1 - p)
    dw = dy.T @ (x * keep / (1 - p))
    return dx, dw


def forward_backward(x, mask, block_size, p, weight, dy):
    y = forward(x, mask, block_size, p, weight)
    dx, dw = backward(x, mask, block_size, p, weight, dy)
    return y, dx, dw


def conv_out_size(H, W, R, S, padding, stride, dilation):
    P = (H + 2 * padding[0] - dilation[0] * (R - 1) - 1) // stride[0] + 1
    Q = (W + 2 * padding[1] - dilation[1] * (S - 1) - 1) // stride[1] + 1
    return P, Q


def im2col_matrix(x: torch.Tensor, R: int, S: int, padding, stride, dilation) -> torch.Tensor:
    """(N*P*Q, C*R*S) fp32 im2col matrix in unfold order — im2col_conv2d.py:17-20."""
    cols = F.unfold(x.detach().to(torch.float32), kernel_size=(R, S), padding=padding, stride=stride,
                    dilation=dilation)                      # (N, CRS, PQ)
    return cols.permute(0, 2, 1).reshape(-1, cols.shape[1])  # (N PQ, CRS)


def im2col_conv2d(x, kernel, padding=(0, 0), stride=(1, 1), dilation=(1, 1)) -> torch.Tensor:
    """Dense conv as unfold + linear — im2col_conv2d.py:5-27."""
    N, C, H, W = x.shape
    Ko, _, R, S = kernel.shape
    P, Q = conv_out_size(H, W, R, S, padding, stride, dilation)
    a = im2col_matrix(x, R, S, padding, stride, dilation)
    out = F.linear(a, kernel.detach().to(torch.float32).reshape(Ko, -1))   # (N PQ, K)
    return out.view(N, P * Q, Ko).permute(0, 2, 1).reshape(N, Ko, P, Q)


def conv_forward(x, kernel, mask, block_size, p, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    """Blockwise dropout on the im2col matrix (M = N*P*Q rows, K = C*R*S columns), then the linear."""
    N, C, H, W = x.shape
    Ko, _, R, S = kernel.shape
    P, Q = conv_out_size(H, W, R, S, padding, stride, dilation)
    a = im2col_matrix(x, R, S, padding, stride, dilation)
    y = forward(a, mask, block_size, p, kernel.reshape(Ko, -1))
    return y.view(N, P * Q, Ko).permute(0, 2, 1).reshape(N, Ko, P, Q)


def conv_backward(x, kernel, mask, block_size, p, dy, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    """(dx, dkernel) of conv_forward; dx folds the masked im2col gradient back (adjoint of unfold)."""
    N, C, H, W = x.shape
    Ko, _, R, S = kernel.shape
    a = im2col_matrix(x, R, S, padding, stride, dilation)
    dy2 = dy.detach().to(torch.float32).permute(0, 2, 3, 1).reshape(-1, Ko)
    da, dw = backward(a, mask, block_size, p, kernel.reshape(Ko, -1), dy2)
    da = da.view(N, -1, C * R * S).permute(0, 2, 1)
    dx = F.fold(da, output_size=(H, W), kernel_size=(R, S), padding=padding, stride=stride, dilation=dilation)
    return dx, dw.view(Ko, C, R, S)
