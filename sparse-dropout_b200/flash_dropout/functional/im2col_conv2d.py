"""Convolution as im2col + matmul (reference: flash_dropout/functional/im2col_conv2d.py:5-27)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def conv_output_size(H: int, W: int, R: int, S: int, padding, stride, dilation) -> tuple[int, int]:
    P = (H + 2 * padding[0] - dilation[0] * (R - 1) - 1) // stride[0] + 1
    Q = (W + 2 * padding[1] - dilation[1] * (S - 1) - 1) // stride[1] + 1
    return P, Q


def im2col_matrix(input: torch.Tensor, kernel_size, padding, stride, dilation) -> torch.Tensor:
    """(N, P*Q, C*R*S) im2col view of an NCHW input; column order k = c*R*S + r*S + s."""
    cols = F.unfold(input, kernel_size=kernel_size, padding=padding, stride=stride, dilation=dilation)
    return cols.transpose(1, 2)


def im2col_conv2d(input: torch.Tensor, kernel: torch.Tensor, padding=(0, 0), stride=(1, 1),
                  dilation=(1, 1)) -> torch.Tensor:
    N, _, H, W = input.shape
    Ko, _, R, S = kernel.shape
    P, Q = conv_output_size(H, W, R, S, padding, stride, dilation)
    a = im2col_matrix(input, (R, S), padding, stride, dilation)
    out = F.linear(a, kernel.reshape(Ko, -1))          # (N, PQ, Ko)
    return out.transpose(1, 2).reshape(N, Ko, P, Q)
