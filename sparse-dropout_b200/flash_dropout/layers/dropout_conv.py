"""Bias-free Conv2d with dropout on its input (reference: flash_dropout/layers/dropout_conv.py).

Keeps the reference's variants (``none``, ``im2col``, ``vanilla``, ``vanilla_2d``) and adds the blockwise
ones the reference left commented out (dropout_conv.py:86-99): ``blockwise[naive]`` (masked-dense in
PyTorch) and ``blockwise[cuda]`` (sm_100a kernels); both drop blocks of the im2col matrix.
"""
from __future__ import annotations

import math

import torch
from torch import nn

import flash_dropout.functional as F
from flash_dropout.functional.im2col_conv2d import conv_output_size, im2col_matrix
from flash_dropout.functional.naive import blockwise_dropout_matmul as naive_matmul

from .dropout_mm import _block_size


class DropoutConv2d(nn.Module):
    __constants__ = ["stride", "padding", "dilation", "in_channels", "out_channels", "kernel_size", "p", "variant"]

    def __init__(self, in_channels: int, out_channels: int, kernel_size: tuple[int, int],
                 stride: tuple[int, int] = (1, 1), padding: tuple[int, int] = (0, 0),
                 dilation: tuple[int, int] = (1, 1), p: float = 0.1, variant: str = "vanilla", **kwargs) -> None:
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.dilation = kernel_size, stride, padding, dilation
        self.p, self.variant, self.kwargs = p, variant, kwargs
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels, *kernel_size))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def _conv(self, input: torch.Tensor) -> torch.Tensor:
        return nn.functional.conv2d(input, self.weight, stride=self.stride, padding=self.padding,
                                    dilation=self.dilation)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if not self.training:
            return self._conv(input)
        v = self.variant
        geom = dict(padding=self.padding, stride=self.stride, dilation=self.dilation)
        if v == "none":
            return self._conv(input)
        if v == "im2col":
            return F.im2col_conv2d(input, self.weight, **geom)
        if v == "vanilla":
            return self._conv(nn.functional.dropout(input, p=self.p))
        if v == "vanilla_2d":
            return self._conv(nn.functional.dropout2d(input, p=self.p))
        if v == "blockwise[naive]":
            N, _, H, W = input.shape
            R, S = self.kernel_size
            P, Q = conv_output_size(H, W, R, S, self.padding, self.stride, self.dilation)
            a = im2col_matrix(input, (R, S), **geom).reshape(N * P * Q, -1)
            out = naive_matmul(a, self.weight.reshape(self.out_channels, -1), _block_size(self.kwargs), self.p)
            return out.reshape(N, P * Q, self.out_channels).transpose(1, 2).reshape(N, self.out_channels, P, Q)
        if v in ("blockwise[cuda]", "blockwise[triton]"):
            return F.cuda_blockwise_dropout_conv2d(input, self.weight, _block_size(self.kwargs), self.p, **geom)
        # the reference falls through with an unbound result here (dropout_conv.py:100)
        raise ValueError(f"Unknown variant {v}")
