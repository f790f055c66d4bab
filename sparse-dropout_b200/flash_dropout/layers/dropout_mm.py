"""Bias-free linear layer with dropout fused into its matmul (reference: flash_dropout/layers/dropout_mm.py)."""
from __future__ import annotations

import math

import torch
from torch import nn

import flash_dropout.functional as F

VARIANTS = ("none", "vanilla", "blockwise[naive]", "blockwise[triton]", "blockwise[cuda]")


def _block_size(kwargs: dict) -> int:
    """``block_size`` keyword as an int; an (m, k) pair with equal entries is accepted because the
    reference's model configs pass ``(128, 128)`` (eval/mlp/config.py:23-27)."""
    bs = kwargs["block_size"]
    if isinstance(bs, (tuple, list)):
        if len(bs) != 2 or bs[0] != bs[1]:
            raise ValueError(f"block_size pair must have equal entries, got {bs}")
        bs = bs[0]
    return int(bs)


class DropoutMM(nn.Module):
    """``y = dropout(x) @ W.T``; in eval mode a plain linear.  Same constructor as the reference
    (dropout_mm.py:15-35): weight ``(out_features, in_features)``, kaiming-uniform(a=sqrt(5)), no bias."""

    __constants__ = ["in_features", "out_features"]

    def __init__(self, in_features: int, out_features: int, p: float = 0.1, variant: str = "vanilla",
                 **kwargs) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.p, self.variant, self.kwargs = p, variant, kwargs
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def extra_repr(self) -> str:
        return f"{self.in_features}, {self.out_features}, p={self.p}, variant={self.variant!r}"

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if not self.training:
            return nn.functional.linear(input, self.weight)
        lead = input.shape[:-1]
        x = input.reshape(-1, input.shape[-1])
        v = self.variant
        if v == "none":
            out = nn.functional.linear(x, self.weight)
        elif v == "vanilla":
            out = F.vanilla_dropout_matmul(x, self.weight, self.p)
        elif v == "blockwise[naive]":
            out = F.naive_blockwise_dropout_matmul(x, self.weight, _block_size(self.kwargs), self.p)
        elif v in ("blockwise[cuda]", "blockwise[triton]"):
            out = F.cuda_blockwise_dropout_matmul(x, self.weight, _block_size(self.kwargs), self.p)
        else:
            raise ValueError(f"Unknown variant {v}")
        return out.reshape(*lead, self.out_features)
