"""Bias-free linear layer with dropout fused into its matmul (reference: flash_dropout/layers/dropout_mm.py)."""
from __future__ import annotations

import math

import torch
from torch import nn

import flash_dropout.functional as F

VARIANTS = ("none", "vanilla", "blockwise[naive]", "blockwise[triton]", "blockwise[cuda]")


def _block_size(kwargs: dict):
    """``block_size`` keyword: an int, or an ``(m, k)`` pair as the reference's model configs pass
    (eval/mlp/config.py:23-27) — m rows by k columns of the layer's input per dropout decision.  A pair with equal
    entries is returned as an int."""
    bs = kwargs["block_size"]
    if isinstance(bs, (tuple, list)):
        if len(bs) != 2 or int(bs[0]) <= 0 or int(bs[1]) <= 0:
            raise ValueError(f"block_size must be an int or an (m, k) pair of positive ints, got {bs}")
        return int(bs[0]) if bs[0] == bs[1] else (int(bs[0]), int(bs[1]))
    return int(bs)


class DropoutMM(nn.Module):
    """``y = dropout(x) @ W.T``; in eval mode a plain linear.  Same constructor as the reference
    (dropout_mm.py:15-35): weight ``(out_features, in_features)``, kaiming-uniform(a=sqrt(5)), no bias.
    Extra keyword for the CUDA variant: ``recompute_plan=True`` keeps only the mask's (seed, offset) between forward
    and backward and draws the block plan again there instead of keeping its buffer alive."""

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

    def forward(self, input: torch.Tensor, activation: str | None = None, input_relu: bool = False,
                grad_premasked: bool = False) -> torch.Tensor:
        """``activation="relu"`` applies ReLU to the result.  On the CUDA variant it is fused into the forward kernel,
        ``input_relu`` (the input is a ReLU's output) fuses that ReLU's derivative into the dX kernel, and
        ``grad_premasked`` says the consumer of this layer's output does the same for this layer's ReLU; the other
        variants apply a plain ReLU and ignore the two hints.  With no arguments: the reference's forward."""
        if activation not in (None, "relu"):
            raise ValueError(f"Unknown activation {activation}")
        v = self.variant
        if self.training and v in ("blockwise[cuda]", "blockwise[triton]"):
            lead = input.shape[:-1]
            x = input.reshape(-1, input.shape[-1])
            wgrad = getattr(self.weight, "_sd_wgrad", None) if torch.is_grad_enabled() else None
            # a 16-bit copy of the weight kept by the training step, valid while the weight has not changed since
            lowp = getattr(self.weight, "_sd_w16", None)
            lowp = lowp[0] if (lowp is not None and wgrad is not None and lowp[1] == self.weight._version) else None
            out = F.cuda_blockwise_dropout_matmul(x, self.weight, _block_size(self.kwargs), self.p, weight_lowp=lowp,
                                                  relu=activation == "relu", input_relu=input_relu,
                                                  grad_premasked=grad_premasked and activation == "relu", wgrad=wgrad,
                                                  recompute_plan=bool(self.kwargs.get("recompute_plan", False)))
            return out.reshape(*lead, self.out_features)
        out = self._forward_plain(input)
        return torch.relu(out) if activation == "relu" else out

    def _forward_plain(self, input: torch.Tensor) -> torch.Tensor:
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
