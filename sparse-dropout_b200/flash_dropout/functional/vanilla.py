"""Element-wise dropout followed by a dense linear (flash_dropout/functional/vanilla.py:5-7)."""
import torch
import torch.nn.functional as F


def dropout_matmul(input: torch.Tensor, weight: torch.Tensor, p: float) -> torch.Tensor:
    return F.linear(F.dropout(input, p=p), weight)
