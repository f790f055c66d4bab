"""LayerNorm in front of SparseDrop layers, on the library's two HBM-bound kernels.

Same module as ``torch.nn.LayerNorm`` (same parameters and ``state_dict`` keys; the reference's models use
``nn.LayerNorm`` in front of their DropoutMM layers: eval/llm/model.py:72-74,113, eval/vit/model.py:11,53,106-108).
On a CUDA fp32 input whose normalised width is a multiple of 4 up to 1024 the forward is one pass that writes its
result in the dtype the consumer reads (the autocast dtype when autocast is on, so the separate cast disappears) and
the backward one pass for dx plus a small reduction for the parameter gradients; everything else (CPU tensors, other
dtypes, wider rows, several normalised dimensions) goes to ``F.layer_norm`` unchanged.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from flash_dropout import _lib

_CODES = {torch.float16: _lib.SD_F16, torch.bfloat16: _lib.SD_BF16, torch.float32: _lib.SD_F32}


def _ptr(t):
    return t.data_ptr() if t is not None else None


class _LayerNormCUDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_dtype):
        n = x.shape[-1]
        x2 = x.reshape(-1, n)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty((rows, n), device=x.device, dtype=out_dtype)
        mean = torch.empty(rows, device=x.device, dtype=torch.float32)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().sd_layernorm_fwd(x2.data_ptr(), rows, n, weight.data_ptr(), _ptr(bias), float(eps),
                                                   y.data_ptr(), _CODES[out_dtype], mean.data_ptr(), rstd.data_ptr(),
                                                   _lib.stream_ptr(x.device)))
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.has_bias = bias is not None
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, n = x2.shape
        dy2 = dy.reshape(rows, n)
        if dy2.dtype not in _CODES:
            dy2 = dy2.float()
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        L = _lib.lib()
        dx = torch.empty_like(x2)
        dgamma = torch.empty_like(weight)
        dbeta = torch.empty_like(weight) if ctx.has_bias else None
        ws = torch.empty(L.sd_layernorm_bwd_workspace_bytes(rows, n), device=x2.device, dtype=torch.uint8)
        with torch.cuda.device(x2.device):
            _lib.check(L.sd_layernorm_bwd(x2.data_ptr(), dy2.data_ptr(), _CODES[dy2.dtype], weight.data_ptr(),
                                          mean.data_ptr(), rstd.data_ptr(), rows, n, dx.data_ptr(), dgamma.data_ptr(),
                                          _ptr(dbeta), 0, ws.data_ptr(), _lib.stream_ptr(x2.device)))
        return dx.view(ctx.shape), dgamma, dbeta, None, None


def layer_norm(x: torch.Tensor, normalized_shape, weight, bias, eps: float) -> torch.Tensor:
    """``F.layer_norm`` with the fused path where it applies (see the module docstring)."""
    n = x.shape[-1] if x.dim() else 0
    fused = (x.is_cuda and x.dtype == torch.float32 and len(normalized_shape) == 1 and weight is not None
             and weight.dtype == torch.float32 and (bias is None or bias.dtype == torch.float32)
             and n % 4 == 0 and 0 < n <= 1024 and x.numel() > 0 and x.numel() // n < 2 ** 31
             and weight.is_contiguous() and (bias is None or bias.is_contiguous()))
    if not fused:
        return F.layer_norm(x, normalized_shape, weight, bias, eps)
    out_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else torch.float32
    if out_dtype not in _CODES:
        out_dtype = torch.float32
    with torch.autocast("cuda", enabled=False):
        return _LayerNormCUDA.apply(x, weight, bias, eps, out_dtype)


class LayerNorm(torch.nn.LayerNorm):
    """Drop-in ``torch.nn.LayerNorm`` that takes the fused path on CUDA (see the module docstring)."""

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return layer_norm(input, self.normalized_shape, self.weight, self.bias, self.eps)
