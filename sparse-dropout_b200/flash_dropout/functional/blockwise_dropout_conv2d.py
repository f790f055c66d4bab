"""Conv2d with blockwise dropout on its im2col matrix, on the sm_100a kernels.

The reference has no such op (its blockwise conv variants are commented out,
flash_dropout/layers/dropout_conv.py:86-99).  Semantics defined here: the im2col matrix of
flash_dropout/functional/im2col_conv2d.py:17-20 — M = N*P*Q rows, K = C*R*S columns in unfold order
k = c*R*S + r*S + s — gets one Bernoulli(p) drop decision per block_size x block_size block
(K zero-padded to the next multiple of the block), then the linear with the kernel viewed (Kout, CRS).

Data flow (nothing goes through F.unfold).  The K-outer im2col matrix is kept in panels of 128 pixels,
colP[ceil(M/128)][K64][128], so that every kept 128x128 block is one contiguous 32 KB run:
  forward   im2col_kept  : x (NCHW) -> kept blocks of colP                       (HBM-bound gather)
            DSD          : y2d[M, Kout] = (keep o col) . W2d^T / (1-p)           (col is an MN-major operand)
            y is returned as an NCHW-shaped view of y2d (channels_last strides), no permute copy
  backward  DSD          : dW2d[Kout, K] written transposed, reduction over kept row blocks of each K tile
            SDD          : kept blocks of dcolP = W2d^T . dy2d^T / (1-p)         (plan of the transposed result)
            col2im_kept  : dx (NCHW) = adjoint gather over kept blocks           (HBM-bound)
  By default the kept blocks of colT are saved for backward (151 MB for a 256x64x32x32 input with a 3x3 filter, half of what an
  unfold-based layer keeps); ``recompute_cols=True`` saves only the input (33 MB) and rebuilds colT in backward.
"""
from __future__ import annotations

from math import ceil

import torch

from flash_dropout import _lib
from flash_dropout import random as sd_random
from flash_dropout.cuda.binding_gemm import (BlockPlan, _on_device, conv_dsd_dw, conv_dsd_fwd, conv_fused_supported,
                                             dsd_panels, sdd_kept_t_panels)

from .im2col_conv2d import conv_output_size


def _round8(v: int) -> int:
    return (v + 7) & ~7


def _round64(v: int) -> int:
    return (v + 63) & ~63


def im2col_kept(x: torch.Tensor, kernel_size, padding, stride, dilation, plan: BlockPlan | None,
                k_gemm: int | None = None, panels: bool = False) -> torch.Tensor:
    """K-outer im2col matrix with only the plan's kept blocks filled in: ``colT[k_gemm][ldm]``, or with ``panels``
    ``[ceil(M/128)][k_gemm][128]`` (a kept block is then one contiguous run; ``k_gemm`` a multiple of 64)."""
    N, C, H, W = x.shape
    R, S = kernel_size
    P, Q = conv_output_size(H, W, R, S, padding, stride, dilation)
    M, K = N * P * Q, C * R * S
    if panels:
        k_gemm = k_gemm or _round64(K)
        colP = torch.empty((ceil(M / 128), k_gemm, 128), dtype=x.dtype, device=x.device)
        if k_gemm > K:
            colP[:, K:].zero_()
        x = x.contiguous()
        with _on_device(x.device):
            _lib.check(_lib.lib().sd_im2col_kept_panels(
                x.data_ptr(), N, C, H, W, R, S, padding[0], padding[1], stride[0], stride[1], dilation[0],
                dilation[1], colP.data_ptr(), k_gemm, plan.buf.data_ptr() if plan is not None else None,
                _lib.stream_ptr(x.device)))
        return colP
    k_gemm = k_gemm or _round8(K)
    ldm = _round8(M)
    colT = torch.empty((k_gemm, ldm), dtype=x.dtype, device=x.device)
    if k_gemm > K:
        colT[K:].zero_()
    x = x.contiguous()
    with _on_device(x.device):
        _lib.check(_lib.lib().sd_im2col_kept(
            x.data_ptr(), N, C, H, W, R, S, padding[0], padding[1], stride[0], stride[1], dilation[0], dilation[1],
            colT.data_ptr(), ldm, k_gemm, plan.buf.data_ptr() if plan is not None else None,
            _lib.stream_ptr(x.device)))
    return colT


def col2im_kept(dcolT: torch.Tensor, x_shape, kernel_size, padding, stride, dilation,
                plan: BlockPlan | None) -> torch.Tensor:
    """Adjoint of ``im2col_kept``; a 3-D ``dcolT`` is taken as the panel layout."""
    N, C, H, W = x_shape
    R, S = kernel_size
    dx = torch.empty(x_shape, dtype=dcolT.dtype, device=dcolT.device)
    if dcolT.dim() == 3:
        if not dcolT.is_contiguous() or dcolT.size(2) != 128:
            raise RuntimeError("a panel matrix must be contiguous [ceil(M/128)][k_gemm][128]")
        with _on_device(dcolT.device):
            _lib.check(_lib.lib().sd_col2im_kept_panels(
                dcolT.data_ptr(), dcolT.size(1), N, C, H, W, R, S, padding[0], padding[1], stride[0], stride[1],
                dilation[0], dilation[1], dx.data_ptr(), plan.buf.data_ptr() if plan is not None else None,
                _lib.dtype_code(dcolT.dtype), _lib.stream_ptr(dcolT.device)))
        return dx
    with _on_device(dcolT.device):
        _lib.check(_lib.lib().sd_col2im_kept(
            dcolT.data_ptr(), dcolT.stride(0), dcolT.size(0), N, C, H, W, R, S, padding[0], padding[1], stride[0],
            stride[1], dilation[0], dilation[1], dx.data_ptr(), plan.buf.data_ptr() if plan is not None else None,
            _lib.dtype_code(dcolT.dtype), _lib.stream_ptr(dcolT.device)))
    return dx


class BlockwiseDropoutConv2dCUDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, kernel, block_size, p, padding, stride, dilation, plan, recompute_cols, fused):
        assert 0 <= p < 1, "Dropout probability must be in [0, 1)"
        if not (input.is_cuda and kernel.is_cuda):
            raise RuntimeError("input and kernel must be CUDA")
        if input.dtype != kernel.dtype:
            raise RuntimeError(f"input ({input.dtype}) and kernel ({kernel.dtype}) must have the same dtype")
        _lib.dtype_code(input.dtype)
        N, C, H, W = input.shape
        Ko, Ck, R, S = kernel.shape
        if Ck != C:
            raise RuntimeError(f"kernel expects {Ck} input channels, input has {C}")
        P, Q = conv_output_size(H, W, R, S, padding, stride, dilation)
        M, K = N * P * Q, C * R * S
        Kg, Kog = _round64(K), _round8(Ko)       # the im2col matrix is kept in panels: k extent a multiple of 64
        if plan is None:
            plan = BlockPlan.draw(M, Kg, block_size, p, input.device)
        w2d = kernel.reshape(Ko, K)
        if Kg != K or Kog != Ko:                         # 16-byte rows for TMA; zero padding changes nothing
            w2d = torch.nn.functional.pad(w2d, (0, Kg - K, 0, Kog - Ko))
        w2d = w2d.contiguous()
        input = input.contiguous()
        ctx.fused = fused and conv_fused_supported(input.shape, (R, S), padding, stride, dilation)
        if ctx.fused:
            # im2col + DSD in one kernel: the matrix is gathered stage by stage from the input, never stored
            y2d = conv_dsd_fwd(input, w2d, plan, (R, S), padding, stride, dilation, 1.0 / (1.0 - p))   # (M, Kog)
            ctx.save_for_backward(input, w2d)
        else:
            colT = im2col_kept(input, (R, S), padding, stride, dilation, plan, Kg, panels=True)
            y2d = dsd_panels(colT, M, w2d, plan, _lib.SD_PLAN_ROWS, 1.0 / (1.0 - p))   # (M, Kog)
            if recompute_cols:
                ctx.save_for_backward(input, w2d)
            else:
                ctx.save_for_backward(input, w2d, colT)
        ctx.plan, ctx.p = plan, p
        ctx.geom = (padding, stride, dilation, (R, S), Ko, K)
        return y2d.view(N, P, Q, Kog)[..., :Ko].permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, grad_output):
        input, w2d, *saved_cols = ctx.saved_tensors
        plan, scale = ctx.plan, 1.0 / (1.0 - ctx.p)
        padding, stride, dilation, (R, S), Ko, K = ctx.geom
        N, C, H, W = input.shape
        Kog, Kg = w2d.shape
        M = grad_output.numel() // Ko
        dy2d = grad_output.to(input.dtype).permute(0, 2, 3, 1).reshape(M, Ko)   # free for channels_last gradients
        if Kog != Ko:
            dy2d = torch.nn.functional.pad(dy2d, (0, Kog - Ko))
        dy2d = dy2d.contiguous()
        grad_input = grad_kernel = None
        if ctx.needs_input_grad[1] and ctx.fused:
            dw2d = torch.empty((Kog, Kg), dtype=input.dtype, device=input.device)
            conv_dsd_dw(input, dy2d, plan, (R, S), padding, stride, dilation, scale, out=dw2d)
            grad_kernel = dw2d[:Ko, :K].reshape(Ko, C, R, S)
        elif ctx.needs_input_grad[1]:
            colT = saved_cols[0] if saved_cols else im2col_kept(input, (R, S), padding, stride, dilation, plan, Kg,
                                                                 panels=True)
            dw2d = torch.empty((Kog, Kg), dtype=input.dtype, device=input.device)
            dsd_panels(colT, M, dy2d.T, plan, _lib.SD_PLAN_COLS, scale, out=dw2d.T)
            grad_kernel = dw2d[:Ko, :K].reshape(Ko, C, R, S)
            del colT
        if ctx.needs_input_grad[0]:
            dcolT = torch.empty((ceil(M / 128), Kg, 128), dtype=input.dtype, device=input.device)
            # dcolT = w2d.T @ dy2d.T on the kept blocks, written into panels; col2im reads kept blocks only
            sdd_kept_t_panels(w2d.T, dy2d, plan, scale, out=dcolT)
            grad_input = col2im_kept(dcolT, input.shape, (R, S), padding, stride, dilation, plan)
        return grad_input, grad_kernel, None, None, None, None, None, None, None, None


def blockwise_dropout_conv2d(input: torch.Tensor, kernel: torch.Tensor, block_size: int, p: float,
                             padding=(0, 0), stride=(1, 1), dilation=(1, 1), plan=None,
                             recompute_cols: bool = False, fused: bool = True) -> torch.Tensor:
    """Conv2d (no bias) whose im2col matrix is block-dropped with probability ``p``; NCHW in, NCHW-shaped out.

    ``fused`` (default): geometries the fused kernels serve (3-wide filters, unit horizontal stride / dilation, one
    column of padding, rows of 8..64 pixels) never materialise the im2col matrix; others, and ``fused=False``, go
    through the kept-block im2col stage."""
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        input, kernel = input.to(dt), kernel.to(dt)
    with torch.autocast("cuda", enabled=False):
        return BlockwiseDropoutConv2dCUDA.apply(input, kernel, block_size, p, tuple(padding), tuple(stride),
                                                tuple(dilation), plan, recompute_cols, fused)
