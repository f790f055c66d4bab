"""SparseDrop linear on the sm_100a kernels: the autograd glue of the operator API.

Same contract as the reference's ``BlockwiseDropoutMatmulCUDA``
(flash_dropout/functional/blockwise_dropout_matmul_cuda.py:7-59): forward ``y = (keep o x) W^T / (1-p)``
by a DSD product, backward ``dx`` by an SDD product and ``dW`` by a DSD product over the transposed
operands.  Differences: the mask comes from the device-side Philox plan kernel instead of
``torch.rand`` (one launch, no host sync, and the same plan object is reused by all three products);
bf16 is accepted as well as fp16; launches go to the current stream of the tensors' device.
"""
from __future__ import annotations

import weakref

import torch

from flash_dropout import _lib
from flash_dropout import random as sd_random
from flash_dropout.cuda.binding_gemm import BlockPlan, dsd, sdd


def _operand(x: torch.Tensor) -> torch.Tensor:
    """Row- or column-major with a TMA-compatible leading stride, else a contiguous copy."""
    if x.dim() == 2 and x.data_ptr() % 16 == 0:
        if x.stride(1) == 1 and (x.stride(0) % 8 == 0 or x.size(0) == 1) and x.stride(0) >= x.size(1):
            return x
        if x.stride(0) == 1 and (x.stride(1) % 8 == 0 or x.size(1) == 1) and x.stride(1) >= x.size(0):
            return x
    return x.contiguous()


class BlockwiseDropoutMatmulCUDA(torch.autograd.Function):
    """forward(input, weight, block_size, p, plan, relu, input_relu, grad_premasked, wgrad, recompute_plan, anchor)

    The first four arguments are the reference's.  The others fuse the layer's elementwise neighbours into the
    kernels' epilogues (all off by default):
      relu            the result goes through ReLU in the forward epilogue (eval/mlp/model.py:33-38 applies it as a
                      separate op after every layer);
      input_relu      ``input`` is the output of a ReLU: the dX epilogue multiplies by its derivative (input > 0), so
                      the gradient this layer returns is already the gradient of the ReLU's input;
      grad_premasked  with ``relu``: the incoming gradient already carries this layer's ReLU derivative (its only
                      consumer is a layer called with ``input_relu``), so backward does not apply it again;
      wgrad           ``(fp32 tensor [out, in], accumulate, notify)``: the weight gradient is written (or added) in fp32
                      straight into that tensor by the dW epilogue instead of being returned to autograd as a 16-bit
                      tensor that is then cast and accumulated by two more kernels; ``notify()`` is called afterwards.
      recompute_plan  keep only (seed, offset) of the mask between forward and backward and draw the plan again there
                      (one more plan launch per layer in backward; the plan buffer, 4 bytes per tile and list entry, is
                      not kept alive).  Applies to plans drawn from a host-side offset; a plan whose offset was read
                      from the device-side counter (CUDA-graph mode, where plan buffers are static anyway) is kept.
      anchor          a tensor that ties the result into the autograd graph when ``weight`` is a 16-bit copy made outside
                      autograd (see ``blockwise_dropout_matmul(weight_lowp=...)``); it receives no gradient.
    """

    @staticmethod
    def forward(ctx, input: torch.Tensor, weight: torch.Tensor, block_size: int, p: float,
                plan: BlockPlan | None = None, relu: bool = False, input_relu: bool = False,
                grad_premasked: bool = False, wgrad=None, recompute_plan: bool = False, anchor=None):
        assert 0 <= p < 1, "Dropout probability must be in [0, 1)"
        if not (input.is_cuda and weight.is_cuda):
            # no CPU path: flash_dropout/cuda/src/gemm_binding.cu:19 raises the same way
            raise RuntimeError("input and weight must be CUDA")
        if input.dim() != 2 or weight.dim() != 2:
            raise RuntimeError("input and weight must be 2D")
        if input.dtype != weight.dtype:
            raise RuntimeError(f"input ({input.dtype}) and weight ({weight.dtype}) must have the same dtype")
        M, K = input.shape
        if K % 8 or weight.size(0) % 8:
            raise RuntimeError("in_features and out_features must be multiples of 8 (16-byte TMA rows)")
        input, weight = _operand(input), _operand(weight)
        if input_relu and input.stride(1) != 1:
            input = input.contiguous()
        if plan is None:
            plan = BlockPlan.draw(M, K, block_size, p, input.device)
        out = dsd(input, weight, plan, _lib.SD_PLAN_ROWS, 1.0 / (1.0 - p), relu=relu)
        if relu and not grad_premasked:
            ctx.save_for_backward(input, weight, out)
        else:
            ctx.save_for_backward(input, weight)
        ctx.origin = plan.origin if recompute_plan else None
        ctx.plan = None if ctx.origin is not None else plan
        ctx.p = p
        ctx.relu, ctx.input_relu, ctx.grad_premasked, ctx.wgrad = relu, input_relu, grad_premasked, wgrad
        return out

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        input, weight, *rest = ctx.saved_tensors
        plan, scale = ctx.plan, 1.0 / (1.0 - ctx.p)
        if plan is None:
            plan = BlockPlan.from_seed(*ctx.origin, input.device)    # the same mask and lists, drawn again
        dy = grad_output.to(input.dtype)
        if ctx.relu and not ctx.grad_premasked:
            dy = torch.ops.aten.threshold_backward(dy, rest[0], 0)       # ReLU derivative, one kernel
        dy = _operand(dy)
        grad_input = grad_weight = None
        if ctx.needs_input_grad[0]:
            # dx (M, K) = keep o (dy (M, N) . W (N, K)) * scale: B operand is W^T, a column-major view
            grad_input = sdd(dy, weight.T, plan, scale, relu_mask=input if ctx.input_relu else None)
        if ctx.wgrad is not None:
            # dW^T (K, N) in fp32, straight into the caller's gradient buffer
            target, accumulate, notify = ctx.wgrad
            dsd(input.T, dy.T, plan, _lib.SD_PLAN_COLS, scale, out=target.T, accumulate=accumulate)
            if notify is not None:
                notify()
        elif ctx.needs_input_grad[1]:
            # dW^T (K, N) = (keep o x)^T (K, M) . dy (M, N) * scale, stored straight into dW (N, K)
            grad_weight = torch.empty_like(weight, memory_format=torch.contiguous_format)
            dsd(input.T, dy.T, plan, _lib.SD_PLAN_COLS, scale, out=grad_weight.T)
        return grad_input, grad_weight, None, None, None, None, None, None, None, None, None


_last_cast = {"key": None, "src": None, "ref": None}


def _autocast_input(input: torch.Tensor, dt: torch.dtype) -> torch.Tensor:
    """``input.to(dt)``, shared between consecutive layers that are fed the very same tensor (the q / k / v
    projections of an attention block): one cast forward, and one cast of the summed gradient backward.

    The entry is valid only for the very tensor it was made from, unmodified since.  A layer sees a fresh 2-D
    view object on every call, so the tensor is identified by the object that owns its memory (the view's base)
    plus the view's geometry; the entry holds only a weak reference to that owner, so once it is freed the entry
    is dead and a new tensor that the allocator places at the same address can never be taken for it."""
    if input.dtype == dt:
        return input
    owner = input._base if input._base is not None else input
    key = (input._version, tuple(input.shape), tuple(input.stride()), input.storage_offset(), input.dtype, dt,
           input.requires_grad, torch.is_grad_enabled())
    src = _last_cast["src"]
    if src is not None and src() is owner and _last_cast["key"] == key:
        cached = _last_cast["ref"]()
        if cached is not None:
            return cached
    out = input.to(dt)
    _last_cast["key"], _last_cast["src"], _last_cast["ref"] = key, weakref.ref(owner), weakref.ref(out)
    return out


def blockwise_dropout_matmul(input: torch.Tensor, weight: torch.Tensor, block_size: int, p: float,
                             plan: BlockPlan | None = None, relu: bool = False, input_relu: bool = False,
                             grad_premasked: bool = False, wgrad=None, recompute_plan: bool = False,
                             weight_lowp: torch.Tensor | None = None) -> torch.Tensor:
    """``y = (mask o input) . weight^T / (1 - p)`` with a fresh block mask (or the given plan).

    Under CUDA autocast both operands are cast to the autocast dtype (the reference casts to fp16,
    blockwise_dropout_matmul_cuda.py:9); otherwise they must already be fp16 or bf16.  The keyword arguments after
    ``plan`` fuse elementwise neighbours into the kernels (see ``BlockwiseDropoutMatmulCUDA``).  ``weight_lowp`` is an
    up-to-date copy of ``weight`` in the autocast dtype that the caller keeps (a training step that casts all weights
    with one launch): it is used instead of casting again, which needs ``wgrad`` (the copy is outside autograd, so
    the weight gradient has to leave through the fused store).
    """
    anchor = None
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        input = _autocast_input(input, dt)
        if weight_lowp is not None and wgrad is not None and weight_lowp.dtype == dt and weight_lowp.shape == weight.shape:
            anchor, weight = weight, weight_lowp
        else:
            weight = weight.to(dt)
    with torch.autocast("cuda", enabled=False):
        return BlockwiseDropoutMatmulCUDA.apply(input, weight, block_size, p, plan, relu, input_relu, grad_premasked,
                                                wgrad, recompute_plan, anchor)
