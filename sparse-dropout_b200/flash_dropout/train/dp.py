"""Batch-sharded data parallelism for the SparseDrop training steps.

The reference is single-GPU (no torch.distributed call site anywhere in it); this is the part of the
1/2/4/8-GPU training-step workload that is new.  One process per GPU.  Every rank runs the identical hot path
on its own batch shard with its own mask stream (Philox subsequence = rank), and the only exchange is the
all-reduce (mean) of the gradients:

  * all gradients live in ONE flat buffer of the parameters' dtype (fp32 master weights); each parameter's ``.grad`` is a view into it, so there is no
    pack / unpack copy around the collective;
  * the buffer is cut into buckets in reverse parameter order; a bucket's all-reduce is launched
    asynchronously (NCCL's own stream) the moment autograd has accumulated its last gradient, so communication
    overlaps the rest of backward;
  * ``finish()`` waits for the outstanding buckets before the optimizer step.
Works with any backend torch.distributed offers (NCCL on GPUs, gloo for the CPU tests).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from flash_dropout import random as sd_random


class FlatGradDataParallel:
    def __init__(self, module: torch.nn.Module, process_group=None, bucket_bytes: int = 16 << 20,
                 broadcast_from: int | None = 0, fuse_wgrad: bool = False):
        self.module = module
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.params = [p for p in module.parameters() if p.requires_grad]
        dev = self.params[0].device
        total = sum(p.numel() for p in self.params)
        dtype = self.params[0].dtype
        if any(p.dtype != dtype for p in self.params):
            raise ValueError("all trainable parameters must share one dtype (the master-weight dtype)")
        self.flat_grad = self._alloc_flat(total, dtype, dev)
        self._esize = self.flat_grad.element_size()
        # NCCL averages inside the collective; other backends (gloo in the CPU tests) sum and the mean is taken after
        self._avg_in_collective = (self.world > 1 and dev.type == "cuda" and
                                   dist.get_backend(process_group) == "nccl")
        self._reduce_op = dist.ReduceOp.AVG if self._avg_in_collective else dist.ReduceOp.SUM
        # parameters are laid out in REVERSE registration order: backward produces gradients roughly last
        # layer first, so bucket 0 (the front of the buffer) completes first
        off = 0
        self._slices = {}
        for p in reversed(self.params):
            n = p.numel()
            p.grad = self.flat_grad[off:off + n].view_as(p)
            self._slices[p] = (off, off + n)
            off += n
        # buckets = contiguous ranges of the flat buffer
        self.buckets: list[tuple[int, int]] = []
        self._bucket_of = {}
        start, cur = 0, 0
        for p in reversed(self.params):
            lo, hi = self._slices[p]
            self._bucket_of[p] = len(self.buckets)
            cur = hi
            if (cur - start) * self._esize >= bucket_bytes:
                self.buckets.append((start, cur))
                start = cur
        if cur > start:
            self.buckets.append((start, cur))
        self._bucket_size = [0] * len(self.buckets)
        for p in self.params:
            self._bucket_size[self._bucket_of[p]] += 1
        self._pending = list(self._bucket_size)
        self._handles = []
        if self.world > 1:
            if broadcast_from is not None:
                for p in module.parameters():
                    dist.broadcast(p.data, src=broadcast_from, group=self.group)
                for b in module.buffers():
                    dist.broadcast(b.data, src=broadcast_from, group=self.group)
            for p in self.params:
                p.register_post_accumulate_grad_hook(self._on_grad_ready)
        self._shadow_params: list = []
        self._shadows = None
        if fuse_wgrad:
            self._fuse_weight_gradients()
        sd_random.set_subsequence(self.rank)     # every rank draws its own masks from the shared seed

    # ------------------------------------------------------------------
    def _alloc_flat(self, total: int, dtype: torch.dtype, dev: torch.device) -> torch.Tensor:
        """The flat gradient buffer.  With NCCL on several GPUs it comes from a memory pool that is registered with
        the communicator as a user buffer, so that NCCL can reduce it in place (through NVLink SHARP where the fabric
        offers it) instead of staging it through its own buffers, which also takes fewer of its thread blocks away
        from the compute kernels.  Where this torch build or backend has no such pool, a plain tensor is used."""
        self.registered_buffer = False
        self._symm_group = None
        self._side = None
        import os
        if (self.world > 1 and dev.type == "cuda" and dist.get_backend(self.group) == "nccl"
                and os.environ.get("SD_DP_MULTIMEM", "0") == "1"):
            # Opt-in (SD_DP_MULTIMEM=1): symmetric memory with an NVLink multicast mapping; a bucket is then reduced by
            # one kernel of multimem loads and stores (the switch adds the ranks' values).  Measured on 2 B200s with
            # the MLP step (12 MB of gradients) it was no faster than NCCL on a registered buffer (0.355 vs 0.316 ms
            # per step with one bucket), so NCCL stays the default.
            try:
                import torch.distributed._symmetric_memory as symm_mem
                group = self.group or dist.group.WORLD
                flat = symm_mem.empty(total, dtype=dtype, device=dev)
                hdl = symm_mem.rendezvous(flat, group.group_name)
                if getattr(hdl, "multicast_ptr", 0):
                    flat.zero_()
                    self._symm_group = group.group_name
                    self._side = torch.cuda.Stream(dev)
                    return flat
            except Exception:                           # noqa: BLE001 - not available here: fall through to NCCL
                pass
        if self.world > 1 and dev.type == "cuda" and dist.get_backend(self.group) == "nccl":
            try:
                backend = (self.group or dist.group.WORLD)._get_backend(dev)
                pool = torch.cuda.MemPool(backend.mem_allocator)
                with torch.cuda.use_mem_pool(pool):
                    flat = torch.zeros(total, dtype=dtype, device=dev)
                backend.register_mem_pool(pool)
                self._pool = pool                       # keeps the registration alive
                self.registered_buffer = True
                return flat
            except Exception:                           # noqa: BLE001 - any failure means: not available here
                pass
        return torch.zeros(total, dtype=dtype, device=dev)

    def _fuse_weight_gradients(self) -> None:
        """Lets the dW kernel of every DropoutMM layer on the CUDA variant write its fp32 result straight into the
        layer's slice of the flat buffer (overwriting: the step zeroes the buffer and runs one backward), instead of
        returning a 16-bit gradient that autograd casts and accumulates with two more kernels per layer.  Autograd
        then never sees a gradient for these weights, so the bucket bookkeeping is notified from the layer's backward.
        Only for steps that run exactly one backward between ``zero_grad`` calls, without weight sharing."""
        from flash_dropout.layers import DropoutMM
        for m in self.module.modules():
            if isinstance(m, DropoutMM) and m.variant in ("blockwise[cuda]", "blockwise[triton]"):
                p = m.weight
                if p in self._slices and p.dtype == torch.float32 and p.is_cuda:
                    notify = (lambda p=p: self._on_grad_ready(p)) if self.world > 1 else None
                    p._sd_wgrad = (p.grad, False, notify)
                    self._shadow_params.append(p)

    def refresh_weight_shadows(self, dtype: torch.dtype | None) -> None:
        """Casts the weights of all layers with a fused weight gradient to ``dtype`` with one multi-tensor launch and
        hands the copies to the layers, which then skip their own cast under autocast.  Call it once per step, after
        the optimizer has updated the weights and before the forward pass; a layer ignores a copy that is older than
        its weight (``_version``)."""
        # the multi-tensor launch costs about as much as four casts: it pays for models with many layers (char-GPT:
        # 36 layers, step 4.41 -> 4.29 ms), not for the four layers of the MLP (0.215 -> 0.219 ms)
        if dtype is None or len(self._shadow_params) < self.shadow_min_layers:
            return
        if self._shadows is None or self._shadows[0].dtype != dtype:
            self._shadows = [torch.empty_like(p, dtype=dtype) for p in self._shadow_params]
        with torch.no_grad():
            torch._foreach_copy_(self._shadows, [p.detach() for p in self._shadow_params])
        for p, sh in zip(self._shadow_params, self._shadows):
            p._sd_w16 = (sh, p._version)

    defer_allreduce = False     # hooks stay quiet: the caller reduces the whole flat buffer itself
    shadow_min_layers = 8       # fewest fused layers from which refresh_weight_shadows() makes its copies

    def _reduce_bucket(self, b: int) -> None:
        """Starts the reduction of bucket b without blocking the stream that computes."""
        lo, hi = self.buckets[b]
        if self._symm_group is not None:
            cur = torch.cuda.current_stream(self.flat_grad.device)
            self._side.wait_stream(cur)
            with torch.cuda.stream(self._side):
                torch.ops.symm_mem.multimem_all_reduce_(self.flat_grad[lo:hi], "sum", self._symm_group)
            self._side_used = True
            return
        self._handles.append(dist.all_reduce(self.flat_grad[lo:hi], op=self._reduce_op, group=self.group,
                                             async_op=True))

    def _on_grad_ready(self, p: torch.Tensor) -> None:
        if self.defer_allreduce:
            return
        b = self._bucket_of[p]
        self._pending[b] -= 1
        if self._pending[b] == 0:
            self._reduce_bucket(b)

    def zero_grad(self) -> None:
        self.flat_grad.zero_()
        self._pending = list(self._bucket_size)
        self._handles = []

    def finish(self) -> None:
        """Wait for the bucket all-reduces and turn the sums into means."""
        if self.world == 1:
            return
        for b, left in enumerate(self._pending):       # parameters that received no gradient this step
            if left > 0:
                self._reduce_bucket(b)
                self._pending[b] = 0
        for h in self._handles:
            h.wait()
        self._handles = []
        if self._symm_group is not None:
            torch.cuda.current_stream(self.flat_grad.device).wait_stream(self._side)
            self.flat_grad.div_(self.world)             # the multimem reduction sums
        elif not self._avg_in_collective:
            self.flat_grad.div_(self.world)

    def grads_are_views(self) -> bool:
        """True while autograd kept accumulating in place into the flat buffer."""
        base = self.flat_grad.data_ptr()
        return all(p.grad is not None and p.grad.data_ptr() == base + self._esize * self._slices[p][0] for p in self.params)


_steps_since_check = 0


def _maybe_check_status(device: torch.device, check_every: int) -> None:
    """Every ``check_every`` steps: read the kernels' failure-detection word (one stream synchronisation) and raise
    if a device-side wait ran out of time during those steps."""
    global _steps_since_check
    if device.type != "cuda" or check_every <= 0:
        return
    _steps_since_check += 1
    if _steps_since_check >= check_every:
        _steps_since_check = 0
        from flash_dropout.cuda.binding_gemm import check_status
        check_status(device)


def train_step(model: torch.nn.Module, dp: FlatGradDataParallel, optimizer: torch.optim.Optimizer, loss_fn,
               autocast_dtype: torch.dtype | None = None, check_every: int = 64) -> torch.Tensor:
    """zero grads -> forward/backward (bucket all-reduces overlap backward) -> wait -> optimizer step.

    Every ``check_every`` steps (0 = never) the kernels' status word is read; a step whose kernels gave up on a
    wait raises ``SparseDropError`` instead of training on with undefined gradients."""
    _maybe_check_status(dp.flat_grad.device, check_every)
    dp.zero_grad()
    dev_type = dp.flat_grad.device.type
    if dev_type == "cuda":
        dp.refresh_weight_shadows(autocast_dtype)
    if autocast_dtype is not None:
        with torch.autocast(dev_type, dtype=autocast_dtype):
            loss = loss_fn(model)
    else:
        loss = loss_fn(model)
    loss.backward()
    dp.finish()
    optimizer.step()
    return loss.detach()


class GraphedTrainStep:
    """A whole training step captured once in a CUDA graph and replayed every step: zero the gradients, forward,
    backward with the bucketed gradient all-reduces overlapping it, and the optimizer update.

    The MLP and char-GPT training steps are made of dozens of small launches (a plan kernel and three GEMMs per
    DropoutMM, plus the model's other ops); eagerly they are bound by host launch overhead, which is what the
    reference's report identifies as the limit for small layers (report.pdf section 3.4).  Replaying a graph
    removes that.  Masks stay fresh because the plan kernel takes its Philox offset from a counter in device
    memory that each launch increments (``flash_dropout.random.enable_device_counter``).

    Inside the captured step each gradient bucket is all-reduced the moment backward has finished it, on the
    collective's own stream, so the exchange overlaps the rest of backward; the optimizer joins after the last
    bucket.  This needs an optimizer whose step can be captured (``capturable``: its step count lives on the device);
    an optimizer without that option, or ``whole_step=False``, leaves the collectives and the update outside the
    graph (one flat all-reduce and the update launched after every replay).  ``inputs`` are static device tensors:
    copy each batch into them before calling the step.
    """

    def __init__(self, model: torch.nn.Module, dp: FlatGradDataParallel, optimizer: torch.optim.Optimizer, loss_fn,
                 inputs: tuple, autocast_dtype: torch.dtype | None = None, warmup: int = 3, whole_step: bool = True,
                 batch_plans: bool = True):
        self.model, self.dp, self.optimizer = model, dp, optimizer
        self.inputs = inputs
        dev = dp.flat_grad.device
        if dev.type != "cuda":
            raise RuntimeError("GraphedTrainStep needs CUDA")
        if sd_random.device_counter(dev) is None:
            sd_random.enable_device_counter(dev)
        self.whole_step = whole_step and self._make_capturable(optimizer)
        dp.defer_allreduce = not self.whole_step        # outside the graph: one flat all-reduce after the replay

        from flash_dropout.cuda.binding_gemm import PlanBatch
        self.plan_batch = PlanBatch(dev) if batch_plans else None
        self._plan_stream = torch.cuda.Stream(dev) if batch_plans else None

        def fwd_bwd():
            if self.plan_batch is not None:
                PlanBatch.active = self.plan_batch
                if not self.plan_batch.recording:
                    # every layer's mask of this step from one launch, on a stream of its own: it runs beside the
                    # zeroing of the gradients and whatever else precedes the first SparseDrop layer
                    self.plan_batch.launch(self._plan_stream)
            dp.zero_grad()
            dp.refresh_weight_shadows(autocast_dtype)     # one launch instead of a cast per layer
            try:
                loss = fwd_loss()
            finally:
                PlanBatch.active = None
            if self.plan_batch is not None:
                self.plan_batch.join()                 # a pass that drew nothing still has to pick the launch up
                if self.plan_batch.recording:
                    self.plan_batch.finalize()
            loss.backward()
            if self.whole_step:
                dp.finish()
                optimizer.step()
            return loss.detach()

        def fwd_loss():
            if autocast_dtype is not None:
                with torch.autocast("cuda", dtype=autocast_dtype):
                    return loss_fn(model, *inputs)
            return loss_fn(model, *inputs)

        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):                    # allocations, autotuning and lazy init happen here
                fwd_bwd()
                if not self.whole_step:
                    self._finish()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            self.loss = fwd_bwd()

    @staticmethod
    def _make_capturable(optimizer: torch.optim.Optimizer) -> bool:
        """Switches the optimizer to device-side step counts if it has that option and has not stepped yet."""
        if not all("capturable" in g for g in optimizer.param_groups):
            return False
        if len(optimizer.state) != 0 and not all(g["capturable"] for g in optimizer.param_groups):
            return False                                # step counts already live on the host
        for g in optimizer.param_groups:
            g["capturable"] = True
        return True

    def describe(self) -> str:
        if self.whole_step:
            coll = "multimem (NVLink multicast) all-reduce" if self.dp._symm_group is not None else "NCCL all-reduce"
            return (f"CUDA graph replay of zero_grad + fwd + bwd + bucketed {coll} (overlapping backward) + optimizer"
                    if self.dp.world > 1 else "CUDA graph replay of zero_grad + fwd + bwd + optimizer")
        return "CUDA graph replay of zero_grad + fwd + bwd, then flat all-reduce + optimizer"

    def _finish(self) -> None:
        if self.dp.world > 1:
            if self.dp._symm_group is not None:
                torch.ops.symm_mem.multimem_all_reduce_(self.dp.flat_grad, "sum", self.dp._symm_group)
                self.dp.flat_grad.div_(self.dp.world)
            else:
                dist.all_reduce(self.dp.flat_grad, op=self.dp._reduce_op, group=self.dp.group)
                if not self.dp._avg_in_collective:
                    self.dp.flat_grad.div_(self.dp.world)
        self.optimizer.step()

    check_every = 64      # steps between reads of the kernels' failure-detection word (0 = never)

    def __call__(self) -> torch.Tensor:
        _maybe_check_status(self.dp.flat_grad.device, self.check_every)
        self.graph.replay()
        if not self.whole_step:
            self._finish()
        return self.loss
