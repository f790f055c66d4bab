"""Python face of the sm_100a SparseDrop kernels.

``GEMM`` keeps the interface of the reference's JIT-loaded extension wrapper
(flash_dropout/cuda/binding_gemm.py:7-47: ``gemm``, ``gemm_dsd``, ``gemm_sdd`` on 2-D CUDA
tensors that are row- or column-major, bool mask with True = dropped) but calls the C ABI of
libsparsedrop.so through ctypes instead of a pybind/libtorch module, on the current torch
stream and device (the reference launches on the legacy default stream of device 0,
flash_dropout/cuda/src/matmul_dsd.cuh:101-105).

``BlockPlan`` is the device-resident mask + compacted kept-tile lists the kernels walk.
"""
from __future__ import annotations

import ctypes as C
from functools import cache
from math import ceil

import torch

from flash_dropout import _lib

TILE = 128


def _check_operand(x: torch.Tensor, name: str) -> None:
    # flash_dropout/cuda/src/gemm_binding.cu:18-22
    if not x.is_cuda:
        raise RuntimeError(f"{name} must be CUDA")
    if x.dim() != 2:
        raise RuntimeError(f"{name} must be 2D")
    if not (x.stride(0) == 1 or x.stride(1) == 1):
        raise RuntimeError(f"{name} must be row or column major")


def _rep(block_size) -> tuple[int, int]:
    """(rows, columns) of 128x128 tiles in one logical dropout block.  ``block_size`` is an int or an ``(m, k)`` pair
    as the reference's model configs pass (eval/mlp/config.py:23-27); both must be multiples of 128."""
    if isinstance(block_size, (tuple, list)):
        if len(block_size) != 2:
            raise ValueError(f"block_size must be an int or an (m, k) pair, got {block_size}")
        bm, bk = block_size
    else:
        bm = bk = block_size
    for b in (bm, bk):
        if b <= 0 or b % TILE:
            # flash_dropout/cuda/src/matmul_dsd.cuh:92-93
            raise ValueError(f"block_size must be a positive multiple of {TILE}, got {block_size}")
    return bm // TILE, bk // TILE


class BlockPlan:
    """Drop mask of an ``R x C`` grid of 128x128 tiles plus its compacted index lists, on the device.

    Built by one kernel launch, either from ``(seed, offset, p)`` (Philox4x32-10, see
    ``sd_plan_from_seed``) or from a caller-supplied bool mask.  Never synchronises with the host.
    """

    def __init__(self, R: int, Cc: int, device: torch.device):
        self.R, self.C = int(R), int(Cc)
        self.layout = _lib.plan_layout(self.R, self.C)
        self.buf = torch.empty(self.layout.total_bytes, dtype=torch.uint8, device=device)
        self.mask: torch.Tensor | None = None   # logical bool mask, True = dropped
        self.origin: tuple | None = None        # (M, K, block_size, p, seed, offset) of a plan drawn from a host-side offset

    # ---- construction -------------------------------------------------------------------
    @classmethod
    def from_seed(cls, M: int, K: int, block_size: int, p: float, seed: int, offset: int,
                  device: torch.device) -> "BlockPlan":
        assert 0 <= p < 1, "Dropout probability must be in [0, 1)"
        rr, rc = _rep(block_size)
        plan = cls(ceil(M / TILE), ceil(K / TILE), device)
        mask = torch.empty((ceil(plan.R / rr), ceil(plan.C / rc)), dtype=torch.bool, device=device)
        with _on_device(device):
            _lib.check(_lib.lib().sd_plan_from_seed(
                plan.buf.data_ptr(), plan.R, plan.C, rr, rc, seed & (2**64 - 1), offset & (2**64 - 1), float(p),
                mask.data_ptr(), _lib.stream_ptr(device)))
        plan.mask = mask
        plan.origin = (M, K, block_size, float(p), seed, offset)     # enough to draw the same plan again
        return plan

    @classmethod
    def from_device_counter(cls, M: int, K: int, block_size: int, p: float, seed: int, base_offset: int,
                            counter: torch.Tensor, device: torch.device) -> "BlockPlan":
        """Like ``from_seed`` with offset = base_offset + counter[0], read and incremented on the device."""
        assert 0 <= p < 1, "Dropout probability must be in [0, 1)"
        rr, rc = _rep(block_size)
        plan = cls(ceil(M / TILE), ceil(K / TILE), device)
        mask = torch.empty((ceil(plan.R / rr), ceil(plan.C / rc)), dtype=torch.bool, device=device)
        with _on_device(device):
            _lib.check(_lib.lib().sd_plan_from_seed_counter(
                plan.buf.data_ptr(), plan.R, plan.C, rr, rc, seed & (2**64 - 1), base_offset & (2**64 - 1),
                counter.data_ptr(), float(p), mask.data_ptr(), _lib.stream_ptr(device)))
        plan.mask = mask
        return plan

    @classmethod
    def draw(cls, M: int, K: int, block_size: int, p: float, device: torch.device) -> "BlockPlan":
        """Next mask of the stream ``flash_dropout.random`` describes (host- or device-side counter)."""
        from flash_dropout import random as sd_random
        if PlanBatch.active is not None:
            return PlanBatch.active.request(M, K, block_size, p, device)
        counter = sd_random.device_counter(device)
        if counter is not None:
            seed, base = sd_random.seed_and_base()
            return cls.from_device_counter(M, K, block_size, p, seed, base, counter, device)
        seed, offset = sd_random.next_seed_offset()
        return cls.from_seed(M, K, block_size, p, seed, offset, device)

    @classmethod
    def from_mask(cls, mask: torch.Tensor, M: int, K: int, block_size: int) -> "BlockPlan":
        if mask.dtype != torch.bool:
            raise RuntimeError("Mask must be bool")
        if not mask.is_cuda or mask.dim() != 2:
            raise RuntimeError("Mask must be a 2D CUDA tensor")
        rr, rc = _rep(block_size)
        plan = cls(ceil(M / TILE), ceil(K / TILE), mask.device)
        want = (ceil(plan.R / rr), ceil(plan.C / rc))
        if tuple(mask.shape) != want:
            raise RuntimeError(f"mask shape {tuple(mask.shape)} does not match {want} blocks of {block_size}")
        with torch.cuda.device(mask.device):
            _lib.check(_lib.lib().sd_plan_from_mask(
                plan.buf.data_ptr(), plan.R, plan.C, rr, rc, mask.data_ptr(), mask.stride(0), mask.stride(1),
                _lib.stream_ptr(mask.device)))
        plan.mask = mask
        return plan

    # ---- views (no copies) ---------------------------------------------------------------
    def _ints(self, off: int, n: int) -> torch.Tensor:
        return self.buf[off:off + 4 * n].view(torch.int32)

    @property
    def header(self): return self._ints(self.layout.header, 16)
    @property
    def row_ptr(self): return self._ints(self.layout.row_ptr, self.R + 1)
    @property
    def col_idx(self): return self._ints(self.layout.col_idx, self.R * self.C)
    @property
    def col_ptr(self): return self._ints(self.layout.col_ptr, self.C + 1)
    @property
    def row_idx(self): return self._ints(self.layout.row_idx, self.R * self.C)
    @property
    def kept_pairs(self): return self._ints(self.layout.kept_pairs, 2 * self.R * self.C).view(-1, 2)
    @property
    def drop_pairs(self): return self._ints(self.layout.drop_pairs, 2 * self.R * self.C).view(-1, 2)
    @property
    def row_order(self): return self._ints(self.layout.row_order, self.R)
    @property
    def col_order(self): return self._ints(self.layout.col_order, self.C)
    @property
    def sdd_items(self): return self._ints(self.layout.sdd_items, 3 * self.R * ((self.C + 1) // 2)).view(-1, 3)
    @property
    def tile_mask(self): return self.buf[self.layout.mask:self.layout.mask + self.R * self.C].view(self.R, self.C)


class PlanBatch:
    """All block plans of one pass over a model from ONE kernel launch.

    A step draws one mask per SparseDrop layer, each a launch of a few microseconds.  A ``PlanBatch`` made the
    ``PlanBatch.active`` one first records the ``BlockPlan.draw`` calls of a pass (they run as usual); after
    ``finalize()``, ``launch()`` at the start of every later pass builds all of them side by side in one launch and
    ``BlockPlan.draw`` hands them out in the recorded order.  The masks are the ones the single launches would draw
    (plan i uses offset base + counter + i; the launch moves the device counter on by the number of plans).  Needs
    the device-side counter of ``flash_dropout.random``; plans beyond 3072 x 32 tiles keep their own launch."""

    active: "PlanBatch | None" = None

    def __init__(self, device: torch.device):
        self.device = device
        self.specs: list[tuple] = []
        self.plans: list[BlockPlan] = []
        self.batched: list[int] = []          # indices of the plans the batch launch builds
        self.recording = True
        self.pos = 0
        self.desc = None
        self._ready = None                    # event of a launch made on a side stream that the pass has not joined yet

    def request(self, M: int, K: int, block_size: int, p: float, device: torch.device) -> "BlockPlan":
        from flash_dropout import random as sd_random
        spec = (M, K, block_size if isinstance(block_size, int) else tuple(block_size), float(p))
        if self.recording:
            PlanBatch.active = None
            try:
                plan = BlockPlan.draw(M, K, block_size, p, device)
            finally:
                PlanBatch.active = self
            self.specs.append(spec)
            self.plans.append(plan)
            return plan
        if self.pos >= len(self.plans) or self.specs[self.pos] != spec:
            raise RuntimeError("the pass asks for different block plans than the recorded one")
        self.join(device)
        plan = self.plans[self.pos]
        if self.pos not in self._batched_set:      # too large for the batch kernel: its own launch, same counter
            counter = sd_random.device_counter(device)
            seed, base = sd_random.seed_and_base()
            with _on_device(device):
                _lib.check(_lib.lib().sd_plan_from_seed_counter(
                    plan.buf.data_ptr(), plan.R, plan.C, *_rep(block_size), seed & (2**64 - 1), base & (2**64 - 1),
                    counter.data_ptr(), float(p), plan.mask.data_ptr(), _lib.stream_ptr(device)))
        self.pos += 1
        return plan

    def finalize(self) -> None:
        """Ends the recording pass: describes the recorded plans to the batch kernel."""
        from flash_dropout import random as sd_random
        self.recording = False
        counter = sd_random.device_counter(self.device)
        if counter is None:
            raise RuntimeError("PlanBatch needs flash_dropout.random.enable_device_counter")
        seed, base = sd_random.seed_and_base()
        # the batch draws its plans first, at the start of the pass; larger plans follow with single launches
        self.batched = [i for i, pl in enumerate(self.plans) if pl.C <= 32 and pl.R <= 3072]
        self._batched_set = set(self.batched)
        n = len(self.batched)
        if n == 0:
            return
        L = _lib.lib()
        nbytes = L.sd_plan_batch_desc_bytes(n)
        host = (C.c_ubyte * nbytes)()
        self.desc = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        for j, i in enumerate(self.batched):
            pl = self.plans[i]
            _lib.check(L.sd_plan_batch_describe(host, self.desc.data_ptr(), n, j, pl.buf.data_ptr(), pl.R, pl.C,
                                                *_rep(self.specs[i][2]), seed & (2**64 - 1), base & (2**64 - 1),
                                                counter.data_ptr(), self.specs[i][3], pl.mask.data_ptr()))
        self.desc.copy_(torch.frombuffer(host, dtype=torch.uint8))

    def launch(self, side_stream: "torch.cuda.Stream | None" = None) -> None:
        """Start of a pass: one launch for every batched plan.

        With ``side_stream`` the launch goes there, behind everything the current stream holds so far (the previous
        pass still reads the plans), and the current stream picks it up again at the pass's first ``BlockPlan.draw``
        (or at ``join()``): whatever the pass does before its first SparseDrop layer runs beside the plan kernel."""
        self.pos = 0
        if self.desc is None:
            return
        if side_stream is None:
            with _on_device(self.device):
                _lib.check(_lib.lib().sd_plan_batch_launch(self.desc.data_ptr(), len(self.batched),
                                                           _lib.stream_ptr(self.device)))
            return
        side_stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side_stream):
            _lib.check(_lib.lib().sd_plan_batch_launch(self.desc.data_ptr(), len(self.batched),
                                                       _lib.stream_ptr(self.device)))
            self._ready = torch.cuda.Event()
            self._ready.record(side_stream)

    def join(self, device: "torch.device | None" = None) -> None:
        """The current stream waits for a launch made on a side stream (no-op otherwise)."""
        if self._ready is not None:
            torch.cuda.current_stream(device or self.device).wait_event(self._ready)
            self._ready = None


_workspaces: dict = {}


def workspace(device: torch.device) -> torch.Tensor:
    """Scratch for the split schedule of the GEMM kernel, one per (device, current stream).

    Launches that can overlap on the GPU must not share a workspace, hence the stream in the key.
    """
    stream = _lib.stream_ptr(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.get(key)
    if ws is None:
        with torch.cuda.device(device):
            ws = torch.empty(_lib.lib().sd_workspace_bytes(), dtype=torch.uint8, device=device)
            _lib.check(_lib.lib().sd_workspace_init(ws.data_ptr(), stream))
        _workspaces[key] = ws
    return ws


_status_words: dict = {}
SD_ERR_TIMEOUT = -4


def _dev_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def status_word(device: torch.device) -> torch.Tensor:
    """The device's failure-detection words (int32[4], word 0 is the status): every kernel launch of this module is
    given word 0, and a device-side wait that runs out of time records its code there instead of spinning on."""
    idx = _dev_index(device)
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w


def _status_ptr(device: torch.device) -> int:
    return status_word(device).data_ptr()


def check_status(device: torch.device | int | None = None) -> None:
    """Raises ``SparseDropError`` if a kernel launched on ``device`` since the last check gave up on a bounded wait.

    Waits for the device's current stream, reads the status word, and on a recorded time-out puts the library back
    into a usable state before raising: the counters of every cached split-schedule workspace of the device are
    cleared again (a launch that gave up may have left them non-zero) and the status word is reset.  The results of
    the step that timed out are not valid; later launches are.  Cheap enough to call where the host synchronises
    anyway (after a training step's loss has been read, at the end of a timed region)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    elif isinstance(device, int):
        device = torch.device("cuda", device)
    idx = _dev_index(device)
    w = _status_words.get(idx)
    if w is None:
        return                                  # nothing was ever launched on this device
    L = _lib.lib()
    with _on_device(device):
        rc = L.sd_check_status(w.data_ptr(), _lib.stream_ptr(device))
        if rc == 0:
            return
        msg = L.sd_last_error().decode()
        if rc == SD_ERR_TIMEOUT:
            for (d, stream), ws in _workspaces.items():
                if d == idx:
                    _lib.check(L.sd_workspace_init(ws.data_ptr(), _lib.stream_ptr(device)))
            w.zero_()
            torch.cuda.current_stream(device).synchronize()
    raise _lib.SparseDropError(f"libsparsedrop error {rc}: {msg}")


def _ws_ptr(ws, device: torch.device):
    if ws is None:
        return None
    if isinstance(ws, str):          # "auto"
        return workspace(device).data_ptr()
    return ws.data_ptr()


class _on_device:
    """``torch.cuda.device(dev)`` only when ``dev`` is not already current (the common case costs nothing)."""

    def __init__(self, device: torch.device):
        idx = device.index
        self.guard = None if idx is None or idx == torch.cuda.current_device() else torch.cuda.device(device)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)


def _mat(x: torch.Tensor):
    return (x.data_ptr(), x.stride(0), x.stride(1))


def _out(A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None) -> torch.Tensor:
    if out is None:
        return torch.empty((A.size(0), B.size(0)), dtype=A.dtype, device=A.device)
    if tuple(out.shape) != (A.size(0), B.size(0)) or out.dtype != A.dtype or out.device != A.device:
        raise RuntimeError("out has the wrong shape, dtype or device")
    return out


def _check_pair(A: torch.Tensor, B: torch.Tensor) -> int:
    _check_operand(A, "A")
    _check_operand(B, "B")
    if A.dtype != B.dtype:
        raise RuntimeError("A and B must have the same dtype")
    if A.size(1) != B.size(1):
        raise RuntimeError(f"reduction dimensions differ: A is {tuple(A.shape)}, B is {tuple(B.shape)}")
    if A.device != B.device:
        raise RuntimeError("A and B must be on the same device")
    return _lib.dtype_code(A.dtype)


def dense(A: torch.Tensor, B: torch.Tensor, scale: float = 1.0, out: torch.Tensor | None = None,
          ws="auto") -> torch.Tensor:
    """``scale * A @ B.T`` on the tcgen05 kernel with every tile kept.

    ``ws``: "auto" (cached per device and stream), a uint8 CUDA tensor, or None (whole-tile shares)."""
    dt = _check_pair(A, B)
    Cm = _out(A, B, out)
    with _on_device(A.device):
        _lib.check(_lib.lib().sd_gemm(*_mat(A), *_mat(B), *_mat(Cm), A.size(0), B.size(0), A.size(1),
                                      float(scale), dt, _ws_ptr(ws, A.device), _status_ptr(A.device),
                                      _lib.stream_ptr(A.device)))
    return Cm


def dsd(A: torch.Tensor, B: torch.Tensor, plan: BlockPlan, side: int, scale: float,
        out: torch.Tensor | None = None, ws="auto", relu: bool = False, accumulate: bool = False) -> torch.Tensor:
    """``scale * (keep o A) @ B.T``; ``side`` says whether A's row blocks are the plan's rows or columns.

    ``relu`` applies ReLU to the result in the kernel's epilogue.  An fp32 ``out`` receives the result in fp32
    (overwritten, or added to with ``accumulate``): the way a weight gradient goes straight into an fp32 buffer."""
    dt = _check_pair(A, B)
    M, K = A.shape
    want = (ceil(M / TILE), ceil(K / TILE)) if side == _lib.SD_PLAN_ROWS else (ceil(K / TILE), ceil(M / TILE))
    if (plan.R, plan.C) != want:
        raise RuntimeError(f"plan grid {(plan.R, plan.C)} does not match operand A {tuple(A.shape)} (need {want})")
    if out is not None and out.dtype == torch.float32:
        if relu:
            raise RuntimeError("relu and an fp32 result are not combined")
        if tuple(out.shape) != (M, B.size(0)) or out.device != A.device or not (out.stride(0) == 1 or out.stride(1) == 1):
            raise RuntimeError("out has the wrong shape, device or strides")
        with _on_device(A.device):
            _lib.check(_lib.lib().sd_gemm_dsd_f32(*_mat(A), *_mat(B), *_mat(out), M, B.size(0), K, plan.buf.data_ptr(),
                                                  side, float(scale), dt, int(accumulate), _ws_ptr(ws, A.device),
                                                  _status_ptr(A.device), _lib.stream_ptr(A.device)))
        return out
    if accumulate:
        raise RuntimeError("accumulate needs an fp32 out")
    Cm = _out(A, B, out)
    if relu:
        with _on_device(A.device):
            _lib.check(_lib.lib().sd_gemm_dsd_relu(*_mat(A), *_mat(B), *_mat(Cm), M, B.size(0), K, plan.buf.data_ptr(),
                                                   side, float(scale), dt, _ws_ptr(ws, A.device), _status_ptr(A.device),
                                                   _lib.stream_ptr(A.device)))
        return Cm
    with _on_device(A.device):
        _lib.check(_lib.lib().sd_gemm_dsd(*_mat(A), *_mat(B), *_mat(Cm), M, B.size(0), K, plan.buf.data_ptr(),
                                          side, float(scale), dt, _ws_ptr(ws, A.device), _status_ptr(A.device),
                                          _lib.stream_ptr(A.device)))
    return Cm


def sdd(A: torch.Tensor, B: torch.Tensor, plan: BlockPlan, scale: float,
        out: torch.Tensor | None = None, ws="auto", zero_dropped: bool = True,
        relu_mask: torch.Tensor | None = None) -> torch.Tensor:
    """``scale * keep o (A @ B.T)``: kept output tiles computed, dropped tiles written as zeros
    (or left untouched with ``zero_dropped=False``, for consumers that only read kept tiles).

    ``relu_mask``: a row-major tensor of the result's shape; result elements where it is <= 0 are written as zeros
    (the derivative of the ReLU that produced it), in the kernel's epilogue."""
    dt = _check_pair(A, B)
    M, N = A.size(0), B.size(0)
    if (plan.R, plan.C) != (ceil(M / TILE), ceil(N / TILE)):
        raise RuntimeError(f"plan grid {(plan.R, plan.C)} does not match the output {(M, N)}")
    Cm = _out(A, B, out)
    if relu_mask is not None:
        if tuple(relu_mask.shape) != (M, N) or relu_mask.dtype != A.dtype or relu_mask.stride(1) != 1 or not zero_dropped:
            raise RuntimeError("relu_mask must be a row-major tensor of the result's shape and dtype")
        with _on_device(A.device):
            _lib.check(_lib.lib().sd_gemm_sdd_relu_mask(*_mat(A), *_mat(B), *_mat(Cm), M, N, A.size(1),
                                                        plan.buf.data_ptr(), relu_mask.data_ptr(), relu_mask.stride(0),
                                                        float(scale), dt, _ws_ptr(ws, A.device), _status_ptr(A.device),
                                                        _lib.stream_ptr(A.device)))
        return Cm
    with _on_device(A.device):
        fn = _lib.lib().sd_gemm_sdd if zero_dropped else _lib.lib().sd_gemm_sdd_kept
        _lib.check(fn(*_mat(A), *_mat(B), *_mat(Cm), M, N, A.size(1), plan.buf.data_ptr(),
                   float(scale), dt, _ws_ptr(ws, A.device), _status_ptr(A.device), _lib.stream_ptr(A.device)))
    return Cm


def sdd_kept_t(A: torch.Tensor, B: torch.Tensor, plan: BlockPlan, scale: float, out: torch.Tensor,
               ws="auto") -> torch.Tensor:
    """Kept tiles of ``scale * (A @ B.T)`` for a plan that describes the transpose of the result (grid
    ``ceil(N/128) x ceil(M/128)``); dropped tiles of ``out`` are left untouched."""
    dt = _check_pair(A, B)
    M, N = A.size(0), B.size(0)
    if (plan.R, plan.C) != (ceil(N / TILE), ceil(M / TILE)):
        raise RuntimeError(f"plan grid {(plan.R, plan.C)} does not match the transposed output {(N, M)}")
    Cm = _out(A, B, out)
    with _on_device(A.device):
        _lib.check(_lib.lib().sd_gemm_sdd_kept_t(*_mat(A), *_mat(B), *_mat(Cm), M, N, A.size(1), plan.buf.data_ptr(),
                                                 float(scale), dt, _ws_ptr(ws, A.device), _status_ptr(A.device),
                                                 _lib.stream_ptr(A.device)))
    return Cm


def _check_panels(P: torch.Tensor, pixels: int) -> tuple[int, int]:
    """(kg, dtype code) of a panel matrix ``[ceil(pixels/128)][kg][128]`` (see ``sd_im2col_kept_panels``)."""
    if P.dim() != 3 or P.size(2) != TILE or not P.is_contiguous() or P.size(0) != ceil(pixels / TILE):
        raise RuntimeError(f"panel matrix must be contiguous [ceil({pixels}/128)][kg][128], got {tuple(P.shape)}")
    if P.size(1) % 64:
        raise RuntimeError(f"panel matrix needs kg % 64 == 0, got {P.size(1)}")
    return P.size(1), _lib.dtype_code(P.dtype)


def dsd_panels(P: torch.Tensor, pixels: int, B: torch.Tensor, plan: BlockPlan, side: int, scale: float,
               out: torch.Tensor | None = None, ws="auto") -> torch.Tensor:
    """``dsd`` with the conv's im2col matrix, stored in panels, as A: ``col`` (pixels x kg) for ``SD_PLAN_ROWS``,
    ``col.T`` for ``SD_PLAN_COLS``; the plan is the one of the pixels x kg matrix."""
    kg, dt = _check_panels(P, pixels)
    _check_operand(B, "B")
    if B.dtype != P.dtype or B.device != P.device:
        raise RuntimeError("panel matrix and B must share dtype and device")
    if (plan.R, plan.C) != (ceil(pixels / TILE), ceil(kg / TILE)):
        raise RuntimeError(f"plan grid {(plan.R, plan.C)} does not match the {pixels} x {kg} im2col matrix")
    M, K = (pixels, kg) if side == _lib.SD_PLAN_ROWS else (kg, pixels)
    if B.size(1) != K:
        raise RuntimeError(f"B must have {K} columns, got {tuple(B.shape)}")
    N = B.size(0)
    Cm = out if out is not None else torch.empty((M, N), dtype=P.dtype, device=P.device)
    if tuple(Cm.shape) != (M, N):
        raise RuntimeError(f"out must be {(M, N)}, got {tuple(Cm.shape)}")
    with _on_device(P.device):
        _lib.check(_lib.lib().sd_gemm_dsd_panels(P.data_ptr(), pixels, kg, *_mat(B), *_mat(Cm), N, plan.buf.data_ptr(),
                                                 side, float(scale), dt, _ws_ptr(ws, P.device), _status_ptr(P.device),
                                                 _lib.stream_ptr(P.device)))
    return Cm


def sdd_kept_t_panels(A: torch.Tensor, B: torch.Tensor, plan: BlockPlan, scale: float, out: torch.Tensor,
                      ws="auto") -> torch.Tensor:
    """``sdd_kept_t`` whose result ``(kg x pixels)`` is written into the panel matrix ``out``."""
    dt = _check_pair(A, B)
    kg, pixels = A.size(0), B.size(0)
    okg, odt = _check_panels(out, pixels)
    if okg != kg or odt != dt or out.device != A.device:
        raise RuntimeError("out must be a panel matrix of A's dtype and device with kg = A.size(0)")
    if (plan.R, plan.C) != (ceil(pixels / TILE), ceil(kg / TILE)):
        raise RuntimeError(f"plan grid {(plan.R, plan.C)} does not match the {pixels} x {kg} im2col matrix")
    with _on_device(A.device):
        _lib.check(_lib.lib().sd_gemm_sdd_kept_t_panels(*_mat(A), *_mat(B), out.data_ptr(), kg, pixels, A.size(1),
                                                        plan.buf.data_ptr(), float(scale), dt,
                                                        _ws_ptr(ws, A.device), _status_ptr(A.device),
                                                        _lib.stream_ptr(A.device)))
    return out


def conv_fused_supported(x_shape, kernel_size, padding, stride, dilation) -> bool:
    """True if the geometry is served by the fused im2col + DSD kernels (``conv_dsd_fwd`` / ``conv_dsd_dw``)."""
    N, C, H, W = x_shape
    R, S = kernel_size
    return bool(_lib.lib().sd_conv_fused_supported(N, C, H, W, R, S, padding[0], padding[1], stride[0], stride[1],
                                                   dilation[0], dilation[1]))


def _conv_geom(x: torch.Tensor, kernel_size, padding, stride, dilation):
    if x.dim() != 4 or not x.is_contiguous():
        raise RuntimeError("x must be a contiguous NCHW tensor")
    N, C, H, W = x.shape
    R, S = kernel_size
    return (N, C, H, W, R, S, padding[0], padding[1], stride[0], stride[1], dilation[0], dilation[1])


def conv_dsd_fwd(x: torch.Tensor, w2d: torch.Tensor, plan: BlockPlan, kernel_size, padding, stride, dilation,
                 scale: float, ws="auto") -> torch.Tensor:
    """``y2d[N*P*Q, Ko] = scale * (keep o im2col(x)) @ w2d.T`` with the im2col matrix gathered inside the kernel."""
    dt = _lib.dtype_code(x.dtype)
    _check_operand(w2d, "w2d")
    geom = _conv_geom(x, kernel_size, padding, stride, dilation)
    N, C, H, W, R, S = geom[:6]
    P = (H + 2 * padding[0] - dilation[0] * (R - 1) - 1) // stride[0] + 1
    M, K, Ko = N * P * W, C * R * S, w2d.size(0)
    if (plan.R, plan.C) != (ceil(M / TILE), ceil(K / TILE)):
        raise RuntimeError(f"plan grid {(plan.R, plan.C)} does not match the {M} x {K} im2col matrix")
    if w2d.size(1) < K or w2d.dtype != x.dtype or w2d.device != x.device:
        raise RuntimeError("w2d must be [Ko, >= C*R*S] of x's dtype and device")
    y2d = torch.empty((M, Ko), dtype=x.dtype, device=x.device)
    with _on_device(x.device):
        _lib.check(_lib.lib().sd_conv_dsd_fwd(x.data_ptr(), *geom, *_mat(w2d), *_mat(y2d), Ko, plan.buf.data_ptr(),
                                              float(scale), dt, _ws_ptr(ws, x.device), _status_ptr(x.device),
                                              _lib.stream_ptr(x.device)))
    return y2d


def conv_dsd_dw(x: torch.Tensor, dy2d: torch.Tensor, plan: BlockPlan, kernel_size, padding, stride, dilation,
                scale: float, out: torch.Tensor, ws="auto") -> torch.Tensor:
    """``out[Ko, :C*R*S] = scale * dy2d.T @ (keep o im2col(x))``; ``out`` is [Ko, >= C*R*S] row-major."""
    dt = _lib.dtype_code(x.dtype)
    _check_operand(dy2d, "dy2d")
    geom = _conv_geom(x, kernel_size, padding, stride, dilation)
    N, C, H, W, R, S = geom[:6]
    P = (H + 2 * padding[0] - dilation[0] * (R - 1) - 1) // stride[0] + 1
    M, K, Ko = N * P * W, C * R * S, dy2d.size(1)
    if (plan.R, plan.C) != (ceil(M / TILE), ceil(K / TILE)):
        raise RuntimeError(f"plan grid {(plan.R, plan.C)} does not match the {M} x {K} im2col matrix")
    if dy2d.size(0) != M or dy2d.dtype != x.dtype or dy2d.device != x.device:
        raise RuntimeError(f"dy2d must be [{M}, Ko] of x's dtype and device")
    if out.dim() != 2 or out.size(0) != Ko or out.size(1) < K or out.stride(1) != 1 or out.dtype != x.dtype:
        raise RuntimeError("out must be a row-major [Ko, >= C*R*S] matrix of x's dtype")
    with _on_device(x.device):
        _lib.check(_lib.lib().sd_conv_dsd_dw(x.data_ptr(), *geom, *_mat(dy2d), *_mat(out), Ko, plan.buf.data_ptr(),
                                             float(scale), dt, _ws_ptr(ws, x.device), _status_ptr(x.device),
                                             _lib.stream_ptr(x.device)))
    return out


@cache
class GEMM:
    """Drop-in for the reference's ``GEMM`` wrapper (flash_dropout/cuda/binding_gemm.py:7-47)."""

    def __init__(self, verbose: bool = False):
        self.lib = _lib.lib()   # raises if libsparsedrop.so has not been built
        if verbose:
            print(f"libsparsedrop {self.lib.sd_version()} loaded from {_lib.LIB_PATH}")

    def gemm(self, A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
        return dense(A, B)

    def gemm_dsd(self, A: torch.Tensor, B: torch.Tensor, mask: torch.Tensor, block_size: int,
                 scale: float) -> torch.Tensor:
        _check_operand(A, "A")
        plan = BlockPlan.from_mask(mask, A.size(0), A.size(1), block_size)
        return dsd(A, B, plan, _lib.SD_PLAN_ROWS, scale)

    def gemm_sdd(self, A: torch.Tensor, B: torch.Tensor, mask: torch.Tensor, block_size: int,
                 scale: float) -> torch.Tensor:
        _check_operand(A, "A")
        _check_operand(B, "B")
        plan = BlockPlan.from_mask(mask, A.size(0), B.size(0), block_size)
        return sdd(A, B, plan, scale)
