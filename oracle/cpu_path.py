"""The reference's CPU path for the hot loop, timed.  TEST / BENCH INFRASTRUCTURE.

One "pass" = what andylolu2/sparse-dropout does on the CPU for one SparseDrop linear: the masked-dense
forward of flash_dropout/functional/naive.py:8-25 (clone, two indexed block writes, F.linear) and the backward
autograd derives from it, in fp32 through PyTorch's CPU GEMM on all host threads.  It does not skip dropped
blocks — the reference's CPU path has no sparse kernel.

When oracle/_ref holds the reference's own files (oracle/build_ref.py) the timed function IS the reference's
``blockwise_dropout_matmul_mask`` with autograd (``kind: "reference"``); otherwise it is the restatement in
oracle/masked_dense.py (``kind: "port"``).
"""
from __future__ import annotations

import os
import time

import numpy as np
import torch

from . import build_ref
from . import masked_dense as md
from . import philox_mask as pm


def host_info() -> dict:
    model = "unknown"
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    model = line.split(":", 1)[1].strip()
                    break
    except OSError:
        pass
    return {"cores": os.cpu_count() or 1, "cpu_model": model}


def reference_kind() -> str:
    return "reference" if build_ref.load() is not None else "port"


def _fwd_bwd_fn(block_size: int, p: float):
    """(callable(x, mask, w, dy) -> (y, dx, dw), kind).  The reference's function when oracle/_ref exists."""
    ref = build_ref.load()
    if ref is None:
        return (lambda x, mask, w, dy: md.forward_backward(x, mask, block_size, p, w, dy)), "port"
    fn = ref["naive"].blockwise_dropout_matmul_mask

    def run(x, mask, w, dy):
        xa, wa = x.detach().requires_grad_(), w.detach().requires_grad_()
        y = fn(xa, torch.as_tensor(np.asarray(mask)), block_size, p, wa)
        y.backward(dy)
        return y.detach(), xa.grad, wa.grad
    return run, "reference"


def _median_time(fn, budget_s: float, max_passes: int) -> tuple[float, int]:
    times = []
    t_start = time.perf_counter()
    while len(times) < max_passes and (not times or time.perf_counter() - t_start < budget_s):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2], len(times)


def time_linear_fwd_bwd(M: int, N: int, K: int, block_size: int, p: float, seed: int = 0,
                        budget_s: float = 12.0, max_passes: int = 5, threads: int | None = None) -> dict:
    """Times forward + dX + dW on seeded fp32 inputs; returns seconds per pass and the kept-block count."""
    threads = threads or (os.cpu_count() or 1)
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * K ** -0.25
    w = torch.randn(N, K, generator=g) * K ** -0.25
    dy = torch.randn(M, N, generator=g) * N ** -0.25
    mask = pm.block_mask(M, K, block_size, p, seed=seed, offset=0)
    run, kind = _fwd_bwd_fn(block_size, p)
    rows = max(block_size, 256 // block_size * block_size)
    run(x[:rows], mask[:rows // block_size], w, dy[:rows])          # warm the thread pool
    sec, passes = _median_time(lambda: run(x, mask, w, dy), budget_s, max_passes)
    tiles = pm.expand_to_tiles(mask, M, K, block_size) if block_size % 128 == 0 else mask
    return {"seconds_per_pass": sec, "passes": passes, "threads": threads, "kind": kind,
            "kept_tiles": int((~tiles).sum()), "total_tiles": int(tiles.size)}


def time_forward_1024(seed: int = 0, p: float = 0.5, reps: int = 10, threads: int | None = None) -> dict:
    """The reference's CPU-runnable case: fp32 forward y = (mask o x) . W^T / (1-p) at 1024^3, x ~ N(0,1),
    W ~ N(0, 1/1024), 128x128 blocks, mask from seed 0 (flash_dropout/functional/naive.py:8-25)."""
    threads = threads or (os.cpu_count() or 1)
    torch.set_num_threads(threads)
    n = 1024
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, n, generator=g)
    w = torch.randn(n, n, generator=g) / n ** 0.5
    mask = pm.block_mask(n, n, 128, p, seed=seed, offset=0)
    ref = build_ref.load()
    if ref is not None:
        tmask = torch.as_tensor(np.asarray(mask))
        fn, kind = (lambda: ref["naive"].blockwise_dropout_matmul_mask(x, tmask, 128, p, w)), "reference"
    else:
        fn, kind = (lambda: md.forward(x, mask, 128, p, w)), "port"
    with torch.no_grad():
        for _ in range(3):
            fn()
        sec, passes = _median_time(fn, 5.0, reps)
    return {"ms": sec * 1e3, "reps": passes, "threads": threads, "kind": kind,
            "dense_equivalent_gflops": 2.0 * n ** 3 / sec / 1e9, "kept_blocks": int((~mask).sum())}
