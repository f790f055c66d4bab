"""The reference's CPU path for the hot loop, timed.  TEST / BENCH INFRASTRUCTURE.

One "pass" = what andylolu2/sparse-dropout does on the CPU for one SparseDrop linear: the masked-dense
forward of flash_dropout/functional/naive.py:8-25 and the two backward products autograd derives from it
(oracle/masked_dense.py), in fp32 through PyTorch's CPU GEMM on all host threads.  It does not skip
dropped blocks — the reference's CPU path has no sparse kernel.
"""
from __future__ import annotations

import os
import time

import torch

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
    md.forward_backward(x[:256], mask[:max(1, 256 // block_size)], block_size, p, w, dy[:256])   # warm the pool
    times = []
    t_start = time.perf_counter()
    while len(times) < max_passes and (not times or time.perf_counter() - t_start < budget_s):
        t0 = time.perf_counter()
        md.forward_backward(x, mask, block_size, p, w, dy)
        times.append(time.perf_counter() - t0)
    times.sort()
    tiles = pm.expand_to_tiles(mask, M, K, block_size) if block_size % 128 == 0 else mask
    return {"seconds_per_pass": times[len(times) // 2], "passes": len(times), "threads": threads,
            "kept_tiles": int((~tiles).sum()), "total_tiles": int(tiles.size)}
