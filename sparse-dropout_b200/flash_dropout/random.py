"""Counter-based RNG state for the block masks.

The reference draws masks with ``torch.rand`` (flash_dropout/functional/utils.py:15), so its masks
follow torch's global generator.  Here a mask is a pure function of ``(seed, offset)`` (Philox4x32-10,
evaluated on the device): ``seed`` follows ``torch.manual_seed`` unless set explicitly, ``offset``
counts the masks drawn since the seed last changed, and ``subsequence`` (e.g. the data-parallel rank)
selects a disjoint range of offsets so that ranks draw different masks from one seed.
"""
from __future__ import annotations

import torch

_state = {"seed": None, "torch_seed": None, "offset": 0, "subsequence": 0}
_device_counters: dict = {}      # device index -> uint64 CUDA tensor holding the offset counter
_SUBSEQ_SHIFT = 40


def manual_seed(seed: int, subsequence: int | None = None) -> None:
    """Fix the mask seed independently of torch's generator and restart the offset counter."""
    _state["seed"] = int(seed)
    _state["offset"] = 0
    if subsequence is not None:
        _state["subsequence"] = int(subsequence)


def set_subsequence(subsequence: int) -> None:
    _state["subsequence"] = int(subsequence)
    _state["offset"] = 0


def follow_torch_seed() -> None:
    """Go back to deriving the seed from ``torch.initial_seed()``."""
    _state["seed"] = None
    _state["torch_seed"] = None
    _state["offset"] = 0


def get_state() -> dict:
    return dict(_state)


def set_state(state: dict) -> None:
    _state.update(state)


def next_seed_offset() -> tuple[int, int]:
    """(seed, offset) for the next mask; advances the counter."""
    if _state["seed"] is None:
        ts = torch.initial_seed()
        if ts != _state["torch_seed"]:
            _state["torch_seed"] = ts
            _state["offset"] = 0
        seed = ts
    else:
        seed = _state["seed"]
    off = _state["offset"]
    _state["offset"] = off + 1
    return seed & (2**64 - 1), (_state["subsequence"] << _SUBSEQ_SHIFT) + off


def enable_device_counter(device: torch.device, start: int = 0) -> torch.Tensor:
    """Keep the mask offset counter in device memory from now on (for this device).

    Each plan launch then reads and increments the counter itself, so the sequence of masks no longer depends
    on values the host passes at launch time — a captured CUDA graph draws new masks on every replay.
    """
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = torch.full((1,), int(start), dtype=torch.int64, device=torch.device("cuda", idx))
    _device_counters[idx] = t
    return t


def disable_device_counter(device: torch.device | None = None) -> None:
    if device is None:
        _device_counters.clear()
    else:
        _device_counters.pop(device.index if device.index is not None else torch.cuda.current_device(), None)


def device_counter(device: torch.device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return _device_counters.get(idx)


def seed_and_base() -> tuple[int, int]:
    """(seed, base offset) for device-counter mode: the subsequence bits only; the counter supplies the rest."""
    if _state["seed"] is None:
        seed = torch.initial_seed()
    else:
        seed = _state["seed"]
    return seed & (2**64 - 1), _state["subsequence"] << _SUBSEQ_SHIFT
