"""Byte counters for host <-> device copies, incremented where the copies are issued.

The engines move a step's inputs (token ids, masks, old log-probs, advantages, page tables) to the GPU and its
results (sampled tokens, log-prob grids, loss statistics) back through the two helpers below, so a benchmark or a
profiler can report exactly how many bytes crossed the host link per step instead of estimating them from tensor
shapes.  The counters are per process and cost one integer add per copy.

The reference only logs wall-clock ``h2d`` buckets (arctic_platform/sft/processors/sft_profile.py:31-77); it has no
byte accounting.
"""
from __future__ import annotations

import threading
from typing import Dict

import torch

_lock = threading.Lock()
_bytes = {"h2d": 0, "d2h": 0, "h2d_copies": 0, "d2h_copies": 0}


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def to_device(t: torch.Tensor, device, non_blocking: bool = True, dtype=None) -> torch.Tensor:
    """``t.to(device)`` that counts the bytes when the copy really crosses from host to device memory."""
    device = torch.device(device)
    if torch.is_tensor(t) and t.device.type == "cpu" and device.type != "cpu":
        with _lock:
            _bytes["h2d"] += _nbytes(t)
            _bytes["h2d_copies"] += 1
    return t.to(device, non_blocking=non_blocking) if dtype is None else t.to(device, dtype, non_blocking=non_blocking)


def to_host(t: torch.Tensor) -> torch.Tensor:
    """``t.cpu()`` that counts the bytes when the tensor lives on a device."""
    if torch.is_tensor(t) and t.device.type != "cpu":
        with _lock:
            _bytes["d2h"] += _nbytes(t)
            _bytes["d2h_copies"] += 1
    return t.cpu()


def snapshot() -> Dict[str, int]:
    with _lock:
        return dict(_bytes)


def reset() -> None:
    with _lock:
        for k in _bytes:
            _bytes[k] = 0
