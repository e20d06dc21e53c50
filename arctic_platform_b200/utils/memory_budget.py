"""Does the sampler's KV cache have to leave the GPU while the trainer runs?

In the colocated placement the sampler sleeps during the training half of a step so that the trainer can use its
memory (the reference: ``sleep(level=1)`` of the vLLM engine, arctic_platform/common/ray_server.py:921-933).  Freeing
and re-creating a KV cache of tens of GB costs device-memory mapping time on every step (0.3 s for 43 GB on one GPU,
more than a second when eight processes of a node map at once) and throws the captured decode graphs away.  When
the trainer's measured high-water mark leaves room for the cache, level-1 sleep therefore keeps it.

When trainer and sampler live in ONE process they also share one caching allocator, so handing memory over does
not need the driver at all: the sleeping sampler drops its cache tensors, the trainer's activations are carved out
of the same blocks, and the waking sampler gets the coalesced blocks back -- no ``cudaFree`` / ``cudaMalloc`` of
~100 GB per step (1 s of the step at eight processes per node, where the driver serialises the mapping work).
``shares_allocator`` tells both sides when that holds (``APB_SHARED_ALLOCATOR=0``: always return memory to the
driver, as engines in separate processes must).

The trainer reports its footprint after every optimizer step (``note_training_peak``): the device memory in use at
that moment -- the caching allocator does not return blocks, so this is the training high-water mark, symmetric
buffers included -- minus the KV bytes that were resident meanwhile.  ``kv_may_stay`` answers for the sampler.
``APB_SLEEP_KEEP_KV=0`` / ``1`` forces the answer.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

_train_peak: Dict[int, int] = {}      # device index -> bytes in use by everything but the KV cache, after a step
_kv_resident: Dict[int, int] = {}     # device index -> bytes of KV cache currently allocated by samplers

_trainers: Dict[int, int] = {}        # device index -> training engines built in this process
_samplers: Dict[int, int] = {}        # device index -> sampler engines built in this process

HEADROOM = 0.12                       # fraction of the device left free for fragmentation and workspace


def register(kind: str, device) -> None:
    """Called by the engines' constructors (``kind``: "trainer" or "sampler")."""
    if torch.device(device).type != "cuda":
        return
    book = _trainers if kind == "trainer" else _samplers
    i = _index(device)
    book[i] = book.get(i, 0) + 1


def shares_allocator(device) -> bool:
    """A training engine and a sampler were both built in this process on ``device``."""
    if os.environ.get("APB_SHARED_ALLOCATOR", "1") == "0" or torch.device(device).type != "cuda":
        return False
    i = _index(device)
    return _trainers.get(i, 0) > 0 and _samplers.get(i, 0) > 0


def _index(device) -> int:
    d = torch.device(device)
    return d.index if d.index is not None else torch.cuda.current_device()


def set_kv_resident(device, nbytes: int) -> None:
    _kv_resident[_index(device)] = int(nbytes)


def note_training_peak(device) -> None:
    if not torch.cuda.is_available() or torch.device(device).type != "cuda":
        return
    i = _index(device)
    free, total = torch.cuda.mem_get_info(i)
    _train_peak[i] = max(_train_peak.get(i, 0), total - free - _kv_resident.get(i, 0))


def kv_may_stay(device, kv_bytes: int) -> bool:
    forced = os.environ.get("APB_SLEEP_KEEP_KV")
    if forced in ("0", "1"):
        return forced == "1"
    if not torch.cuda.is_available() or torch.device(device).type != "cuda":
        return False
    i = _index(device)
    if i not in _train_peak:
        return False                  # no training step seen on this device yet: give the memory back
    _free, total = torch.cuda.mem_get_info(i)
    return _train_peak[i] + int(kv_bytes) <= (1.0 - HEADROOM) * total
