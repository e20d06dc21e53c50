"""Activation offload: tensors saved for backward wait in pinned host memory instead of HBM.

``ActivationOffload`` is a context manager around the forward pass.  Its saved-tensor hooks copy every qualifying
activation (CUDA, at least ``min_bytes``, not a parameter) to a pinned host buffer on a dedicated copy stream and
drop the device copy; the unpack hook brings it back.  Details that matter for throughput:

* **keep-last-N**: the most recently packed ``keep_last`` tensors stay on the device -- the backward needs them
  first, long before a round trip could finish;
* **LIFO prefetch**: backward consumes saved tensors roughly in reverse order of packing, so each unpack also starts
  the host-to-device copies of the ``prefetch`` entries packed just before it, on the copy stream;
* **pinned pool**: host buffers are recycled by size so steady-state steps make no ``cudaHostAlloc`` calls;
* the compute stream waits only on the event of the copy it consumes (no device-wide synchronisation).

Counterpart of arctic_platform/model/implementations/qwen35/gpu/activation_offload.py:65-293.  On a 180 GB part
the feature is off by default; it is for sequences or models that would not fit otherwise.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class OffloadStats:
    offloaded_tensors: int = 0
    offloaded_bytes: int = 0
    kept_tensors: int = 0
    skipped_tensors: int = 0
    prefetch_hits: int = 0
    prefetch_misses: int = 0
    pool_allocations: int = 0
    pool_reuses: int = 0
    peak_host_bytes: int = 0

    def as_dict(self) -> Dict[str, int]:
        return dict(self.__dict__)


class PinnedPool:
    """Recycles pinned host buffers keyed by (dtype, numel)."""

    def __init__(self, stats: OffloadStats, pin: bool = True):
        self._free: Dict[tuple, List[torch.Tensor]] = defaultdict(list)
        self._stats = stats
        self._pin = pin
        self.live_bytes = 0

    def get(self, like: torch.Tensor) -> torch.Tensor:
        key = (like.dtype, like.numel())
        if self._free[key]:
            self._stats.pool_reuses += 1
            buf = self._free[key].pop()
        else:
            self._stats.pool_allocations += 1
            buf = torch.empty(like.numel(), dtype=like.dtype, device="cpu", pin_memory=self._pin)
        self.live_bytes += buf.numel() * buf.element_size()
        self._stats.peak_host_bytes = max(self._stats.peak_host_bytes, self.live_bytes)
        return buf

    def put(self, buf: torch.Tensor) -> None:
        self.live_bytes -= buf.numel() * buf.element_size()
        self._free[(buf.dtype, buf.numel())].append(buf)


class _Entry:
    __slots__ = ("idx", "host", "shape", "device", "d2h_done", "dev", "h2d_done", "kept")

    def __init__(self, idx):
        self.idx = idx
        self.host = None
        self.shape = None
        self.device = None
        self.d2h_done = None
        self.dev = None
        self.h2d_done = None
        self.kept = None


class ActivationOffload:
    def __init__(self, enabled: bool = True, min_bytes: int = 1 << 20, keep_last: int = 2, prefetch: int = 2,
                 pool: Optional[PinnedPool] = None):
        self.enabled = enabled
        self.min_bytes = min_bytes
        self.keep_last = keep_last
        self.prefetch = prefetch
        self.stats = OffloadStats()
        self.pool = pool or PinnedPool(self.stats, pin=torch.cuda.is_available())
        self.pool._stats = self.stats
        self._entries: Dict[int, _Entry] = {}
        self._order: List[int] = []          # indices of offloaded entries in pack order
        self._recent: List[_Entry] = []      # candidates still on the device (keep-last window)
        self._next = 0
        self._copy_stream = None
        self._hooks = None

    # ------------------------------------------------------------------ hooks
    def _stream(self, device):
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=device)
        return self._copy_stream

    def _qualifies(self, t: torch.Tensor) -> bool:
        return (t.is_cuda and not isinstance(t, torch.nn.Parameter) and t.numel() * t.element_size() >= self.min_bytes
                and t.is_contiguous())

    def _offload(self, e: _Entry) -> None:
        t = e.kept
        cs = self._stream(t.device)
        cs.wait_stream(torch.cuda.current_stream(t.device))
        e.host = self.pool.get(t)
        e.shape, e.device = t.shape, t.device
        with torch.cuda.stream(cs):
            e.host.copy_(t.reshape(-1), non_blocking=True)
            e.d2h_done = torch.cuda.Event()
            e.d2h_done.record(cs)
        t.record_stream(cs)                   # the device block may be reused only after the copy has read it
        e.kept = None
        self._order.append(e.idx)
        self.stats.offloaded_tensors += 1
        self.stats.offloaded_bytes += t.numel() * t.element_size()

    def _pack(self, t: torch.Tensor):
        if not self.enabled or not self._qualifies(t):
            self.stats.skipped_tensors += 1
            return t
        e = _Entry(self._next)
        self._next += 1
        e.kept = t
        self._entries[e.idx] = e
        self._recent.append(e)
        while len(self._recent) > self.keep_last:
            self._offload(self._recent.pop(0))
        return e

    def _start_h2d(self, e: _Entry) -> None:
        if e.dev is not None or e.host is None:
            return
        cs = self._stream(e.device)
        with torch.cuda.stream(cs):
            cs.wait_event(e.d2h_done)
            e.dev = torch.empty(e.shape, dtype=e.host.dtype, device=e.device)
            e.dev.view(-1).copy_(e.host, non_blocking=True)
            e.h2d_done = torch.cuda.Event()
            e.h2d_done.record(cs)

    def _unpack(self, obj):
        if not isinstance(obj, _Entry):
            return obj
        e = obj
        if e.kept is not None:                                    # never left the device
            self.stats.kept_tensors += 1
            return e.kept
        if e.dev is None:
            self.stats.prefetch_misses += 1
            self._start_h2d(e)
        else:
            self.stats.prefetch_hits += 1
        # LIFO prefetch: the entries packed just before this one are needed next
        if e.idx in self._order:
            pos = self._order.index(e.idx)
            for j in range(max(0, pos - self.prefetch), pos):
                self._start_h2d(self._entries[self._order[j]])
        torch.cuda.current_stream(e.device).wait_event(e.h2d_done)
        out = e.dev
        out.record_stream(torch.cuda.current_stream(e.device))
        return out

    def release(self) -> None:
        """Returns every host buffer to the pool (call after backward; ``__exit__`` does not, because the
        backward runs after the forward context has closed)."""
        for e in self._entries.values():
            if e.host is not None:
                if e.h2d_done is not None:
                    e.h2d_done.synchronize()
                elif e.d2h_done is not None:
                    e.d2h_done.synchronize()
                self.pool.put(e.host)
                e.host = None
            e.dev = e.kept = None
        self._entries.clear()
        self._order.clear()
        self._recent.clear()

    # ------------------------------------------------------------------ context
    def __enter__(self):
        self._hooks = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._hooks.__enter__()
        return self

    def __exit__(self, *exc):
        self._hooks.__exit__(*exc)
        self._hooks = None
        return False
