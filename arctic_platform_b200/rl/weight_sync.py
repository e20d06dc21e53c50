"""Standalone weight-sync coordinator for frameworks that own their training ranks.

A framework that trains outside this platform (its own FSDP / DDP ranks) but samples with it registers the
training-side tensors rank by rank; once every rank has contributed, the coordinator assembles full tensors
(concatenating ``fsdp`` shards along dim 0, taking rank 0's copy for ``dp``) and pushes them to the sampler
workers in buckets of ``bucket_size`` bytes.  Thread-safe; one sync at a time.  Role of
``WeightSyncCoordinator`` in arctic_platform/rl/weight_sync.py:51-243 (which drives NCCL broadcast groups
through ArcticInference; here the push is ``load_named_weight`` on the sampler actors or a direct copy).
"""
from __future__ import annotations

import threading
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

from .config import WeightSyncConfig


class WeightSyncCoordinator:
    def __init__(self, config: WeightSyncConfig, push_fn: Callable[[List[Tuple[str, torch.Tensor]]], None]):
        self.config = config
        self.push_fn = push_fn
        self._lock = threading.Lock()
        self._cond = threading.Condition(self._lock)
        self._contrib: Dict[int, Dict[str, torch.Tensor]] = {}
        self._epoch = 0
        self._done_epoch = 0
        self._error: Optional[BaseException] = None

    def submit(self, rank: int, named_tensors: Iterable[Tuple[str, torch.Tensor]], timeout: Optional[float] = 600.0) -> int:
        """Called by every training rank with its tensors; returns the number of tensors synced once all
        ``training_gpus`` ranks have called.  The last arriving rank performs the push."""
        with self._cond:
            if rank in self._contrib:
                raise RuntimeError(f"rank {rank} submitted twice in one sync")
            self._contrib[rank] = {n: t.detach() for n, t in named_tensors}
            my_epoch = self._epoch
            if len(self._contrib) == self.config.training_gpus:
                try:
                    n = self._push_locked()
                    self._error = None
                except BaseException as exc:
                    self._error = exc
                    n = 0
                self._contrib = {}
                self._epoch += 1
                self._done_epoch = self._epoch
                self._last_count = n
                self._cond.notify_all()
            else:
                if not self._cond.wait_for(lambda: self._done_epoch > my_epoch, timeout):
                    self._contrib.pop(rank, None)
                    raise TimeoutError("weight sync: not every training rank arrived")
            if self._error is not None:
                raise RuntimeError(f"weight sync failed: {self._error}")
            return self._last_count

    def _assemble(self, name: str) -> torch.Tensor:
        parts = [self._contrib[r][name] for r in sorted(self._contrib)]
        if self.config.training_sharding == "fsdp" and len(parts) > 1:
            return torch.cat(parts, 0)
        return parts[0]

    def _push_locked(self) -> int:
        names = list(self._contrib[min(self._contrib)].keys())
        bucket: List[Tuple[str, torch.Tensor]] = []
        size = 0
        count = 0
        for n in names:
            t = self._assemble(n)
            nbytes = t.numel() * t.element_size()
            if bucket and size + nbytes > self.config.bucket_size:
                self.push_fn(bucket)
                bucket, size = [], 0
            bucket.append((n, t))
            size += nbytes
            count += 1
        if bucket:
            self.push_fn(bucket)
        return count
