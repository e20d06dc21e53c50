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

from dataclasses import dataclass

from .config import WeightSyncConfig


@dataclass(frozen=True)
class TransferGroup:
    """One sender and the sampler workers it feeds.  ``workers`` are ``(replica, tp_rank)`` pairs; the group's
    communicator has the sender as rank 0 and the workers after it in this order."""
    group_id: int
    sender_rank: int
    workers: Tuple[Tuple[int, int], ...]

    @property
    def world_size(self) -> int:
        return 1 + len(self.workers)

    @property
    def replica_ids(self) -> List[int]:
        return sorted({r for r, _ in self.workers})


class TransferSchedule:
    """Static assignment of sampler workers to training ranks for a weight transfer.

    ``dp``: every training rank holds the full weights, so ``min(training ranks, workers)`` of them send, each to a
    contiguous block of workers (whole replicas per sender whenever the counts divide) -- the transfer is as parallel
    as the smaller side allows and no worker receives twice.  ``fsdp``: every rank holds one shard of every tensor, so
    every rank sends, and every worker is in every group (it needs all shards)."""

    def __init__(self, groups: List[TransferGroup], training_gpus: int, inference_replicas: int, inference_tp: int,
                 training_sharding: str):
        self.groups = groups
        self.training_gpus, self.inference_replicas, self.inference_tp = training_gpus, inference_replicas, inference_tp
        self.training_sharding = training_sharding

    @staticmethod
    def build(training_sharding: str, training_gpus: int, inference_replicas: int, inference_tp: int) -> "TransferSchedule":
        if training_sharding not in ("dp", "fsdp"):
            raise ValueError("training_sharding must be 'dp' or 'fsdp'")
        if min(training_gpus, inference_replicas, inference_tp) < 1:
            raise ValueError("training_gpus, inference_replicas and inference_tp must be positive")
        workers = [(r, t) for r in range(inference_replicas) for t in range(inference_tp)]
        if training_sharding == "fsdp":
            groups = [TransferGroup(g, g, tuple(workers)) for g in range(training_gpus)]
        else:
            n = min(training_gpus, len(workers))
            base, extra = divmod(len(workers), n)
            groups, at = [], 0
            for g in range(n):
                take = base + (1 if g < extra else 0)
                groups.append(TransferGroup(g, g, tuple(workers[at:at + take])))
                at += take
        return TransferSchedule(groups, training_gpus, inference_replicas, inference_tp, training_sharding)

    @property
    def active_sender_ranks(self) -> List[int]:
        return [g.sender_rank for g in self.groups]

    @property
    def num_groups(self) -> int:
        return len(self.groups)

    def group_of_sender(self, rank: int) -> Optional[TransferGroup]:
        return next((g for g in self.groups if g.sender_rank == rank), None)

    def senders_of_worker(self, replica: int, tp_rank: int) -> List[int]:
        return [g.sender_rank for g in self.groups if (replica, tp_rank) in g.workers]


class WeightSyncCoordinator:
    def __init__(self, config: WeightSyncConfig, push_fn: Optional[Callable[[List[Tuple[str, torch.Tensor]]], None]] = None):
        self.config = config
        self.push_fn = push_fn
        self.schedule = TransferSchedule.build(config.training_sharding, config.training_gpus, config.inference_replicas,
                                               config.inference_tp)
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

    # ---- the reference's vocabulary (arctic_platform/rl/weight_sync.py:88-243)
    @property
    def sender_ranks(self) -> List[int]:
        """Training ranks that send in a transfer."""
        return self.schedule.active_sender_ranks

    @property
    def num_groups(self) -> int:
        return self.schedule.num_groups

    def build_groups(self, master_addr: str) -> List[dict]:
        """Descriptors a receiver side needs to join the transfer groups: one rendezvous port per group, spaced by the
        tensor-parallel width as the reference spaces them."""
        return [{"group_id": g.group_id, "master_addr": master_addr,
                 "master_port": self.config.base_port + g.group_id * self.config.inference_tp,
                 "world_size": g.world_size, "replica_ids": g.replica_ids, "sender_rank": g.sender_rank,
                 "workers": [list(w) for w in g.workers]} for g in self.schedule.groups]

    def sync_weights(self, rank: int, weights: Iterable[Tuple[str, torch.Tensor]], timeout: Optional[float] = 600.0, **_ignored) -> dict:
        """``submit`` under the reference's name: every training rank calls it with its tensors; returns
        ``{"num_tensors", "sender": whether this rank is one of the schedule's senders}``."""
        n = self.submit(rank, weights, timeout)
        return {"num_tensors": n, "sender": rank in self.sender_ranks}

    def destroy(self) -> None:
        with self._cond:
            self._contrib = {}
            self._error = None
            self._cond.notify_all()

    def _assemble(self, name: str) -> torch.Tensor:
        parts = [self._contrib[r][name] for r in sorted(self._contrib)]
        if self.config.training_sharding == "fsdp" and len(parts) > 1:
            return torch.cat(parts, 0)
        return parts[0]

    def _push_locked(self) -> int:
        if self.push_fn is None:
            raise RuntimeError("this coordinator was made without a push function: it can plan transfers, not run them")
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
