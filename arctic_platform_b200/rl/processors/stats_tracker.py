"""Scoped statistics with denominators and distributed export
(arctic_platform/rl/processors/stats_tracker.py:40-208): ``denominator`` registers boolean masks, ``stat``
records tensors against a denominator, ``scalar`` records plain numbers, ``export`` reduces everything to
Python floats (token-weighted means across ranks when a process group is given)."""
from __future__ import annotations

import contextlib
import time
from enum import Enum
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class ReduceType(Enum):
    AVG = "avg"
    SUM = "sum"
    MIN = "min"
    MAX = "max"
    SCALAR = "scalar"


class DistributedStatsTracker:
    def __init__(self, name: str = ""):
        self.scope_stack: List[str] = [name] if name else []
        self.denominators: Dict[str, List[torch.Tensor]] = {}
        self.stats: Dict[str, List] = {}
        self.reduce_types: Dict[str, ReduceType] = {}
        self.denom_of: Dict[str, str] = {}

    @contextlib.contextmanager
    def scope(self, name: str):
        self.scope_stack.append(name)
        try:
            yield
        finally:
            self.scope_stack.pop()

    def _key(self, name: str) -> str:
        return "/".join(self.scope_stack + [name])

    def denominator(self, **masks: torch.Tensor) -> None:
        for name, m in masks.items():
            if m.dtype != torch.bool:
                raise ValueError(f"denominator {name} must be a bool tensor")
            self.denominators.setdefault(self._key(name), []).append(m.detach())

    def stat(self, denominator: str, reduce_type: Optional[ReduceType] = None, **values: torch.Tensor) -> None:
        dkey = self._key(denominator)
        if dkey not in self.denominators:
            raise ValueError(f"unknown denominator {denominator!r}")
        for name, v in values.items():
            if v.shape != self.denominators[dkey][-1].shape:
                raise ValueError(f"stat {name} shape {tuple(v.shape)} does not match its denominator")
            key = self._key(name)
            self.stats.setdefault(key, []).append((v.detach().float(), self.denominators[dkey][-1]))
            self.denom_of[key] = dkey
            if reduce_type is not None:
                self.reduce_types[key] = reduce_type

    def scalar(self, **values: float) -> None:
        for name, v in values.items():
            key = self._key(name)
            self.stats.setdefault(key, []).append(float(v))
            self.reduce_types[key] = ReduceType.SCALAR

    @contextlib.contextmanager
    def record_timing(self, key: str):
        """Wall time of the block in seconds, recorded as the scalar ``key`` (under the current scope)."""
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.scalar(**{key: time.perf_counter() - t0})

    def export(self, key: Optional[str] = None, reduce_group=None, reset: bool = True) -> Dict[str, float]:
        out: Dict[str, float] = {}
        do_reduce = dist.is_initialized() and reduce_group is not False and dist.get_world_size(reduce_group) > 1

        def allreduce(t: torch.Tensor, op) -> torch.Tensor:
            if do_reduce:
                dist.all_reduce(t, op=op, group=reduce_group)
            return t

        for dkey, masks in self.denominators.items():
            n = torch.tensor(float(sum(int(m.sum()) for m in masks)), dtype=torch.float64)
            out[dkey] = float(allreduce(n, dist.ReduceOp.SUM))
        for skey, items in self.stats.items():
            if key is not None and skey != key:
                continue
            rt = self.reduce_types.get(skey)
            if rt == ReduceType.SCALAR:
                t = torch.tensor([sum(items), float(len(items))], dtype=torch.float64)
                allreduce(t, dist.ReduceOp.SUM)
                out[skey] = float(t[0] / t[1].clamp_min(1))
                continue
            s = sum(float((v * m).sum()) for v, m in items)
            n = sum(int(m.sum()) for _, m in items)
            if rt in (None, ReduceType.AVG):
                t = allreduce(torch.tensor([s, float(n)], dtype=torch.float64), dist.ReduceOp.SUM)
                out[skey + ("/avg" if rt is None else "")] = float(t[0] / t[1].clamp_min(1))
                if rt is None:
                    mins = [float(v[m].min()) for v, m in items if m.any()]
                    maxs = [float(v[m].max()) for v, m in items if m.any()]
                    # a rank whose masks are all empty still takes part in the reductions (with the neutral element):
                    # collectives that only some ranks enter would never complete
                    if mins or do_reduce:
                        lo = float(allreduce(torch.tensor(min(mins, default=float("inf")), dtype=torch.float64), dist.ReduceOp.MIN))
                        hi = float(allreduce(torch.tensor(max(maxs, default=float("-inf")), dtype=torch.float64), dist.ReduceOp.MAX))
                        if lo != float("inf"):
                            out[skey + "/min"], out[skey + "/max"] = lo, hi
            elif rt == ReduceType.SUM:
                out[skey] = float(allreduce(torch.tensor(s, dtype=torch.float64), dist.ReduceOp.SUM))
            elif rt == ReduceType.MIN:
                vals = [float(v[m].min()) for v, m in items if m.any()] or [float("inf")]
                out[skey] = float(allreduce(torch.tensor(min(vals), dtype=torch.float64), dist.ReduceOp.MIN))
            elif rt == ReduceType.MAX:
                vals = [float(v[m].max()) for v, m in items if m.any()] or [float("-inf")]
                out[skey] = float(allreduce(torch.tensor(max(vals), dtype=torch.float64), dist.ReduceOp.MAX))
        if reset:
            self.denominators.clear()
            self.stats.clear()
            self.reduce_types.clear()
            self.denom_of.clear()
        return out


DEFAULT_TRACKER = DistributedStatsTracker()
denominator = DEFAULT_TRACKER.denominator
stat = DEFAULT_TRACKER.stat
scalar = DEFAULT_TRACKER.scalar
scope = DEFAULT_TRACKER.scope
export = DEFAULT_TRACKER.export
record_timing = DEFAULT_TRACKER.record_timing

TRACKERS: Dict[str, DistributedStatsTracker] = {}


def get(name: str) -> DistributedStatsTracker:
    """The named tracker, made on first use (one per subsystem that wants its own scope tree)."""
    if name not in TRACKERS:
        TRACKERS[name] = DistributedStatsTracker(name)
    return TRACKERS[name]


def export_all(reduce_group=None, reset: bool = True) -> Dict[str, float]:
    """The default tracker's export merged with every named tracker's."""
    out = DEFAULT_TRACKER.export(reduce_group=reduce_group, reset=reset)
    for tracker in TRACKERS.values():
        out.update(tracker.export(reduce_group=reduce_group, reset=reset))
    return out
