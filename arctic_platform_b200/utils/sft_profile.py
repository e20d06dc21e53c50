"""Opt-in phase timing for SFT steps: ``ARL_SFT_PROFILE=1`` accumulates milliseconds per bucket
(``serialize, rpc, h2d, fwd, bwd, loss, step``) and merges them into the returned metrics under
``_profile_ms`` (arctic_platform/common/utils/sft_profile.py:33-110 in the reference)."""
from __future__ import annotations

import contextlib
import os
import time
from typing import Dict, Optional

BUCKETS = ("serialize", "rpc", "h2d", "fwd", "bwd", "loss", "step")
_acc: Dict[str, float] = {}


def enabled() -> bool:
    return os.environ.get("ARL_SFT_PROFILE", "0") == "1"


@contextlib.contextmanager
def timed(name: str, sync_cuda: bool = True):
    if not enabled():
        yield
        return
    if sync_cuda:
        _sync()
    t0 = time.perf_counter()
    try:
        yield
    finally:
        if sync_cuda:
            _sync()
        _acc[name] = _acc.get(name, 0.0) + (time.perf_counter() - t0) * 1e3


def _sync() -> None:
    try:
        import torch
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    except Exception:
        pass


def snapshot(reset: bool = True) -> Dict[str, float]:
    out = dict(_acc)
    if reset:
        _acc.clear()
    return out


def merge_into(metrics: dict, reset: bool = True) -> dict:
    if enabled():
        prof = metrics.setdefault("_profile_ms", {})
        for k, v in snapshot(reset).items():
            prof[k] = prof.get(k, 0.0) + v
    return metrics


def format_line(prefix_or_buckets, buckets: Optional[Dict[str, float]] = None) -> str:
    """``format_line(buckets)`` -> the buckets by share, largest first; ``format_line(prefix, buckets)`` -> the same
    behind ``[ARL_SFT_PROFILE] prefix:`` (the line the reference prints)."""
    profile_ms = prefix_or_buckets if buckets is None else buckets
    total = sum(profile_ms.values()) or 1.0
    body = " ".join(f"{k}={v:.1f}ms({100 * v / total:.0f}%)" for k, v in sorted(profile_ms.items(), key=lambda kv: -kv[1]))
    return body if buckets is None else f"[ARL_SFT_PROFILE] {prefix_or_buckets}: {body}"


def take_last() -> Dict[str, float]:
    """The buckets accumulated since the last call, cleared (empty when profiling is off)."""
    return snapshot(reset=True) if enabled() else {}


def merge_into_metrics(metrics: Optional[dict], extra: Optional[Dict[str, float]] = None) -> dict:
    """A copy of ``metrics`` with ``_profile_ms`` (the last step's buckets plus ``extra``) attached for the wire."""
    out = dict(metrics or {})
    if not enabled():
        return out
    prof = take_last()
    prof.update(extra or {})
    if prof:
        out["_profile_ms"] = {k: round(v, 3) for k, v in sorted(prof.items())}
    return out


def maybe_print(prefix: str, buckets: Optional[Dict[str, float]] = None) -> None:
    if not enabled():
        return
    data = buckets if buckets is not None else snapshot(reset=False)
    if data:
        print(format_line(prefix, data), flush=True)
