"""Debug and profiling helpers: memory reports, rank-filtered printing, synchronised timers, a profiler
context and full-determinism switch (arctic_platform/common/utils/debug.py:56-483 in the reference)."""
from __future__ import annotations

import contextlib
import cProfile
import fcntl
import gc
import io
import logging
import os
import pstats
import random
import time
from typing import Dict, Optional

import torch
import torch.distributed as dist

DISABLE_DEBUG = os.environ.get("APB_DEBUG", "0") != "1"


def get_mem_metrics() -> Dict[str, float]:
    """Torch allocator, device (NVML via torch) and host RSS figures in GiB."""
    out: Dict[str, float] = {}
    if torch.cuda.is_available():
        gib = 2 ** 30
        out["torch_allocated_gib"] = torch.cuda.memory_allocated() / gib
        out["torch_max_allocated_gib"] = torch.cuda.max_memory_allocated() / gib
        out["torch_reserved_gib"] = torch.cuda.memory_reserved() / gib
        free, total = torch.cuda.mem_get_info()
        out["device_used_gib"] = (total - free) / gib
        out["device_total_gib"] = total / gib
    try:
        import psutil
        out["host_rss_gib"] = psutil.Process().memory_info().rss / 2 ** 30
    except Exception:
        pass
    return out


def see_memory_usage(message: str, force: bool = False, ranks=(0,)) -> Optional[Dict[str, float]]:
    if DISABLE_DEBUG and not force:
        return None
    rank = dist.get_rank() if dist.is_initialized() else 0
    if ranks is not None and rank not in ranks:
        return None
    gc.collect()
    m = get_mem_metrics()
    print(f"[mem][rank {rank}] {message}: " + " ".join(f"{k}={v:.2f}" for k, v in m.items()), flush=True)
    return m


def printflock(*args, **kwargs) -> None:
    """print() under an exclusive file lock so lines of concurrent ranks do not interleave."""
    with open(__file__, "r") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            print(*args, **kwargs, flush=True)
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def pr(*args, force: bool = False, **kwargs) -> None:
    if DISABLE_DEBUG and not force:
        return
    rank = dist.get_rank() if dist.is_initialized() else 0
    printflock(f"[{rank}]", *args, **kwargs)


def pr0(*args, force: bool = False, **kwargs) -> None:
    if (dist.get_rank() if dist.is_initialized() else 0) == 0:
        pr(*args, force=force, **kwargs)


def debug_gathered_tensor(t: torch.Tensor, name: str = "", group=None) -> Dict[str, float]:
    """Norm / min / max of a tensor, all-reduced so every rank reports the same numbers."""
    stats = torch.tensor([t.float().pow(2).sum(), t.float().min(), -t.float().max()], dtype=torch.float64,
                         device=t.device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        sq = stats[:1].clone()
        dist.all_reduce(sq, group=group)
        mm = stats[1:].clone()
        dist.all_reduce(mm, op=dist.ReduceOp.MIN, group=group)
        stats = torch.cat([sq, mm])
    out = {"norm": float(stats[0].sqrt()), "min": float(stats[1]), "max": float(-stats[2])}
    pr0(f"{name}: {out}")
    return out


class SynchronizedWallClockTimer:
    """Named timers that synchronise the device around start/stop so wall time brackets GPU work."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self._start: Dict[str, float] = {}
        self.elapsed_ms: Dict[str, float] = {}
        self.counts: Dict[str, int] = {}

    @staticmethod
    def _sync() -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def start(self, name: str) -> str:
        if self.enabled:
            self._sync()
            self._start[name] = time.perf_counter()
        return name

    def stop(self, name: str) -> float:
        if not self.enabled or name not in self._start:
            return 0.0
        self._sync()
        ms = (time.perf_counter() - self._start.pop(name)) * 1e3
        self.elapsed_ms[name] = self.elapsed_ms.get(name, 0.0) + ms
        self.counts[name] = self.counts.get(name, 0) + 1
        return ms

    def stop_and_print_elapsed(self, name: str) -> float:
        ms = self.stop(name)
        if self.enabled:
            pr0(f"{name}: {ms:.2f} ms", force=True)
        return ms

    def summary(self, reset: bool = False) -> Dict[str, float]:
        out = dict(self.elapsed_ms)
        if reset:
            self.elapsed_ms.clear()
            self.counts.clear()
        return out


class SynchronizedWallClockTimerDummy:
    """Drop-in no-op used when timers are switched off."""

    def __getattr__(self, _name):
        return lambda *a, **k: 0.0


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True):
    on = enabled and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class ProfilerContext:
    """``type="torch"`` -> torch.profiler (CPU + CUDA activities, trace written to ``out_dir``),
    ``type="c"`` -> cProfile (top functions printed on exit), ``type="none"`` -> nothing."""

    def __init__(self, type: str = "none", out_dir: str = "/tmp/apb-prof", name: str = "trace", top: int = 30):
        if type not in ("none", "c", "torch"):
            raise ValueError(f"unknown profiler type {type!r}")
        self.type, self.out_dir, self.name, self.top = type, out_dir, name, top
        self._prof = None
        self.report: Optional[str] = None

    def __enter__(self):
        if self.type == "c":
            self._prof = cProfile.Profile()
            self._prof.enable()
        elif self.type == "torch":
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(activities=acts, with_stack=True)
            self._prof.__enter__()
        return self

    def __exit__(self, *exc):
        if self.type == "c":
            self._prof.disable()
            buf = io.StringIO()
            pstats.Stats(self._prof, stream=buf).sort_stats("cumulative").print_stats(self.top)
            self.report = buf.getvalue()
        elif self.type == "torch":
            self._prof.__exit__(*exc)
            os.makedirs(self.out_dir, exist_ok=True)
            path = os.path.join(self.out_dir, f"{self.name}.json")
            self._prof.export_chrome_trace(path)
            self.report = path
        return False


class MemoryHistory:
    """Allocator history of the block as a snapshot file (open it at pytorch.org/memory_viz): every allocation and
    free with its stack while the block runs, then one ``<out_dir>/<name>.pickle``.  ``enabled=False`` or no GPU: does
    nothing.  The reference has this as a hard-coded switch around one training call
    (arctic_platform/common/deepspeed_worker.py:374-378, 522-529)."""

    def __init__(self, enabled: bool, out_dir: str = "/tmp/apb-mem-prof", name: str = "rank-0", max_entries: int = 100_000):
        self.enabled = bool(enabled) and torch.cuda.is_available()
        self.out_dir, self.name, self.max_entries = out_dir, name, max_entries
        self.path: Optional[str] = None

    def __enter__(self):
        if self.enabled:
            torch.cuda.memory._record_memory_history(max_entries=self.max_entries)
        return self

    def __exit__(self, *exc):
        if self.enabled:
            try:
                os.makedirs(self.out_dir, exist_ok=True)
                self.path = os.path.join(self.out_dir, f"{self.name}.pickle")
                torch.cuda.memory._dump_snapshot(self.path)
            finally:
                torch.cuda.memory._record_memory_history(enabled=None)
        return False


def enable_full_determinism(seed: int, warn_only: bool = True) -> None:
    """Seeds every RNG and switches PyTorch to deterministic algorithms."""
    random.seed(seed)
    try:
        import numpy as np
        np.random.seed(seed)
    except Exception:
        pass
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    os.environ["PYTHONHASHSEED"] = str(seed)
    torch.use_deterministic_algorithms(True, warn_only=warn_only)
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False


# ----------------------------------------------------------------------------- opt-in diagnostics
_moe_imbalance = {"max_chunk": 0, "total": 0, "n_dispatch": 0}


def moe_imbalance_enabled() -> bool:
    """``DSS_MOE_IMBALANCE`` (the reference's name, arctic_platform/model/implementations/qwen35/gpu/debug.py:14) or
    ``APB_MOE_IMBALANCE``.  Read at call time, so a test can switch it."""
    return bool(os.environ.get("DSS_MOE_IMBALANCE") or os.environ.get("APB_MOE_IMBALANCE"))


def maybe_record_recv_tokens(num_recv_tokens: int) -> None:
    """One expert-parallel dispatch received ``num_recv_tokens`` rows on this rank.  The largest value sizes the
    fp32 combine buffer; its spread across ranks is the routing imbalance."""
    if not moe_imbalance_enabled():
        return
    _moe_imbalance["max_chunk"] = max(_moe_imbalance["max_chunk"], int(num_recv_tokens))
    _moe_imbalance["total"] += int(num_recv_tokens)
    _moe_imbalance["n_dispatch"] += 1


def maybe_log_moe_imbalance(rank: int) -> Optional[Dict[str, float]]:
    """Logs and resets this rank's dispatch counters after a forward/backward request (grep ``MOE_IMBALANCE`` and
    compare max / min across ranks).  Returns what it logged, ``None`` when the switch is off."""
    if not moe_imbalance_enabled():
        return None
    stats: Dict[str, float] = dict(_moe_imbalance)
    _moe_imbalance.update(max_chunk=0, total=0, n_dispatch=0)
    if torch.cuda.is_available():
        stats["peak_alloc_GiB"] = torch.cuda.max_memory_allocated() / 2 ** 30
        stats["peak_reserved_GiB"] = torch.cuda.max_memory_reserved() / 2 ** 30
    logging.getLogger(__name__).info(
        "MOE_IMBALANCE rank=%d max_chunk_recv=%d total_recv=%d n_dispatch=%d peak_alloc_GiB=%.2f peak_reserved_GiB=%.2f",
        rank, stats["max_chunk"], stats["total"], stats["n_dispatch"], stats.get("peak_alloc_GiB", 0.0),
        stats.get("peak_reserved_GiB", 0.0))
    return stats


def drop_stale_nccl_topo_file() -> Optional[str]:
    """A network plugin passes its generated topology to NCCL through ``NCCL_TOPO_FILE=/proc/self/fd/<n>``.  That
    handle means something only in the process that created it; a child that inherits it would load an unrelated
    file and the rendezvous would hang.  Called before the process group is created; an administrator's static
    path is left alone.  Returns the dropped value (arctic_platform/common/deepspeed_worker.py:139-153)."""
    topo = os.environ.get("NCCL_TOPO_FILE", "")
    if topo.startswith("/proc/self/fd/"):
        logging.getLogger(__name__).warning("dropping inherited stale NCCL_TOPO_FILE=%s", topo)
        os.environ.pop("NCCL_TOPO_FILE", None)
        return topo
    return None


# ------------------------------------------------------------------------------------------------- more accessors
def get_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else int(os.environ.get("RANK", 0))


def get_device_id() -> int:
    """The physical index of this process's current device: ``CUDA_VISIBLE_DEVICES`` maps logical to physical ids,
    which is what NVML and ``nvidia-smi`` number by."""
    if not torch.cuda.is_available():
        return 0
    logical = torch.cuda.current_device()
    visible = os.environ.get("CUDA_VISIBLE_DEVICES", "").strip()
    if visible:
        ids = [v.strip() for v in visible.split(",") if v.strip()]
        if logical < len(ids) and ids[logical].isdigit():
            return int(ids[logical])
    return logical


def get_nvml_mem() -> Dict[str, float]:
    """Device memory as the driver sees it (every process on the GPU counted), in GiB; ``{}`` without a GPU.
    Read through ``torch.cuda.mem_get_info`` -- the same figures NVML reports, no second library handle."""
    if not torch.cuda.is_available():
        return {}
    free, total = torch.cuda.mem_get_info()
    gib = 2 ** 30
    return {"used_gib": (total - free) / gib, "free_gib": free / gib, "total_gib": total / gib}


def gc_empty_accelerator_cache() -> None:
    """Python garbage first (drops tensors that only cycles keep alive), then the allocator's cached blocks."""
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def print_rank(*msg, force: bool = True, ranks=None, **kwargs) -> None:
    """``pr`` limited to ``ranks`` (None = every rank)."""
    if ranks is not None and get_rank() not in ranks:
        return
    pr(*msg, force=force, **kwargs)


def print_rank0(*msg, force: bool = True, **kwargs) -> None:
    print_rank(*msg, force=force, ranks=(0,), **kwargs)


class SynchronizedWallClockTimerSimple(SynchronizedWallClockTimer):
    """Timers for step loops: ``timers(name).start()`` / ``.stop()`` handles, and ``log(names)`` that prints one line
    with the mean milliseconds of each named timer since the last ``log`` and resets them."""

    class _Handle:
        def __init__(self, owner: "SynchronizedWallClockTimerSimple", name: str):
            self.owner, self.name = owner, name

        def start(self):
            self.owner.start(self.name)
            return self

        def stop(self, record: bool = True) -> float:
            return self.owner.stop(self.name)

        def elapsed(self, reset: bool = True) -> float:
            ms = self.owner.elapsed_ms.get(self.name, 0.0)
            if reset:
                self.owner.elapsed_ms.pop(self.name, None)
                self.owner.counts.pop(self.name, None)
            return ms

    def __call__(self, name: str) -> "_Handle":
        return self._Handle(self, name)

    def means(self, names=None, reset: bool = True) -> Dict[str, float]:
        names = list(names) if names is not None else list(self.elapsed_ms)
        out = {n: self.elapsed_ms[n] / max(1, self.counts.get(n, 1)) for n in names if n in self.elapsed_ms}
        if reset:
            for n in out:
                self.elapsed_ms.pop(n, None)
                self.counts.pop(n, None)
        return out

    def log(self, names=None, reset: bool = True, ranks=(0,)) -> str:
        line = " | ".join(f"{n}: {ms:.2f}" for n, ms in self.means(names, reset).items())
        if line and self.enabled:
            print_rank(f"time (ms) | {line}", ranks=ranks)
        return line


class SynchronizedWallClockTimerSimpleDummy:
    """No-op twin: ``timers(name).start()`` and friends cost nothing."""

    class _Handle:
        def start(self):
            return self

        def stop(self, record: bool = True) -> float:
            return 0.0

        def elapsed(self, reset: bool = True) -> float:
            return 0.0

    def __call__(self, name: str) -> "_Handle":
        return self._Handle()

    def log(self, *a, **k) -> str:
        return ""

    def means(self, *a, **k) -> Dict[str, float]:
        return {}
