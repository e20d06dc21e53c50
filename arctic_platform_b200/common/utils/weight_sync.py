"""Trainer -> sampler weight hand-over strategies used by the job server.

* ``sync_weights_in_process``  -- source and target workers live in this process on the same GPU: one kernel copies
  (stages 0-2) or gathers (stage 3) the flat parameter buffer into the sampler's buffer.  This is what the
  reference's zero-copy CUDA-IPC path (``sync_weights_cuda_ipc``) achieves for colocated engines.
* ``sync_weights_cuda_ipc``    -- different processes on one node (split placement): the trainer exports an IPC handle
  of its flat parameter buffer, the sampler maps it and runs the same one-kernel hand-over on it over NVLink (with its
  tensor-parallel slicing and fp8 requantisation); no tensor travels through the server.
* ``sync_weights_bulk``        -- different processes: one RPC returns every tensor, one RPC loads them.
* ``sync_weights_low_mem``     -- different processes, bounded peak memory: buckets of at most ``bucket_bytes``
  (the reference's ``sync_weights_cuda_ipc_low_mem`` streams one parameter per round trip).
* ``sync_weights_cpu_file``    -- through a safetensors file, normally on tmpfs (``sync_weights_cpu_file`` /
  ``load_weights_from_shm_path`` in the reference).

Every strategy can stage the target's wake-up: weights first, KV cache afterwards, so the two never have to fit next
to the incoming copy.  Contract of arctic_platform/common/utils/weight_sync.py:47-187.
"""
from __future__ import annotations

import os
import tempfile
import uuid
from typing import Any, Dict, Optional


def _staged(dst, fn):
    """wake(weights) -> transfer -> wake(kv_cache) -> reset prefix cache, when the target is a sampler."""
    has_sampler = bool(dst.call("has_sampler")) if hasattr(dst, "call") else False
    if has_sampler:
        dst.call("wake_inference", ["weights"])
    n = fn()
    if has_sampler:
        dst.call("wake_inference", ["kv_cache"])
        dst.call("reset_prefix_cache")
    return n


def load_staged(dst, weights) -> int:
    """Loads already gathered ``(name, tensor)`` pairs into one target with the staged wake-up."""
    return _staged(dst, lambda: dst.call("load_weights", weights))


def sync_weights_in_process(src, dst) -> int:
    return src.obj.sync_weights_to(dst.obj)


def sync_weights_cuda_ipc(src, dst, staged: bool = True) -> Optional[int]:
    """``None`` when the source cannot export its storage (sharded or symmetric-memory buffers) or the target is not
    the paged CUDA sampler: the caller then picks another strategy."""
    try:
        info = src.call("export_ipc_source")
    except Exception:
        info = None
    if not info:
        return None

    def run():
        return dst.call("sync_from_ipc", [info])
    try:
        return _staged(dst, run) if staged else run()
    except RuntimeError:
        return None


def sync_weights_bulk(src, dst, staged: bool = False) -> int:
    run = lambda: dst.call("load_weights", src.call("get_weights"))
    return _staged(dst, run) if staged else run()


def sync_weights_low_mem(src, dst, bucket_bytes: int = 256 << 20, staged: bool = False) -> int:
    def run():
        n = 0
        for names in src.call("weight_buckets", bucket_bytes):
            n += dst.call("load_weights", src.call("get_weight_bucket", names))
        return n
    return _staged(dst, run) if staged else run()


def sync_weights_cpu_file(src, dst, directory: Optional[str] = None, staged: bool = False) -> int:
    root = directory or ("/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir())
    path = os.path.join(root, f"apb200-weights-{uuid.uuid4().hex}.safetensors")

    def run():
        try:
            src.call("save_weights_to_path", path)
            return dst.call("load_weights_from_path", path)
        finally:
            if os.path.exists(path):
                os.remove(path)
    return _staged(dst, run) if staged else run()


def same_rank_process(src, dst) -> bool:
    a, b = getattr(src, "actor", None), getattr(dst, "actor", None)
    return a is not None and a is b


def sync_pair(src, dst, cuda_ipc: Optional[bool] = None, low_memory: Optional[bool] = None,
              via_file: bool = False, bucket_bytes: int = 256 << 20) -> Dict[str, Any]:
    """Picks the strategy for one (source worker, target worker) pair and reports which one ran."""
    same_process = getattr(src, "obj", None) is not None and getattr(dst, "obj", None) is not None
    if same_process and cuda_ipc is not False:
        return {"strategy": "in_process", "num_tensors": sync_weights_in_process(src, dst)}
    if same_rank_process(src, dst) and cuda_ipc is not False:
        # both engines live in the same spawned rank process: the in-process kernel runs there
        return {"strategy": "in_process", "num_tensors": src.sync_to(dst)}
    if cuda_ipc is True and hasattr(src, "call") and hasattr(dst, "call"):
        n = sync_weights_cuda_ipc(src, dst)
        if n is not None:
            return {"strategy": "cuda_ipc", "num_tensors": n}
    if via_file:
        return {"strategy": "cpu_file", "num_tensors": sync_weights_cpu_file(src, dst)}
    if low_memory:
        return {"strategy": "low_mem", "num_tensors": sync_weights_low_mem(src, dst, bucket_bytes)}
    return {"strategy": "bulk", "num_tensors": sync_weights_bulk(src, dst)}
