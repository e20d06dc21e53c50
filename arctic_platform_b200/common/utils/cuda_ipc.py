"""Per-rank CUDA-IPC exports of a training job, merged into what one sampler process needs.

Every trainer rank answers ``export_ipc_source`` with ``{"handle", "offset", "layout", "device"}`` for its flat bf16
parameter buffer (``engine/worker.py``).  A sampler that maps them (``sync_from_ipc``) wants the sources in trainer
rank order, all describing the same layout, each from a different GPU.  ``merge_ipc_sources`` builds that list from the
ranks' answers and refuses inconsistent sets; a rank that could not export (``None``) makes the whole set unusable --
the caller then falls back to shipping tensors -- because a hand-over from some of the shards is not a hand-over.

The reference merges per-parameter ``{gpu_uuid: handle}`` dictionaries
(``merge_cuda_ipc_payloads``, arctic_platform/common/utils/cuda_ipc.py:24-62); here one handle per rank covers every
parameter, so the merge is a list and the per-parameter addressing is the sync table's job.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

LAYOUT_KEYS = ("total", "world")


def layout_signature(layout: Dict[str, Any]) -> tuple:
    return tuple(layout.get(k) for k in LAYOUT_KEYS) + (layout.get("zero3") is not None, len(layout.get("params", {})))


def merge_ipc_sources(results: Sequence[Optional[Dict[str, Any]]]) -> Optional[List[Dict[str, Any]]]:
    """Answers of all trainer ranks (rank order) -> the source list for ``sync_from_ipc``, or ``None`` when any rank
    could not export.  Raises ``ValueError`` for answers that do not belong together."""
    if not results or any(r is None for r in results):
        return None
    sig = layout_signature(results[0]["layout"])
    seen_handles = set()
    for rank, r in enumerate(results):
        for key in ("handle", "offset", "layout"):
            if key not in r:
                raise ValueError(f"rank {rank}: the export carries no {key!r}")
        if layout_signature(r["layout"]) != sig:
            raise ValueError(f"rank {rank} describes another parameter layout than rank 0")
        h = bytes(r["handle"]) + int(r["offset"]).to_bytes(8, "little")
        if h in seen_handles:
            raise ValueError(f"rank {rank} exported the same buffer as an earlier rank")
        seen_handles.add(h)
    world = results[0]["layout"].get("world")
    if world is not None and int(world) != len(results):
        raise ValueError(f"the layout was built for {world} trainer ranks, {len(results)} answered")
    return [dict(r) for r in results]


def merge_cuda_ipc_payloads(results: Sequence[Optional[Dict[str, Any]]]) -> Dict[str, Any]:
    """The reference's entry point name.  ``{"sources": [...] | None, "num_ranks": n, "num_params": p}``."""
    live = [r for r in results if r]
    sources = merge_ipc_sources(list(results)) if results else None
    n_params = len(live[0]["layout"].get("params", {})) if live else 0
    return {"sources": sources, "num_ranks": len(live), "num_params": n_params}
