"""Splitting a global batch over data-parallel workers and merging their answers.

``split_batch_for_ranks`` cuts every tensor along dim 0 (``torch.chunk`` semantics), injects the global
quantities each shard needs to normalise its loss (``dp_size``, ``batch_num_tokens``,
``global_batch_size``), rebuilds ``position_ids`` when the client dropped them to save bandwidth and,
when ``meta['load_balancer']`` is set, first reorders the samples so every rank gets whole prompt groups
of similar cost (ZoRRo load balancer).  The answers are merged in rank order and un-permuted.
Contract of arctic_platform/common/utils/batch.py:39-492 in the reference.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch


def tensorize(obj: Any) -> Any:
    """Lists of numbers -> tensors (recursively through dicts), everything else untouched."""
    if isinstance(obj, dict):
        return {k: tensorize(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)) and obj and all(isinstance(x, (int, float, list, tuple)) for x in obj):
        try:
            return torch.tensor(obj)
        except (ValueError, TypeError):
            return obj
    return obj


def detensorize(obj: Any) -> Any:
    """Tensors -> Python numbers / lists so a metrics dict is JSON-serialisable."""
    if torch.is_tensor(obj):
        return obj.item() if obj.numel() == 1 else obj.tolist()
    if isinstance(obj, dict):
        return {k: detensorize(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [detensorize(v) for v in obj]
    return obj


def reconstruct_position_ids_(batch: Dict[str, torch.Tensor]) -> None:
    """``position_ids = cumsum(attention_mask) - 1`` clipped at 0, in place, when missing."""
    if "position_ids" in batch or "attention_mask" not in batch:
        return
    m = batch["attention_mask"].long()
    batch["position_ids"] = (m.cumsum(-1) - 1).clamp_min(0) * m


def split_dict(batch: Dict[str, Any], n: int) -> List[Dict[str, Any]]:
    outs: List[Dict[str, Any]] = [dict() for _ in range(n)]
    for k, v in batch.items():
        if torch.is_tensor(v) and v.dim() > 0:
            parts = list(torch.chunk(v, n, dim=0))
            while len(parts) < n:
                parts.append(v[:0])
            for o, p in zip(outs, parts):
                o[k] = p
        else:
            for o in outs:
                o[k] = v
    return outs


def merge_dict_shards(shards: Sequence[Dict[str, Any]]) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    keys = []
    for s in shards:
        for k in s:
            if k not in keys:
                keys.append(k)
    for k in keys:
        vals = [s[k] for s in shards if k in s]
        if all(torch.is_tensor(v) for v in vals):
            if vals[0].dim() == 0:
                out[k] = torch.stack(vals)
            else:
                width = max(v.shape[1] for v in vals) if vals[0].dim() > 1 else None
                if width is not None and any(v.shape[1] != width for v in vals):
                    vals = [torch.nn.functional.pad(v, (0, width - v.shape[1])) for v in vals]
                out[k] = torch.cat(vals, 0)
        elif all(isinstance(v, list) for v in vals):
            out[k] = [x for v in vals for x in v]
        else:
            out[k] = vals[0]
    return out


def restore_batch_order(batch: Dict[str, Any], order: torch.Tensor) -> Dict[str, Any]:
    """Inverse of the permutation applied before splitting: row ``i`` of the result is the sample that was
    at position ``i`` of the client's batch."""
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel())
    out = {}
    for k, v in batch.items():
        out[k] = v[inv] if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == order.numel() else v
    return out


def shard_token_stats(shards: Sequence[Dict[str, Any]]) -> List[int]:
    return [int(s["attention_mask"].sum()) if "attention_mask" in s else 0 for s in shards]


def rank_token_stats(batch: Dict[str, Any], meta: Optional[Dict[str, Any]] = None) -> Dict[str, int]:
    """Valid-token summary of the shard one data-parallel rank received -- what to compare across ranks when one
    of them is the straggler (arctic_platform/common/utils/batch.py:25-52 in the reference)."""
    stats: Dict[str, int] = {}
    am = batch.get("attention_mask")
    if torch.is_tensor(am) and am.ndim == 2:
        lens = am.sum(dim=1).to(torch.int64)
        stats.update(valid_tokens=int(lens.sum()), batch_size=int(am.shape[0]), seq_len_min=int(lens.min()),
                     seq_len_max=int(lens.max()))
    cu = batch.get("cu_seqlens")
    if torch.is_tensor(cu) and cu.numel() > 0:
        stats["cu_seqlens_packed"] = int(cu[-1])
    ids = batch.get("input_ids")
    if torch.is_tensor(ids) and (ids.ndim == 1 or (ids.ndim == 2 and ids.shape[0] == 1)):
        stats["packed_tokens"] = int(ids.numel())
    for key in ("loss_mask", "response_mask"):
        m = batch.get(key)
        if torch.is_tensor(m):
            stats[f"{key}_tokens"] = int(m.sum())
    bnt = (meta or {}).get("batch_num_tokens")
    if bnt is not None:
        stats["meta_batch_num_tokens"] = int(bnt)
    return stats


def log_dp_shard_tokens(rank: int, tag: str, batch: Dict[str, Any], meta: Optional[Dict[str, Any]] = None) -> None:
    """Prints :func:`rank_token_stats` when ``ARL_LOG_DP_SHARD_TOKENS`` is set (silent otherwise)."""
    import os
    if not os.environ.get("ARL_LOG_DP_SHARD_TOKENS"):
        return
    stats = rank_token_stats(batch, meta)
    if stats:
        print(f"[{rank}] [DP-shard] {tag}: " + " ".join(f"{k}={v}" for k, v in sorted(stats.items())), flush=True)


def split_batch_for_ranks(batch, meta: Dict[str, Any], n: int) -> Tuple[List[Any], Optional[torch.Tensor]]:
    """Returns ``(shards, order)``; ``order`` is the permutation applied to the samples (or None).
    ``meta`` is updated in place with ``dp_size`` and the global normalisers."""
    meta.setdefault("dp_size", n)
    if isinstance(batch, (list, tuple)):
        # client-side micro-batches: each micro-batch is split on its own, rank r gets the list of its parts
        per_mb = [split_batch_for_ranks(mb, dict(meta), n)[0] for mb in batch]
        return [[mb[r] for mb in per_mb] for r in range(n)], None
    batch = dict(batch)
    if meta.get("drop_position_ids"):
        reconstruct_position_ids_(batch)
    if "response_mask" in batch and meta.get("batch_num_tokens") is None:
        meta["batch_num_tokens"] = float(batch["response_mask"].sum())
    if "input_ids" in batch and meta.get("global_batch_size") is None:
        meta["global_batch_size"] = float(batch["input_ids"].shape[0])
    order = None
    if n > 1 and meta.get("load_balancer") and "input_ids" in batch:
        from ...rl.zorro_train.seqlen_balancing import reorg_global_batch
        batch, order = reorg_global_batch(batch, meta, n)
    return split_dict(batch, n), order


# ------------------------------------------------------------------ the rest of the reference's helper names
def unpack_batch(payload: Dict[str, Any]) -> Tuple[dict, Any, Dict[str, Any], Optional[dict]]:
    """``(args, batch, meta, processing)`` of a call payload (``args`` is always empty: calls take keyword data)."""
    return {}, payload["batch"], payload.get("meta") or {}, payload.get("processing")


def ray_split_batch(payload: Dict[str, Any], num_workers: int) -> Tuple[List[Dict[str, Any]], Optional[torch.Tensor]]:
    """A decoded call payload (``{"batch", "meta", "processing"}``) -> per-rank payloads (same ``meta`` and
    ``processing`` on every rank, the batch split by ``split_batch_for_ranks``) and the permutation that was applied
    to the rows, if any."""
    _args, batch, meta, processing = unpack_batch(payload)
    meta = dict(meta)
    shards, order = split_batch_for_ranks(batch, meta, num_workers)
    return [{"batch": s, "meta": dict(meta), "processing": processing} for s in shards], order


def http_split_batch(frame: bytes, num_workers: int) -> Tuple[List[Dict[str, Any]], Optional[torch.Tensor]]:
    """The same for one DSSST1 request frame as it arrives over HTTP."""
    from ... import wire
    return ray_split_batch(wire.loads(frame), num_workers)


def get_reverse_idx(idx_map) -> List[int]:
    """The inverse permutation: ``out[idx_map[i]] = i``."""
    out = [0] * len(idx_map)
    for i, j in enumerate(idx_map):
        out[int(j)] = i
    return out


def dump_dict_payload(payload: Dict[str, Any], tag: str, out=None) -> None:
    """One line per entry (tensors by shape / dtype, everything else by value) when ``ARL_DUMP_PAYLOADS`` is set;
    silent otherwise."""
    if not os.environ.get("ARL_DUMP_PAYLOADS"):
        return
    import sys
    out = out or sys.stderr
    for k, v in payload.items():
        what = f"tensor{tuple(v.shape)} {v.dtype}" if torch.is_tensor(v) else repr(v)[:200]
        out.write(f"{tag}: {k} = {what}\n")


def __getattr__(name: str):
    # metric reducers live in ``metrics.py``; the reference reaches them through this module
    if name in ("combine_metric_shards", "combine_metric_microbatches", "finalize_fwd_bwd_metrics"):
        from . import metrics
        return getattr(metrics, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
