"""Load balancing of a global RL batch over data-parallel ranks, prompt-group aware.

A ZoRRo micro-batch costs ``P + sum(R_i)`` linear work and ``P^2 + sum((P + R_i) * R_i)`` attention work
per prompt group rather than per sample, so the unit of placement is the *group*.  This module provides

* ``karmarkar_karp`` / ``greedy_partition`` / ``get_seqlen_balanced_partitions`` -- k-way partitions of
  sequence lengths (optionally with equal item counts),
* ``create_prompt_groups`` -- groups by prompt content with a cap on rollouts per group,
* ``compute_group_costs`` -- the linear/quadratic blend above,
* ``reorg_global_batch`` -- permutes a padded batch so that ``torch.chunk`` over ranks hands every rank
  whole groups, the same number of samples and similar cost; returns the permutation for un-doing it,
* ``rearrange_micro_batches_with_dedup`` -- token-budget micro-batches made of whole groups.

Behavioural contract of arctic_platform/rl/zorro_train/seqlen_balancing.py:76-953 in the reference.
"""
from __future__ import annotations

import ctypes
import heapq
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ...ops import _lib
from .layout import find_prompt_groups


# ----------------------------------------------------------------------------- number partitioning
def greedy_partition(sizes: Sequence[int], k: int, equal_size: bool = False) -> List[List[int]]:
    """Largest-first into the lightest bin; with ``equal_size`` every bin gets ``len(sizes) / k`` items."""
    n = len(sizes)
    if equal_size and n % k:
        raise ValueError(f"{n} items cannot be split into {k} equal bins")
    cap = n // k if equal_size else n
    order = sorted(range(n), key=lambda i: -sizes[i])
    bins: List[List[int]] = [[] for _ in range(k)]
    load = [0] * k
    for i in order:
        cands = [b for b in range(k) if len(bins[b]) < cap]
        b = min(cands, key=lambda j: (load[j], j))
        bins[b].append(i)
        load[b] += sizes[i]
    return bins


def karmarkar_karp(sizes: Sequence[int], k: int, equal_size: bool = False) -> List[List[int]]:
    """Largest differencing method generalised to ``k`` parts: repeatedly merge the two partial solutions
    with the largest spread, pairing the heaviest part of one with the lightest of the other."""
    n = len(sizes)
    if equal_size and n % k:
        raise ValueError(f"{n} items cannot be split into {k} equal bins")
    if equal_size:
        # process items in blocks of k so every part receives exactly one item per block
        order = sorted(range(n), key=lambda i: sizes[i])
        states = []
        for off in range(0, n, k):
            block = order[off:off + k]
            parts = [([i], sizes[i]) for i in block]
            states.append(parts)
    else:
        states = [[([i], sizes[i])] + [([], 0)] * (k - 1) for i in range(n)]
    if not states:
        return [[] for _ in range(k)]
    heap = []
    for idx, parts in enumerate(states):
        parts = sorted(parts, key=lambda p: -p[1])
        heap.append((-(parts[0][1] - parts[-1][1]), idx, parts))
    heapq.heapify(heap)
    counter = len(states)
    while len(heap) > 1:
        _, _, a = heapq.heappop(heap)
        _, _, b = heapq.heappop(heap)
        merged = [(a[i][0] + b[k - 1 - i][0], a[i][1] + b[k - 1 - i][1]) for i in range(k)]
        merged.sort(key=lambda p: -p[1])
        heapq.heappush(heap, (-(merged[0][1] - merged[-1][1]), counter, merged))
        counter += 1
    return [sorted(p[0]) for p in heap[0][2]]


def get_seqlen_balanced_partitions(seqlens: Sequence[int], k_partitions: int, equal_size: bool = False) -> List[List[int]]:
    if len(seqlens) < k_partitions:
        raise ValueError(f"{len(seqlens)} sequences cannot fill {k_partitions} partitions")
    parts = karmarkar_karp(list(seqlens), k_partitions, equal_size)
    assert sorted(i for p in parts for i in p) == list(range(len(seqlens)))
    return parts


def ceildiv(a: int, b: int) -> int:
    return -(a // -b)


def roundup_divisible(a: int, b: int) -> int:
    """``a`` rounded up to a multiple of ``b``."""
    return ceildiv(a, b) * b


def compute_variation(costs: Sequence[float]) -> Tuple[float, float, float]:
    """How uneven a list of costs is: ``(max, max / min, (max - median) / median)``; the last is 0 when the largest
    item is typical and grows with a heavy outlier."""
    import statistics
    ordered = sorted(costs)
    med = statistics.median(ordered)
    return ordered[-1], (ordered[-1] / ordered[0] if ordered[0] else float("inf")), ((ordered[-1] - med) / med if med else 0.0)


def log_seqlen_unbalance(seqlens: Sequence[int], partitions: List[List[int]], prefix: str = "") -> Dict[str, float]:
    loads = [sum(seqlens[i] for i in p) for p in partitions]
    return {f"{prefix}/min": float(min(loads)), f"{prefix}/max": float(max(loads)),
            f"{prefix}/minmax_diff": float(max(loads) - min(loads)),
            f"{prefix}/balance": float(min(loads) / max(1, max(loads)))}


# ----------------------------------------------------------------------------- prompt groups
def create_prompt_groups(input_ids: torch.Tensor, attention_mask: torch.Tensor, response_length: int,
                         max_group_size: Optional[int] = None, max_token_len: Optional[int] = None
                         ) -> List[List[int]]:
    """Sample indices grouped by identical prompt; groups larger than ``max_group_size`` are split.
    ``max_token_len`` (a micro-batch token budget) must fit one prompt plus ``max_group_size`` responses."""
    gid = find_prompt_groups(input_ids, response_length)
    groups: Dict[int, List[int]] = {}
    for b, g in enumerate(gid.tolist()):
        groups.setdefault(g, []).append(b)
    out: List[List[int]] = []
    P = input_ids.shape[1] - response_length
    for g in sorted(groups):
        mem = groups[g]
        cap = max_group_size or len(mem)
        if max_token_len is not None:
            p_len = int(attention_mask[mem[0], :P].sum())
            if p_len + response_length * min(cap, len(mem)) > max_token_len and cap >= 1:
                fit = (max_token_len - p_len) // max(1, response_length)
                if fit < 1:
                    raise ValueError(f"max_token_len={max_token_len} cannot hold a prompt of {p_len} tokens plus one "
                                     f"response of {response_length}")
                cap = min(cap, fit)
        for s in range(0, len(mem), cap):
            out.append(mem[s:s + cap])
    return out


def compute_group_costs(groups: List[List[int]], prompt_lens: Sequence[int], response_lens: Sequence[int],
                        quadratic_weight: float = 0.0) -> List[float]:
    """``(1-w) * (P + sum R) + w * (P^2 + sum (P + R) R) / normaliser`` per group."""
    costs = []
    for mem in groups:
        P = float(prompt_lens[mem[0]])
        Rs = [float(response_lens[i]) for i in mem]
        lin = P + sum(Rs)
        quad = P * P + sum((P + r) * r for r in Rs)
        costs.append((1.0 - quadratic_weight) * lin + quadratic_weight * quad / max(1.0, lin))
    return costs


def reorg_global_batch(batch: Dict[str, torch.Tensor], meta: dict, n_ranks: int
                       ) -> Tuple[Dict[str, torch.Tensor], torch.Tensor]:
    """Returns ``(permuted_batch, order)`` where ``permuted[i] = batch[order[i]]`` and the first ``B / n``
    rows belong to rank 0, etc.  Groups are atomic when that is compatible with equal sample counts;
    otherwise the batch is returned unchanged with the identity permutation."""
    ids = batch["input_ids"]
    B = ids.shape[0]
    R = int(meta.get("response_length") or (batch["response_mask"].shape[1] if "response_mask" in batch
                                             else batch["responses"].shape[1]))
    mask = batch.get("attention_mask", torch.ones_like(ids))
    P = ids.shape[1] - R
    groups = create_prompt_groups(ids, mask, R, meta.get("max_rollouts"))
    p_lens = mask[:, :P].sum(-1).tolist()
    r_lens = mask[:, P:].sum(-1).tolist()
    costs = compute_group_costs(groups, p_lens, r_lens, float(meta.get("quadratic_weight", 0.5)))
    identity = torch.arange(B)
    if B % n_ranks:
        return batch, identity
    rank_of = np.empty(len(groups), dtype=np.int32)
    c = np.ascontiguousarray(np.asarray(costs, dtype=np.float64))
    s = np.ascontiguousarray(np.asarray([len(g) for g in groups], dtype=np.int32))
    rc = _lib.rt_lib().apb_rt_balance_groups(c.ctypes.data_as(ctypes.POINTER(ctypes.c_double)),
                                             s.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), len(groups), n_ranks, 1,
                                             rank_of.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)))
    if rc != 0:
        return batch, identity
    order: List[int] = []
    for r in range(n_ranks):
        for g, mem in enumerate(groups):
            if rank_of[g] == r:
                order.extend(mem)
    order_t = torch.tensor(order, dtype=torch.long)
    out = {k: (v[order_t] if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == B else v) for k, v in batch.items()}
    return out, order_t


def rearrange_micro_batches_with_dedup(batch: Dict[str, torch.Tensor], response_length: int, max_token_len: int,
                                       max_rollouts: Optional[int] = None, dp_group=None
                                       ) -> Tuple[List[Dict[str, torch.Tensor]], List[List[int]]]:
    """Micro-batches of whole prompt groups under a budget of DEDUPLICATED tokens (prompt counted once per
    group).  The micro-batch count is raised to the maximum over data-parallel ranks."""
    from ..processors.microbatch import ffd_allocate
    ids, mask = batch["input_ids"], batch["attention_mask"]
    P = ids.shape[1] - response_length
    groups = create_prompt_groups(ids, mask, response_length, max_rollouts, max_token_len)
    sizes = [int(mask[g[0], :P].sum()) + int(mask[g, P:].sum()) for g in groups]
    bins = ffd_allocate(sizes, max_token_len)
    if dist.is_initialized() and dist.get_world_size(dp_group) > 1:
        t = torch.tensor([len(bins)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=dp_group)
        if int(t) > len(bins):
            bins = ffd_allocate(sizes, max_token_len, min_groups=int(t))
    bins = [b for b in bins if b]
    mbs, idx_lists = [], []
    for b in bins:
        rows = [i for g in b for i in groups[g]]
        idx = torch.tensor(rows, dtype=torch.long)
        mbs.append({k: (v[idx] if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == ids.shape[0] else v)
                    for k, v in batch.items()})
        idx_lists.append(rows)
    return mbs, idx_lists


def reorg_global_batch_verl(super_batch, response_length: int, world_size: int, max_token_len: Optional[int] = None,
                            max_group_length_threshold: Optional[int] = None):
    """The balancer for a verl-style super-batch object (``.batch``: tensors keyed by name, ``.non_tensor_batch``:
    numpy arrays with the same leading dimension): rows are permuted so that contiguous ``B / world_size`` blocks
    hold whole prompt groups of balanced cost.  The object is reordered in place when it offers ``reorder(indices)``,
    else its two dicts are re-indexed; it is returned either way, untouched when there is nothing to balance
    (arctic_platform/rl/zorro_train/seqlen_balancing.py:489-600)."""
    batch = super_batch.batch
    ids = batch["input_ids"]
    B = ids.shape[0]
    if B <= world_size:
        return super_batch
    view = {k: batch[k] for k in ("input_ids", "attention_mask", "response_mask", "responses") if k in batch.keys()}
    meta = {"response_length": response_length, "max_rollouts": max_group_length_threshold}
    _, order = reorg_global_batch(view, meta, world_size)
    if torch.equal(order, torch.arange(B)):
        return super_batch
    if hasattr(super_batch, "reorder"):
        super_batch.reorder(order)
        return super_batch
    for k in list(batch.keys()):
        v = batch[k]
        if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == B:
            batch[k] = v[order]
    non_tensor = getattr(super_batch, "non_tensor_batch", None) or {}
    idx = order.numpy()
    for k in list(non_tensor.keys()):
        v = non_tensor[k]
        if hasattr(v, "__len__") and len(v) == B:
            non_tensor[k] = v[idx] if isinstance(v, np.ndarray) else [v[i] for i in idx]
    return super_batch
