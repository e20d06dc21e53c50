"""Forest-cascade decode attention: one query token per sequence over a tree of shared KV prefixes.

Sequences that decode together often share long prefixes -- the rollouts of one prompt share the prompt, and prompts
of one task share a system / few-shot header -- so their KV pages form a forest: header -> prompt -> rollout.  Reading
every sequence's full context per step re-reads the shared pages once per sequence.  Here every NODE of the forest is
attended once per step by all sequences below it (``decode_prefix.cu``: their query rows form one 128-row tensor-core
tile, the node's pages are streamed once), every sequence attends to its private pages by itself
(``paged_decode_mma_kernel``), and a log-sum-exp merge joins a sequence's levels.  KV traffic per step drops from
``sum over sequences of context length`` to ``sum over nodes of node length + private tokens``.

The reference switches the same idea on in its sampler with ``use_fca`` ("forest cascade attention",
arctic_platform/common/utils/server_models.py:123-132, README.md:87-97); the kernels live in ArcticInference.

``ForestTables`` is the device-side description (built on the host from node lists), ``forest_decode_attention``
runs the passes.  ``forest_decode_reference`` is the dense fp32 oracle used by the tests.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib

PAGE = 16
MAX_SHARED_LEVELS = 3

_FN = {}


def _fn(name: str):
    if not _FN:
        c = ctypes
        vp, i, ll, f = c.c_void_p, c.c_int, c.c_longlong, c.c_float
        _FN["dec"] = _lib.declare("apb_paged_decode_partial", [vp, vp, vp, vp, i, vp, vp, vp, vp, vp, i, i, i, i, i, f, vp])
        _FN["merge"] = _lib.declare("apb_decode_merge", [vp, vp, vp, i, vp, vp, vp, i, i, i, vp])
        _FN["prefix_tc"] = _lib.declare("apb_decode_prefix_tc",
                                        [vp, i, vp, vp, vp, i, vp, vp, vp, vp, ll, vp, vp, i, i, i, i, i, i, f, vp])
    return _FN[name]


@dataclass
class ForestNode:
    """One shared node: the sequences (slots) below it, its KV pages in order and how many tokens they hold."""
    level: int
    slots: Sequence[int]
    pages: np.ndarray
    kv_len: int


@dataclass
class ForestTables:
    q_start: torch.Tensor      # [G] int32: first slot of the node's run of consecutive slots
    q_count: torch.Tensor      # [G] int32: slots in the run (0 = unused table row)
    pages: torch.Tensor        # [G, max_pages] int32
    kv_len: torch.Tensor       # [G] int32
    level: torch.Tensor        # [G] int32
    row_mask: torch.Tensor     # [B] int32: bit l = the slot has a node at shared level l, bit n_levels = private pass
    n_nodes: int
    n_levels: int
    shared_tokens: int         # tokens stored in shared nodes (each counted once)
    covered_tokens: int        # tokens the sequences see through shared nodes (what a per-sequence pass would read)


def plan_forest(nodes: Sequence[ForestNode], num_slots: int, max_pages: int, max_rows: int,
                n_levels: Optional[int] = None):
    """Host tables for a set of nodes.  A node's slots are cut into runs of consecutive slots of at most ``max_rows``
    (one tensor-core tile each; a node whose slots are scattered or too many is simply attended by several runs).
    Returns numpy arrays ``(q_start, q_count, pages, kv_len, level, row_mask, n_nodes, n_levels, shared, covered)``."""
    runs: List[Tuple[int, int, int, np.ndarray, int]] = []
    levels_seen = 0
    shared = covered = 0
    for nd in nodes:
        if nd.kv_len <= 0 or len(nd.slots) == 0:
            continue
        if not 0 <= nd.level < MAX_SHARED_LEVELS:
            raise ValueError(f"forest level {nd.level} outside 0..{MAX_SHARED_LEVELS - 1}")
        if len(nd.pages) * PAGE < nd.kv_len or len(nd.pages) > max_pages:
            raise ValueError("a forest node's page list does not match its length")
        levels_seen = max(levels_seen, nd.level + 1)
        shared += nd.kv_len
        covered += nd.kv_len * len(nd.slots)
        mem = sorted(int(s) for s in nd.slots)
        i = 0
        while i < len(mem):
            j = i
            while j + 1 < len(mem) and mem[j + 1] == mem[j] + 1 and j + 1 - i < max_rows:
                j += 1
            runs.append((nd.level, mem[i], j - i + 1, nd.pages, nd.kv_len))
            i = j + 1
    n_levels = max(1, levels_seen) if n_levels is None else int(n_levels)
    G = len(runs)
    q_start = np.zeros(max(G, 1), dtype=np.int32)
    q_count = np.zeros(max(G, 1), dtype=np.int32)
    kv_len = np.zeros(max(G, 1), dtype=np.int32)
    level = np.zeros(max(G, 1), dtype=np.int32)
    pages = np.zeros((max(G, 1), max_pages), dtype=np.int32)
    row_mask = np.full(num_slots, 1 << n_levels, dtype=np.int32)
    for k, (lv, s0, cnt, pg, ln) in enumerate(runs):
        q_start[k], q_count[k], kv_len[k], level[k] = s0, cnt, ln, lv
        pages[k, :len(pg)] = pg
        row_mask[s0:s0 + cnt] |= 1 << lv
    return q_start, q_count, pages, kv_len, level, row_mask, G, n_levels, shared, covered


def build_forest_tables(nodes: Sequence[ForestNode], num_slots: int, max_pages: int, max_rows: int, device,
                        n_levels: Optional[int] = None) -> ForestTables:
    from ..utils.transfer_stats import to_device
    qs, qc, pg, ln, lv, mask, G, nl, shared, covered = plan_forest(nodes, num_slots, max_pages, max_rows, n_levels)
    from ..utils import checked
    if checked.enabled():                           # host arrays: no synchronisation involved
        checked.check_forest(qs, qc, pg, ln, lv, num_slots, np.iinfo(np.int32).max, nl, max_rows, PAGE)
    t = lambda a: to_device(torch.from_numpy(a), device)
    return ForestTables(t(qs), t(qc), t(pg), t(ln), t(lv), t(mask), G, nl, shared, covered)


def forest_decode_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, forest: ForestTables,
                            priv_start: torch.Tensor, priv_active: torch.Tensor, priv_table: torch.Tensor,
                            priv_len: torch.Tensor, part_o: Sequence[torch.Tensor], part_ml: Sequence[torch.Tensor],
                            splits: int, seq_splits: int, scale: Optional[float] = None,
                            out: Optional[torch.Tensor] = None, n_nodes: Optional[int] = None) -> torch.Tensor:
    """``q [B, Hq, D]`` bf16 (one token per slot) -> ``[B, Hq, D]`` bf16.

    ``kcache / vcache [num_pages, Hkv, 16, D]`` (one layer).  ``forest``: shared nodes.  ``priv_*``: the per-sequence
    pass (``priv_start [B]`` = slot ids, ``priv_active [B]`` = 1 for live slots, ``priv_table [B, max_pages]``,
    ``priv_len [B]``).  ``part_o[i] [B, Hq, splits, D]`` / ``part_ml[i] [B, Hq, splits, 2]`` fp32 scratch for source
    ``i`` (shared levels first, the private pass last).  ``n_nodes`` bounds the launch grid (rows of the node tables
    beyond the live nodes have ``q_count == 0`` and cost an empty CTA)."""
    B, Hq, D = q.shape
    Hkv = kcache.shape[1]
    num_pages = kcache.shape[0]
    max_pages = priv_table.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    s = _lib.stream_ptr()
    nl = forest.n_levels
    G = forest.n_nodes if n_nodes is None else int(n_nodes)
    if out is None:
        out = torch.empty((B, Hq, D), device=q.device, dtype=torch.bfloat16)
    from ..utils import checked
    if checked.active_for(q):
        if G > 0:
            checked.check_forest(forest.q_start[:G], forest.q_count[:G], forest.pages[:G], forest.kv_len[:G],
                                 forest.level[:G], B, num_pages, nl, 128, PAGE)
        checked.check_range("priv_start", priv_start, 0, max(1, B), priv_active)
        checked.check_page_table("priv_table", priv_table, priv_len, num_pages, PAGE, priv_active)
    if G > 0:
        o_lv = (ctypes.c_void_p * 3)(*[part_o[min(i, nl - 1)].data_ptr() for i in range(3)])
        ml_lv = (ctypes.c_void_p * 3)(*[part_ml[min(i, nl - 1)].data_ptr() for i in range(3)])
        _lib.check(_fn("prefix_tc")(_lib.ptr(q), B, _lib.ptr(forest.q_start), _lib.ptr(forest.q_count),
                                    _lib.ptr(forest.pages), forest.pages.shape[1], _lib.ptr(forest.kv_len),
                                    _lib.ptr(forest.level), _lib.ptr(kcache), _lib.ptr(vcache), num_pages, o_lv, ml_lv,
                                    nl, G, Hq, Hkv, D, splits, scale, s), "decode_prefix_tc")
    _lib.check(_fn("dec")(_lib.ptr(q), _lib.ptr(priv_start), _lib.ptr(priv_active), _lib.ptr(priv_table), max_pages,
                          _lib.ptr(priv_len), _lib.ptr(kcache), _lib.ptr(vcache), _lib.ptr(part_o[nl]),
                          _lib.ptr(part_ml[nl]), B, Hq, Hkv, D, seq_splits, scale, s), "paged_decode(private)")
    n_src = nl + 1
    o_ptrs = (ctypes.c_void_p * 4)(*[part_o[i].data_ptr() if i < n_src else 0 for i in range(4)])
    ml_ptrs = (ctypes.c_void_p * 4)(*[part_ml[i].data_ptr() if i < n_src else 0 for i in range(4)])
    sp = (ctypes.c_int * 4)(*[(splits if i < nl else seq_splits) if i < n_src else 0 for i in range(4)])
    _lib.check(_fn("merge")(o_ptrs, ml_ptrs, sp, n_src, _lib.ptr(forest.row_mask), _lib.ptr(out), None, B, Hq, D, s),
               "decode_merge")
    return out


def forest_decode_reference(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                            contexts: Sequence[Sequence[Tuple[np.ndarray, int]]], scale: Optional[float] = None):
    """Dense fp32 oracle: ``contexts[b]`` lists ``(pages, tokens)`` pieces of slot ``b``'s context in order (shared
    nodes first, then its private pages); attention of ``q[b]`` over the concatenation."""
    B, Hq, D = q.shape
    Hkv = kcache.shape[1]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros((B, Hq, D), dtype=torch.float32, device=q.device)
    for b, pieces in enumerate(contexts):
        ks, vs = [], []
        for pages, n in pieces:
            if n <= 0:
                continue
            idx = torch.as_tensor(np.asarray(pages, dtype=np.int64), device=q.device)
            k = kcache[idx].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n]       # [Hkv, tokens, D]
            v = vcache[idx].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n]
            ks.append(k.float())
            vs.append(v.float())
        if not ks:
            continue
        k = torch.cat(ks, 1).repeat_interleave(rep, 0)
        v = torch.cat(vs, 1).repeat_interleave(rep, 0)
        s = torch.einsum("hd,hkd->hk", q[b].float(), k) * scale
        p = torch.softmax(s, -1)
        out[b] = torch.einsum("hk,hkd->hd", p, v)
    return out
