"""Checked mode: every table that drives a kernel's addresses is validated before the launch.

The kernels of this package index memory through tables that other code built -- page tables of the KV cache, node
tables of the prefix forest, ``cu_seqlens`` of a packed batch, routing entries of expert parallelism, tile maps of the
grouped GEMMs.  A wrong entry there is an out-of-bounds access on the device: at best a fault that takes the context
down, at worst a silent write into somebody else's tensor.  With ``APB_DEBUG_CHECKS=1`` the wrappers that launch such
kernels call the validators below first.  A validator names the table, the first offending position and value and
raises ``TableError`` on the host -- nothing is launched with a bad table, so a bug surfaces as a Python exception
with the GPU context intact.  Tables that live on the device are reduced there (min / max / comparisons) and only the
verdict crosses to the host, which is one synchronisation per checked launch: the mode is for debugging and for the
test suite, not for production steps, and it is skipped while a CUDA graph is being captured (a capture cannot
synchronise; the eager warm-up step before every capture is checked).

The complementary device-side protection is always on: bounded waits with a status record, and routing entries that
are range-checked in the kernel before a peer store (``kBadRouting``).
"""
from __future__ import annotations

import os
from typing import Any, Optional, Sequence

import numpy as np
import torch


class TableError(ValueError):
    """A table that would make a kernel read or write out of bounds."""


_forced: Optional[bool] = None


def enabled() -> bool:
    if _forced is not None:
        return _forced
    return os.environ.get("APB_DEBUG_CHECKS", "0") not in ("0", "", "false", "False")


def force(on: Optional[bool]) -> None:
    """Overrides the environment for this process (None = follow ``APB_DEBUG_CHECKS`` again)."""
    global _forced
    _forced = on


def active_for(*tensors: Any) -> bool:
    """Checked mode is on and a check may synchronise (no CUDA graph capture in progress on a tensor's device)."""
    if not enabled():
        return False
    for t in tensors:
        if torch.is_tensor(t) and t.is_cuda:
            return not torch.cuda.is_current_stream_capturing()
    return True


def _as_tensor(x: Any) -> torch.Tensor:
    return x if torch.is_tensor(x) else torch.as_tensor(np.asarray(x))


def _first_bad(bad: torch.Tensor):
    idx = torch.nonzero(bad.reshape(-1), as_tuple=False)[0, 0]
    return int(idx)


def check_range(name: str, table: Any, low: int, high: int, where: Optional[Any] = None) -> None:
    """Every entry (of the rows / elements selected by the boolean ``where``) lies in ``[low, high)``."""
    t = _as_tensor(table)
    if t.numel() == 0:
        return
    bad = (t < low) | (t >= high)
    if where is not None:
        w = _as_tensor(where).bool()
        while w.dim() < bad.dim():
            w = w.unsqueeze(-1)
        bad = bad & w
    if bool(bad.any()):
        i = _first_bad(bad)
        pos = np.unravel_index(i, tuple(t.shape))
        raise TableError(f"{name}{list(int(p) for p in pos)} = {int(t.reshape(-1)[i])} outside [{low}, {high})")


def check_cu_seqlens(cu: Any, total_tokens: Optional[int] = None, name: str = "cu_seqlens") -> None:
    """Starts at 0, never decreases, ends at the number of packed tokens."""
    t = _as_tensor(cu).reshape(-1).long()
    if t.numel() < 1 or int(t[0]) != 0:
        raise TableError(f"{name} must start at 0")
    d = t[1:] - t[:-1]
    if bool((d < 0).any()):
        i = _first_bad(d < 0)
        raise TableError(f"{name}[{i + 1}] = {int(t[i + 1])} is smaller than {name}[{i}] = {int(t[i])}")
    if total_tokens is not None and int(t[-1]) != int(total_tokens):
        raise TableError(f"{name} ends at {int(t[-1])}, the batch holds {int(total_tokens)} tokens")


def check_page_table(name: str, table: Any, lengths: Any, num_pages: int, page: int = 16, active: Optional[Any] = None) -> None:
    """Rows of page ids: a row of ``lengths[i]`` tokens uses its first ``ceil(len / page)`` entries, which must be
    valid page ids and fit the row."""
    tab, ln = _as_tensor(table), _as_tensor(lengths).reshape(-1).long()
    if tab.dim() != 2 or tab.shape[0] < ln.numel():
        raise TableError(f"{name}: expected [rows >= {ln.numel()}, max_pages], got {tuple(tab.shape)}")
    tab = tab[:ln.numel()]
    act = _as_tensor(active).reshape(-1).bool()[:ln.numel()] if active is not None else torch.ones_like(ln, dtype=torch.bool)
    if bool(((ln < 0) & act).any()):
        i = _first_bad((ln < 0) & act)
        raise TableError(f"{name}: row {i} has negative length {int(ln[i])}")
    need = (ln + page - 1) // page
    if bool(((need > tab.shape[1]) & act).any()):
        i = _first_bad((need > tab.shape[1]) & act)
        raise TableError(f"{name}: row {i} holds {int(ln[i])} tokens = {int(need[i])} pages, the table has {tab.shape[1]} columns")
    used = (torch.arange(tab.shape[1], device=tab.device).unsqueeze(0) < need.to(tab.device).unsqueeze(1)) & act.to(tab.device).unsqueeze(1)
    check_range(name, tab, 0, int(num_pages), used)


def check_forest(q_start: Any, q_count: Any, pages: Any, kv_len: Any, level: Any, num_slots: int, num_pages: int,
                 n_levels: int, max_rows: int = 128, page: int = 16) -> None:
    """Node tables of the forest pass: slot runs inside the batch and at most one tile high, levels in range, page
    lists long enough for the node's tokens and made of valid pages."""
    qs, qc = _as_tensor(q_start).long(), _as_tensor(q_count).long()
    live = qc > 0
    check_range("forest.q_count", qc, 0, max_rows + 1)
    check_range("forest.q_start", qs, 0, max(1, num_slots), live)
    over = (qs + qc > num_slots) & live
    if bool(over.any()):
        i = _first_bad(over)
        raise TableError(f"forest node {i}: slots {int(qs[i])}..{int(qs[i] + qc[i]) - 1} exceed the batch of {num_slots}")
    check_range("forest.level", level, 0, max(1, n_levels), live)
    check_page_table("forest.pages", pages, kv_len, num_pages, page, live)


def check_routing(dst_rank: Any, dst_row: Any, world: int, rows_cap: int, name: str = "routing") -> None:
    """Dispatch entries: rank -1 = dropped; every other entry names a rank of the group and a row of its buffer."""
    r, row = _as_tensor(dst_rank).long(), _as_tensor(dst_row).long()
    live = r >= 0
    check_range(f"{name}.dst_rank", r, -1, world)
    check_range(f"{name}.dst_row", row, 0, max(1, rows_cap), live)


def check_tile_map(tile_map: Any, num_tiles: int, groups: int, m_tiles_cap: int, name: str = "tile_map") -> None:
    """Grouped-GEMM tile records ``(group, m_tile, ...)``: the first ``num_tiles`` rows name a valid group and an
    M tile inside the padded rows."""
    t = _as_tensor(tile_map)
    if t.dim() != 2 or t.shape[0] < num_tiles:
        raise TableError(f"{name}: {num_tiles} tiles announced, the table holds {tuple(t.shape)}")
    if num_tiles <= 0:
        return
    check_range(f"{name}.group", t[:num_tiles, 0], 0, groups)
    check_range(f"{name}.m_tile", t[:num_tiles, 1], 0, max(1, m_tiles_cap))


def check_gather_index(name: str, index: Any, source_rows: int) -> None:
    check_range(name, index, 0, max(1, source_rows))


def check_copy_table(name: str, src_off: Sequence[int], dst_off: Sequence[int], sizes: Sequence[int], src_size: int,
                     dst_size: int) -> None:
    """Segment copies ``dst[dst_off : dst_off + n] = src[src_off : src_off + n]`` stay inside both buffers and no two
    destinations overlap."""
    so, do, n = (np.asarray(x, dtype=np.int64) for x in (src_off, dst_off, sizes))
    if not (len(so) == len(do) == len(n)):
        raise TableError(f"{name}: offset and size lists differ in length")
    if len(n) == 0:
        return
    for label, off, lim in (("source", so, src_size), ("destination", do, dst_size)):
        bad = (off < 0) | (n < 0) | (off + n > lim)
        if bad.any():
            i = int(np.argmax(bad))
            raise TableError(f"{name}: segment {i} covers {label} [{int(off[i])}, {int(off[i] + n[i])}) of a buffer of {lim}")
    order = np.argsort(do, kind="stable")
    ends = (do + n)[order]
    clash = ends[:-1] > do[order][1:]
    if clash.any():
        i = int(np.argmax(clash))
        raise TableError(f"{name}: destinations of segments {int(order[i])} and {int(order[i + 1])} overlap")
