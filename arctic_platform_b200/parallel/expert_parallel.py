"""Expert parallelism for the MoE layers: dispatch and combine as in-kernel NVLink stores.

Experts are sharded over the ranks of a group (rank ``d`` owns experts ``[d*El, (d+1)*El)``).  One MoE layer is

1. routing (fp32 softmax + top-k) and an all-gather of the per-expert pair counts (``[W, E]`` int64 -- the only
   library collective, 8 * E bytes; the reference all-reduces a chunk count there,
   arctic_platform/model/implementations/qwen35/models/layers/moe.py:451-454).  The count matrix STAYS ON THE
   GPU: every offset, the owner's padded expert-major row layout and the tile tables of the grouped GEMMs are
   derived from it by device code (``plan_routing_device``, ``models.moe.MoEPlan``), and the receive buffers are
   sized for a fixed capacity (``max_recv_rows``), so a layer call never synchronises with the host;
2. **dispatch**: every routed (token, expert) pair is written by ``ep_scatter_rows_kernel`` straight into the
   owner rank's receive buffer at its final, expert-sorted row (offsets are computed identically on every
   rank from the count matrix, so no second exchange is needed), together with a ``(source rank, pair)`` tag;
3. the owner runs the grouped tcgen05 GEMMs over its rows (``models/moe.py``: forward, data gradients and weight
   gradients from device tables);
4. **combine**: in inference the second expert GEMM stores each output row directly into the source rank's
   combine buffer from its epilogue (``apb_gemm_scatter`` -- compute and all-to-all in one kernel); in training
   the rows go back through the same scatter kernel so that every stage has an exact transpose for autograd;
5. the source sums its ``k`` returned rows with the routing weights.

Epoch flags in symmetric memory order the stages (bounded waits).  ``impl="collective"`` performs the same
exchange with ``torch.distributed.all_to_all_single`` -- the NCCL baseline and the CPU/gloo path.  The
reference uses DeepEP buffers for this (``.../qwen35/distributed/deepep.py:29-347``).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from .symm import EpochFlags, SymmetricBuffer

_FN: Dict[str, object] = {}


def _fns():
    if not _FN:
        c = ctypes
        vp, i, ll = c.c_void_p, c.c_int, c.c_longlong
        _FN["scatter"] = _lib.declare("apb_ep_scatter_rows", [vp, ll, vp, vp, vp, vp, vp, ll, vp, i, i, i, i, vp])
        _FN["gscatter"] = _lib.declare("apb_gemm_scatter_dev",
                                       [vp, vp, vp, i, vp, i, i, i, ll, ll, ll, vp, i, vp, ll, vp])
        _FN["wait"] = _lib.declare("apb_epoch_wait", [vp, i, i, i, vp])
    return _FN


@dataclass
class Routing:
    """Everything both directions of the exchange need, computed once per layer call."""
    order: torch.Tensor        # [P] pair indices sorted by expert
    src_tok: torch.Tensor      # [P] token of each sorted pair (int32)
    dst_rank: torch.Tensor     # [P] owner rank of each sorted pair (int32)
    dst_row: torch.Tensor      # [P] row in the owner's receive buffer (int32)
    recv_counts: torch.Tensor  # [El] rows per local expert on THIS rank (int64, CPU)
    recv_rows: int
    send_splits: list          # rows this rank sends to each rank
    recv_splits: list          # rows this rank receives from each rank
    num_pairs: int


def plan_routing(idx: torch.Tensor, num_experts: int, world: int, rank: int, group=None) -> Routing:
    """Sorts the routed pairs by expert and derives every destination row from the all-gathered counts."""
    P = idx.numel()
    k = idx.shape[1]
    El = num_experts // world
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    if world > 1:
        allc = torch.empty((world, num_experts), dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(allc.view(-1), counts.contiguous(), group=group)
    else:
        allc = counts[None]
    tot = allc.sum(0)                                              # pairs per expert over all ranks
    blk = tot.view(world, El)
    base = (blk.cumsum(1) - blk).reshape(-1)                       # start of each expert inside its owner's buffer
    before_me = allc[:rank].sum(0) if rank > 0 else torch.zeros_like(tot)
    start = base + before_me                                       # where MY pairs of each expert begin
    sorted_e = flat[order]
    first = counts.cumsum(0) - counts                              # first sorted position of each expert
    pos = torch.arange(P, device=idx.device) - first[sorted_e]
    dst_row = (start[sorted_e] + pos).to(torch.int32)
    dst_rank = torch.div(sorted_e, El, rounding_mode="floor").to(torch.int32)
    # ONE device->host copy per layer call: the count matrix; every host-side number derives from it
    allc_h = allc.cpu()
    mine_h = allc_h[:, rank * El:(rank + 1) * El]
    recv_counts = mine_h.sum(0)
    send = allc_h[rank].view(world, El).sum(1).tolist()
    recv = mine_h.sum(1).tolist()
    routing = Routing(order, torch.div(order, k, rounding_mode="floor").to(torch.int32), dst_rank, dst_row,
                      recv_counts, int(recv_counts.sum()), send, recv, P)
    routing._allc = allc
    from ..utils.debug import maybe_record_recv_tokens
    maybe_record_recv_tokens(routing.recv_rows)
    return routing


@dataclass
class DeviceRouting:
    """The fused path's plan: nothing here was computed on the host except ``num_pairs`` and the capacity."""
    order: torch.Tensor        # [P] pair indices sorted by expert
    src_tok: torch.Tensor      # [P] token of each sorted pair (int32)
    dst_rank: torch.Tensor     # [P] owner rank of each sorted pair (int32; -1 = dropped: capacity exceeded)
    dst_row: torch.Tensor      # [P] padded row in the owner's receive buffer (int32)
    recv_counts: torch.Tensor  # [El] rows per local expert on THIS rank (int32, GPU)
    valid: torch.Tensor        # [cap] bool: the receive-buffer row holds a routed pair (not padding)
    plan: object               # models.moe.MoEPlan of this rank's experts
    recv_rows: int             # = capacity (host)
    num_pairs: int
    # training pass: received rows are copied out of the symmetric buffer with the padding rows zeroed (they are
    # saved for backward and read by the weight-gradient GEMMs); inference reads the buffer in place.  Decided by
    # the layer, not from the autograd mode inside the exchange (a Function's forward always runs without it).
    materialize: bool = True


def plan_routing_device(idx: torch.Tensor, num_experts: int, world: int, rank: int, group, cap: int, hidden: int,
                        expert_width: int, overflow: torch.Tensor) -> DeviceRouting:
    """Like :func:`plan_routing`, for the padded layout of :class:`models.moe.MoEPlan` (every expert's rows on its
    owner start at a multiple of 64) and without a device->host copy.  ``overflow`` (int32 [1], GPU) is raised when
    a rank would receive more rows than ``cap``; such pairs are dropped instead of written out of bounds."""
    from ..models.moe import MoEPlan, _expert_histogram
    P = idx.numel()
    k = idx.shape[1]
    El = num_experts // world
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = _expert_histogram(flat, num_experts)
    allc = torch.empty((world, num_experts), dtype=counts.dtype, device=counts.device)
    dist.all_gather_into_tensor(allc.view(-1), counts.contiguous(), group=group)
    tot = allc.sum(0)                                              # pairs per expert over all ranks
    padded = (tot + 63) // 64 * 64
    blk = padded.view(world, El)
    base = (blk.cumsum(1) - blk).reshape(-1)                       # padded start of each expert on its owner
    before_me = allc[:rank].sum(0) if rank > 0 else torch.zeros_like(tot)
    start = base + before_me
    sorted_e = flat[order]
    first = counts.cumsum(0) - counts
    dst_row = start[sorted_e] + (torch.arange(P, device=idx.device) - first[sorted_e])
    used = blk.sum(1)                                              # padded rows in use on every rank
    overflow |= (used.max() > cap).to(overflow.dtype)
    dst_rank = torch.div(sorted_e, El, rounding_mode="floor")
    dst_rank = torch.where(dst_row < cap, dst_rank, torch.full_like(dst_rank, -1)).to(torch.int32)
    mine = tot[rank * El:(rank + 1) * El].to(torch.int32)
    plan = MoEPlan(mine, 0, hidden, expert_width, rows_cap=cap)
    rows = torch.arange(cap, device=idx.device)
    seg = plan.seg_start.to(torch.int64)
    e_of = torch.searchsorted(seg[1:].contiguous(), rows, right=True).clamp_(max=El - 1)
    valid = (rows - seg[e_of]) < mine.to(torch.int64)[e_of]
    valid &= rows < seg[El]
    return DeviceRouting(order, torch.div(order, k, rounding_mode="floor").to(torch.int32), dst_rank,
                         dst_row.to(torch.int32), mine, valid, plan, cap, P)


class ExpertParallel:
    def __init__(self, hidden: int, num_experts: int, group=None, device="cuda", max_recv_rows: int = 1 << 16,
                 max_pairs: int = 1 << 16, impl: str = "fused"):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.hidden = hidden
        self.num_experts = num_experts
        self.device = torch.device(device)
        self.impl = impl if (self.device.type == "cuda" and self.world > 1) else "collective"
        if self.impl == "fused":
            self.flags = EpochFlags(device, group)
            self.recv = SymmetricBuffer(max_recv_rows * hidden, torch.bfloat16, device, group)
            self.meta = SymmetricBuffer(max_recv_rows * 2, torch.int32, device, group)
            self.comb = SymmetricBuffer(max_pairs * hidden, torch.bfloat16, device, group)
            self.overflow = torch.zeros(1, dtype=torch.int32, device=device)
        self.max_recv_rows, self.max_pairs = max_recv_rows // 128 * 128, max_pairs

    def raise_if_overflowed(self) -> None:
        """One host read: did any layer call since the last check receive more rows than the buffers hold?  (The
        pairs beyond the capacity were dropped, not written.)  The training engine asks once per optimizer step."""
        if self.impl == "fused" and int(self.overflow.item()) != 0:
            self.overflow.zero_()
            raise ValueError(f"expert-parallel receive capacity ({self.max_recv_rows} rows) exceeded; "
                             "raise max_recv_rows")

    # ------------------------------------------------------------------ exchange primitives
    def _barrier(self) -> None:
        _lib.check(_fns()["wait"](self.flags.ptr_table(), self.rank, self.world, self.flags.next(), _lib.stream_ptr()),
                   "apb_epoch_wait")

    def _to_owners(self, rows: torch.Tensor, src_row: torch.Tensor, r: Routing) -> torch.Tensor:
        """Rows (indexed by ``src_row``) -> owner ranks' receive buffers; returns this rank's received rows."""
        H = self.hidden
        if self.impl == "collective":
            send = rows.index_select(0, src_row.long())
            return _all_to_all_rows(send, r.send_splits, r.recv_splits, self.group, sort_recv=(self.world, r))
        if r.recv_rows > self.max_recv_rows or r.num_pairs > self.max_pairs:
            raise ValueError("expert-parallel scratch too small for this batch")
        tags = r.order.to(torch.int32)
        _lib.check(_fns()["scatter"](_lib.ptr(rows), rows.stride(0), _lib.ptr(src_row), _lib.ptr(r.dst_rank),
                                     _lib.ptr(r.dst_row), _lib.ptr(tags), self.recv.ptr_table(), H,
                                     self.meta.ptr_table(), self.rank, self.world, r.num_pairs, H, _lib.stream_ptr()),
                   "apb_ep_scatter_rows")
        self._barrier()
        got = self.recv.tensor[: r.recv_rows * H].view(r.recv_rows, H)
        if not getattr(r, "materialize", True):
            return got          # read in place: the layer's closing barrier comes before the next dispatch lands here
        # padding rows of the layout still hold rows of an earlier call: they must read as zeros (the weight-gradient
        # GEMMs walk whole 64-row blocks)
        return torch.where(r.valid[:, None], got, torch.zeros((), dtype=got.dtype, device=got.device))

    def _to_sources(self, rows: torch.Tensor, r: Routing) -> torch.Tensor:
        """This rank's processed rows -> the source ranks' combine buffers (pair order); returns ``[P, H]``."""
        H = self.hidden
        if self.impl == "collective":
            back = _all_to_all_rows(rows, r.recv_splits, r.send_splits, self.group, unsort_send=(self.world, r))
            out = torch.empty((r.num_pairs, H), device=rows.device, dtype=rows.dtype)
            out[r.order] = back
            return out
        meta = self.meta.tensor[: r.recv_rows * 2].view(r.recv_rows, 2)
        src_row = torch.arange(r.recv_rows, device=rows.device, dtype=torch.int32)
        # named tensors: a temporary handed to ptr() would be freed (and its block reused) before the launch
        to_rank = torch.where(r.valid, meta[:, 0], torch.full_like(meta[:, 0], -1))      # padding rows go nowhere
        to_row = meta[:, 1].contiguous()
        _lib.check(_fns()["scatter"](_lib.ptr(rows), rows.stride(0), _lib.ptr(src_row), _lib.ptr(to_rank),
                                     _lib.ptr(to_row), None, self.comb.ptr_table(), H, None, self.rank,
                                     self.world, r.recv_rows, H, _lib.stream_ptr()), "apb_ep_scatter_rows")
        self._barrier()
        return self.comb.tensor[: r.num_pairs * H].view(r.num_pairs, H).clone()

    # ------------------------------------------------------------------ layer
    def forward(self, moe, x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        from ..models.moe import grouped_ffn
        T, H = x.shape
        k = idx.shape[1]
        if self.impl == "fused":
            from ..models.moe import _GroupedFFNPaddedFn
            if idx.numel() > self.max_pairs:
                raise ValueError("expert-parallel scratch too small for this batch")
            r = plan_routing_device(idx, self.num_experts, self.world, self.rank, self.group, self.max_recv_rows, H,
                                    moe.wgu.shape[1] // 2, self.overflow)
            moe.last_tokens_per_expert = r.recv_counts
            r.materialize = torch.is_grad_enabled()
            from ..utils import checked
            if checked.active_for(x):
                checked.check_routing(r.dst_rank, r.dst_row, self.world, self.max_recv_rows, "expert_parallel")
                checked.check_range("expert_parallel.src_tok", r.src_tok, 0, max(1, T))
            x_recv = _DispatchFn.apply(x, self, r)
            if not torch.is_grad_enabled():
                y_pairs = self._ffn_with_fused_combine(moe, x_recv, r)
            else:
                y_recv = _GroupedFFNPaddedFn.apply(x_recv, moe.wgu, moe.wdown, r.plan)
                y_pairs = _CombineFn.apply(y_recv, self, r)
            return (y_pairs.view(T, k, H).float() * w[..., None]).sum(1).to(x.dtype)
        r = plan_routing(idx, self.num_experts, self.world, self.rank, self.group)
        moe.last_tokens_per_expert = r.recv_counts
        x_recv = _DispatchFn.apply(x, self, r)
        y_recv = grouped_ffn(x_recv, moe.wgu, moe.wdown, r.recv_counts)
        y_pairs = _CombineFn.apply(y_recv, self, r)
        return (y_pairs.view(T, k, H).float() * w[..., None]).sum(1).to(x.dtype)

    def _ffn_with_fused_combine(self, moe, x_recv: torch.Tensor, r: Routing) -> torch.Tensor:
        """Inference path: GEMM 1 with the SwiGLU epilogue, GEMM 2 whose epilogue stores every output row into
        the source rank's combine buffer (no separate combine kernel)."""
        from ..models.moe import _grouped_dev_fns
        from ..ops import gemm
        El, I2, H = moe.wgu.shape
        rows, plan = r.recv_rows, r.plan
        w1 = moe.wgu.view(El * I2, H)
        act = torch.empty((rows, I2 // 2), device=x_recv.device, dtype=x_recv.dtype)
        _lib.check(_grouped_dev_fns()["gemm"](_lib.ptr(x_recv), _lib.ptr(w1), None, rows, I2, H, x_recv.stride(0),
                                              w1.stride(0), 0, gemm.EPI_SWIGLU, 1.0, _lib.ptr(act), act.stride(0),
                                              _lib.ptr(plan.maps[0]), plan.max_tiles[0], _lib.ptr(plan.n_tiles),
                                              El * I2, _lib.stream_ptr()), "grouped gate/up")
        # (rank, row) of every receive-buffer row; padding rows are dropped by the epilogue (rank -1)
        meta = self.meta.tensor[: rows * 2].view(rows, 2)
        row_map = torch.where(r.valid[:, None], meta, torch.tensor([-1, 0], dtype=meta.dtype, device=meta.device))
        row_map = row_map.contiguous()
        _lib.check(_fns()["gscatter"](_lib.ptr(act), _lib.ptr(moe.wdown.view(El * H, I2 // 2)), self.comb.ptr_table(),
                                      self.world, _lib.ptr(row_map), rows, H, I2 // 2, act.stride(0), I2 // 2, H,
                                      _lib.ptr(plan.maps[1]), plan.max_tiles[1], _lib.ptr(plan.n_tiles[1:]), El * H,
                                      _lib.stream_ptr()), "apb_gemm_scatter_dev")
        self._barrier()
        return self.comb.tensor[: r.num_pairs * H].view(r.num_pairs, H).clone()


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ep: ExpertParallel, r: Routing):
        ctx.ep, ctx.r, ctx.shape = ep, r, x.shape
        return ep._to_owners(x.contiguous(), r.src_tok, r)

    @staticmethod
    def backward(ctx, d_recv):
        ep, r = ctx.ep, ctx.r
        T, H = ctx.shape
        d_pairs = ep._to_sources(d_recv.contiguous(), r)             # [P, H] in pair order
        return d_pairs.view(T, -1, H).float().sum(1).to(d_recv.dtype), None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_recv, ep: ExpertParallel, r: Routing):
        ctx.ep, ctx.r = ep, r
        return ep._to_sources(y_recv.contiguous(), r)

    @staticmethod
    def backward(ctx, d_pairs):
        ep, r = ctx.ep, ctx.r
        return ep._to_owners(d_pairs.contiguous(), r.order.to(torch.int32), r), None, None


def _all_to_all_rows(send: torch.Tensor, send_splits, recv_splits, group, sort_recv=None, unsort_send=None):
    """Collective baseline.  Rows are sent grouped by destination rank in expert-sorted order; the receiver
    re-sorts them by (expert, source) to match the fused layout (``sort_recv``), and undoes that before
    sending results back (``unsort_send``)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if unsort_send is not None:
        _, r = unsort_send
        send = send.index_select(0, r._recv_perm)
    if world == 1:
        recv = send
    else:
        recv = send.new_empty((sum(recv_splits), send.shape[1]))
        dist.all_to_all_single(recv, send.contiguous(), list(recv_splits), list(send_splits), group=group)
    if sort_recv is not None:
        _, r = sort_recv
        perm = _recv_permutation(r, world, group, recv.device)
        r._recv_perm = perm
        # rows arrive source-major; the fused layout is expert-major with sources inside an expert
        out = torch.empty_like(recv)
        out[perm] = recv
        return out
    return recv


def _recv_permutation(r: Routing, world: int, group, device) -> torch.Tensor:
    """Destination row (expert-major) of every row received in source-major order."""
    El = r.recv_counts.numel()
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    # per-source, per-local-expert counts on this rank
    mine = r._allc[:, rank * El:(rank + 1) * El] if hasattr(r, "_allc") else None
    if mine is None:
        raise RuntimeError("collective expert-parallel path needs the count matrix (plan_routing_collective)")
    mine = mine.to(device)
    tot = mine.sum(0)
    base = tot.cumsum(0) - tot
    within = mine.cumsum(0) - mine                      # rows of earlier sources inside each expert
    perm = []
    for s in range(world):
        for e in range(El):
            n = int(mine[s, e])
            if n:
                perm.append(torch.arange(n, device=device) + base[e] + within[s, e])
    return torch.cat(perm) if perm else torch.zeros(0, dtype=torch.long, device=device)


def attach_expert_parallel(model, ep_size: int, group=None, impl: str = "fused", **kw) -> None:
    """Shards every MoE layer's expert weights over ``ep_size`` ranks (this rank keeps its slice) and installs
    the dispatch/combine engine on the layer."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if ep_size != world:
        raise ValueError(f"expert_parallel={ep_size} must equal the size of the expert-parallel group ({world})")
    for blk in model.blocks:
        moe = blk.mlp
        if moe is None:
            continue
        if getattr(moe, "latent", False):
            raise NotImplementedError("expert parallelism is built for the SwiGLU expert layout; "
                                      "the latent relu^2 layer runs data-parallel")
        E = moe.wgu.shape[0]
        if E % world:
            raise ValueError(f"{E} experts do not divide over {world} ranks")
        El = E // world
        dev = moe.wgu.device
        ep = ExpertParallel(moe.cfg.hidden_size, E, group, dev, impl=impl, **kw)
        with torch.no_grad():
            moe.wgu = torch.nn.Parameter(moe.wgu.data[rank * El:(rank + 1) * El].clone())
            moe.wdown = torch.nn.Parameter(moe.wdown.data[rank * El:(rank + 1) * El].clone())
        moe.wgu.expert_parallel = moe.wdown.expert_parallel = True    # excluded from data-parallel reduction
        moe.ep = ep
