"""Ulysses sequence parallelism on the packed token axis.

Every rank of the sequence-parallel group holds ``T / sp`` consecutive rows of the packed batch for all the
token-wise work (norms, projections, MLP, lm-head).  Around attention the layout is flipped with an
all-to-all: ``[T/sp, H, D]`` (all heads, my rows) -> ``[T, H/sp, D]`` (my heads, all rows), the segment
attention kernel runs on the full packed axis with the global layout, and a second all-to-all flips back.
When ``sp`` exceeds the number of KV heads the KV heads are replicated first so every rank owns one.
The exchanges are autograd functions whose backward is the opposite exchange.

Counterpart of arctic_platform/model/implementations/qwen35/sequence_parallel.py:33-203 (which assumes a
``[1, S]`` packed batch and calls varlen flash-attention between the exchanges).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x.contiguous(), group=group)
    return out


class _SeqToHead(torch.autograd.Function):
    """``[T/sp, H, D]`` -> ``[T, H/sp, D]``."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return seq_to_head(x, group)

    @staticmethod
    def backward(ctx, g):
        return head_to_seq(g.contiguous(), ctx.group), None


class _HeadToSeq(torch.autograd.Function):
    """``[T, H/sp, D]`` -> ``[T/sp, H, D]``."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return head_to_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return seq_to_head(g.contiguous(), ctx.group), None


def seq_to_head(x: torch.Tensor, group) -> torch.Tensor:
    sp = dist.get_world_size(group)
    Tl, H, D = x.shape
    if H % sp:
        raise ValueError(f"{H} heads do not divide over sp={sp}")
    send = x.view(Tl, sp, H // sp, D).permute(1, 0, 2, 3).contiguous()        # [dest rank, Tl, H/sp, D]
    return _a2a(send, group).view(sp * Tl, H // sp, D)                          # source rank = sequence chunk


def head_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    sp = dist.get_world_size(group)
    T, Hl, D = x.shape
    if T % sp:
        raise ValueError(f"{T} rows do not divide over sp={sp}")
    recv = _a2a(x.view(sp, T // sp, Hl, D), group)                              # [source rank = head group, Tl, Hl, D]
    return recv.permute(1, 0, 2, 3).reshape(T // sp, sp * Hl, D)


def replicate_kv_heads(k: torch.Tensor, v: torch.Tensor, sp: int) -> Tuple[torch.Tensor, torch.Tensor]:
    Hkv = k.shape[1]
    if Hkv >= sp:
        if Hkv % sp:
            raise ValueError(f"{Hkv} KV heads do not divide over sp={sp}")
        return k, v
    if sp % Hkv:
        raise ValueError(f"sp={sp} is not a multiple of the {Hkv} KV heads")
    rep = sp // Hkv
    return k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout, group) -> torch.Tensor:
    """``q [T/sp, Hq, D]``, ``k/v [T/sp, Hkv, D]`` (this rank's rows) -> attention output ``[T/sp, Hq, D]``.
    ``layout`` describes the FULL packed axis (identical on every rank)."""
    from ..ops.attention import segment_attention
    sp = dist.get_world_size(group) if group is not None else 1
    if sp == 1:
        return segment_attention(q, k, v, layout)
    k, v = replicate_kv_heads(k, v, sp)
    qh = _SeqToHead.apply(q, group)
    kh = _SeqToHead.apply(k, group)
    vh = _SeqToHead.apply(v, group)
    oh = segment_attention(qh.contiguous(), kh.contiguous(), vh.contiguous(), layout)
    return _HeadToSeq.apply(oh, group)


def shard_rows(t: torch.Tensor, rank: int, sp: int, pad_value=0) -> torch.Tensor:
    """This rank's ``ceil(T/sp)`` rows of a tensor on the packed axis (the tail is padded)."""
    T = t.shape[0]
    Tl = (T + sp - 1) // sp
    if Tl * sp != T:
        pad = t.new_full((Tl * sp - T,) + tuple(t.shape[1:]), pad_value)
        t = torch.cat([t, pad], 0)
    return t[rank * Tl:(rank + 1) * Tl]


def gather_rows(t_local: torch.Tensor, group, total: Optional[int] = None) -> torch.Tensor:
    """All-gather of the row shards (no autograd); drops the padding when ``total`` is given."""
    sp = dist.get_world_size(group)
    out = torch.empty((sp * t_local.shape[0],) + tuple(t_local.shape[1:]), dtype=t_local.dtype, device=t_local.device)
    dist.all_gather_into_tensor(out.view(-1), t_local.contiguous().view(-1), group=group)
    return out if total is None else out[:total]


class _GatherRowsFn(torch.autograd.Function):
    """All-gather of row shards with a gradient: the backward sums, over the ranks, the gradient every rank holds for
    the full tensor and hands each rank the rows of its own shard (a reduce-scatter; an all-reduce + slice where the
    backend has no reduce-scatter)."""

    @staticmethod
    def forward(ctx, t_local, group):
        ctx.group, ctx.rows = group, t_local.shape[0]
        return gather_rows(t_local, group)

    @staticmethod
    def backward(ctx, grad_full):
        g = grad_full.contiguous()
        r = dist.get_rank(ctx.group)
        if dist.get_backend(ctx.group) == "nccl":
            out = torch.empty((ctx.rows,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out.view(-1), g.view(-1), group=ctx.group)
            return out, None
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g[r * ctx.rows:(r + 1) * ctx.rows].contiguous(), None


def gather_rows_with_grad(t_local: torch.Tensor, group) -> torch.Tensor:
    return _GatherRowsFn.apply(t_local, group)


def apply_sequence_parallelism(model, group) -> None:
    """Routes every block's attention through the Ulysses exchange.  The caller feeds each rank its row shard
    of ``input_ids`` / ``positions`` (``shard_rows``) and the global layout padded to ``sp * ceil(T/sp)`` rows."""
    for blk in model.blocks:
        blk.sp_group = group
        if getattr(blk, "linear_attn", None) is not None:
            # recurrent layers carry state along the whole sequence: every rank runs them on the gathered rows and
            # keeps its own slice (correct, not sequence-scaled; attention and MLP / experts stay sharded)
            blk.linear_attn.sp_group = group
    model.sp_group = group


def pad_layout(layout, padded_tokens: int):
    """The same segments plus one causal segment over the padding rows, so every row of the padded axis is
    written by the attention kernels (an uncovered row would carry uninitialised values into weight gradients)."""
    import numpy as np
    from ..ops.attention import AttnLayout
    T = layout.total_tokens
    if padded_tokens == T:
        return layout
    pad = padded_tokens - T
    seg = np.array([[T, pad, 0, 0, T, pad]], dtype=np.int32)
    return AttnLayout(np.concatenate([layout.segs, seg], 0), padded_tokens)


def sp_token_logprobs(model, packed, group, inv_temperature=1.0, with_entropy: bool = True):
    """Sequence-parallel version of ``models.decoder.token_logprobs``: every rank runs the model on its row shard
    and scores the prediction rows it owns.  Returns ``(logprobs_local, entropy_local, owned)`` where ``owned`` is
    the boolean mask over ``packed.labels`` of the entries this rank produced (their order is preserved)."""
    from ..ops.logprob import lm_head_logprobs
    sp = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T = packed.total_tokens
    Tl = (T + sp - 1) // sp
    ids = shard_rows(packed.input_ids, rank, sp)
    pos = shard_rows(packed.positions, rank, sp)
    layout = pad_layout(packed.layout, Tl * sp)
    hidden = model.forward_hidden(ids, pos, layout)
    owned = (packed.pred_index >= rank * Tl) & (packed.pred_index < (rank + 1) * Tl)
    pred = hidden.index_select(0, packed.pred_index[owned] - rank * Tl)
    it = inv_temperature[owned] if torch.is_tensor(inv_temperature) and inv_temperature.dim() > 0 else inv_temperature
    lp, ent = lm_head_logprobs(pred, model.output_weight, packed.labels[owned], it, with_entropy)
    return lp, ent, owned
