"""Sampler tensor parallelism with the collective fused into the GEMM.

* ``ag_gemm`` (column-parallel qkv / gate_up): the activation is row-sharded over ranks; the GEMM's TMA
  producer fetches every A tile from the rank that owns it (plain, non-multicast TMA loads from the peer
  mapping) while earlier tiles are multiplied -- no gathered copy of the activation is ever written.
* ``gemm_rs`` (row-parallel o_proj / down_proj): the epilogue adds each output row into the fp32 buffer of
  the rank that owns the row (``red.add`` over NVLink), ``apb_tp_finalize`` waits for all ranks and converts.
* ``*_collective`` are the NCCL + library-GEMM baselines of the same operations.

The reference gets sampler TP from vLLM (``tensor_parallel_size``, arctic_platform/common/ray_server.py:375)."""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _lib, gemm
from .symm import EpochFlags, SymmetricBuffer

_FN: Dict[str, object] = {}


def _fns():
    if not _FN:
        c = ctypes
        vp, i, ll = c.c_void_p, c.c_int, c.c_longlong
        _FN["ag"] = _lib.declare("apb_gemm_ag", [vp, i, i, vp, vp, i, i, ll, ll, ll, i, vp])
        _FN["rs"] = _lib.declare("apb_gemm_rs", [vp, vp, vp, i, i, i, i, ll, ll, ll, i, i, vp])
        _FN["fin"] = _lib.declare("apb_tp_finalize", [vp, i, i, i, vp, vp, ll, vp])
        _FN["wait"] = _lib.declare("apb_epoch_wait", [vp, i, i, i, vp])
    return _FN


class TPContext:
    """Symmetric scratch of one tensor-parallel group: an activation shard buffer for ``ag_gemm`` and two
    alternating fp32 accumulators for ``gemm_rs``."""

    def __init__(self, device, group=None, max_rows: int = 1024, max_cols: int = 32768):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device)
        self.flags = EpochFlags(device, group if self.world > 1 else False)
        self.max_rows, self.max_cols = max_rows, max_cols
        g = group if self.world > 1 else False
        # two activation buffers used alternately: a rank overwrites buffer b again only two calls later, after it
        # has passed the next call's barrier -- which every peer reaches only once its reads of b have finished --
        # so ONE barrier per call orders both "shards are written" and "shards may be overwritten"
        self.act = [SymmetricBuffer(max_rows * max_cols, torch.bfloat16, device, g) for _ in range(2)]
        self.acc = [SymmetricBuffer(max_rows * max_cols, torch.float32, device, g) for _ in range(2)]
        self._flip = 0
        self._act_flip = 0

    def next_act(self, rows: int, cols: int):
        buf = self.act[self._act_flip]
        self._act_flip ^= 1
        if rows * cols > buf.numel:
            raise ValueError("activation exceeds the tensor-parallel scratch")
        return buf, buf.tensor[: rows * cols].view(rows, cols)


def ag_gemm(ctx: TPContext, x_local: torch.Tensor, w_local: torch.Tensor, bn: int = 0) -> torch.Tensor:
    """``all_gather(x_local, dim 0) @ w_local^T`` -> ``[world * rows, N_local]``; ``x_local [rows, K]``."""
    rows, K = x_local.shape
    N = w_local.shape[0]
    if ctx.world == 1:
        return gemm.matmul_nt(x_local, w_local)
    symm, buf = ctx.next_act(rows, K)
    buf.copy_(x_local)
    f = _fns()
    s = _lib.stream_ptr()
    flags = ctx.flags.ptr_table()
    _lib.check(f["wait"](flags, ctx.rank, ctx.world, ctx.flags.next(), s), "apb_epoch_wait")
    out = torch.empty((ctx.world * rows, N), device=x_local.device, dtype=torch.bfloat16)
    _lib.check(f["ag"](symm.ptr_table(), ctx.world, rows, _lib.ptr(w_local), _lib.ptr(out), N, K, K, w_local.stride(0),
                       out.stride(0), bn, s), "apb_gemm_ag")
    return out


def gemm_rs(ctx: TPContext, x: torch.Tensor, w_local: torch.Tensor, bn: int = 0, splits: int = 1) -> torch.Tensor:
    """``reduce_scatter(x @ w_local^T, dim 0)`` -> ``[M / world, N]``; ``x [M, K_local]``, ``w_local [N, K_local]``."""
    M, K = x.shape
    N = w_local.shape[0]
    if ctx.world == 1:
        return gemm.matmul_nt(x, w_local)
    if M % ctx.world:
        raise ValueError("rows must divide over the tensor-parallel ranks")
    rows = M // ctx.world
    if rows * N > ctx.acc[0].numel:
        raise ValueError("output exceeds the tensor-parallel scratch")
    acc = ctx.acc[ctx._flip]
    ctx._flip ^= 1
    f = _fns()
    s = _lib.stream_ptr()
    _lib.check(f["rs"](_lib.ptr(x), _lib.ptr(w_local), acc.ptr_table(), ctx.world, M, N, K, x.stride(0),
                       w_local.stride(0), N, bn, splits, s), "apb_gemm_rs")
    out = torch.empty((rows, N), device=x.device, dtype=torch.bfloat16)
    _lib.check(f["fin"](ctx.flags.ptr_table(), ctx.rank, ctx.world, ctx.flags.next(), _lib.ptr(acc.tensor), _lib.ptr(out),
                        rows * N, s), "apb_tp_finalize")
    return out


def ag_gemm_collective(x_local: torch.Tensor, w_local: torch.Tensor, group=None) -> torch.Tensor:
    world = dist.get_world_size(group)
    full = torch.empty((world * x_local.shape[0], x_local.shape[1]), device=x_local.device, dtype=x_local.dtype)
    dist.all_gather_into_tensor(full, x_local.contiguous(), group=group)
    return full @ w_local.t()


def gemm_rs_collective(x: torch.Tensor, w_local: torch.Tensor, group=None) -> torch.Tensor:
    world = dist.get_world_size(group)
    part = (x @ w_local.t()).float()
    out = torch.empty((x.shape[0] // world, w_local.shape[0]), device=x.device, dtype=torch.float32)
    dist.reduce_scatter_tensor(out, part, group=group)
    return out.to(x.dtype)
