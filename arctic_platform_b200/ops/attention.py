"""Segment attention: packed varlen causal attention and ZoRRo shared-prefix attention.

A *segment* is a run of query rows on the packed token axis together with two key
ranges on the same axis: a fully visible **prefix** range (under ZoRRo the group's
prompt, stored once) and its **own** range under a bottom-right aligned causal mask::

    segs[i] = (q_start, q_len, pre_start, pre_len, own_start, own_len)

* packed causal varlen (``cu_seqlens``): ``pre_len = 0``, own range = the sequence;
* ZoRRo prompt segment: own range = the prompt itself;
* ZoRRo response segment: prefix = its group's prompt, own range = the response.

The reference obtains the same numbers by building per-sample ``[prompt || response]``
K/V with ``torch.cat`` and calling flash-attn varlen twice per layer
(arctic_platform/rl/zorro_train/qwen_attention_patcher.py:1197-1231).  Here one kernel
launch handles every segment and the prompt K/V is never replicated; its backward
accumulates the prompt's dK/dV over all rollouts inside one CTA.

CUDA tensors run ``attention_fwd.cu`` / ``attention_bwd.cu``; CPU tensors run the dense
masked-softmax reference below (also the oracle of the GPU tests).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib


@dataclass
class AttnLayout:
    """Host description of the segments of one packed batch plus cached device tables."""
    segs: np.ndarray            # int32 [S, 6]
    total_tokens: int
    _fwd: dict = None           # (Hq, Hkv, device) -> work tensor
    _bwd: dict = None

    def __post_init__(self):
        self.segs = np.ascontiguousarray(self.segs, dtype=np.int32).reshape(-1, 6)
        self._fwd = {}
        self._bwd = {}

    @staticmethod
    def from_cu_seqlens(cu_seqlens) -> "AttnLayout":
        cu = np.asarray(cu_seqlens, dtype=np.int64)
        from ..utils import checked
        if checked.enabled():
            checked.check_cu_seqlens(cu)
        starts, lens = cu[:-1], cu[1:] - cu[:-1]
        segs = np.stack([starts, lens, np.zeros_like(starts), np.zeros_like(starts), starts, lens], 1)
        return AttnLayout(segs[lens > 0], int(cu[-1]))

    def fwd_work(self, Hq: int, Hkv: int, device) -> torch.Tensor:
        key = (Hq, Hkv, str(device))
        if key not in self._fwd:
            rt = _lib.rt_lib()
            fn = rt.apb_rt_attn_fwd_work
            fn.restype = ctypes.c_int64
            fn.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                           ctypes.c_int64]
            n = fn(self.segs.ctypes.data, len(self.segs), Hq, Hkv, None, 0)
            out = np.empty((max(n, 1), 8), dtype=np.int32)
            fn(self.segs.ctypes.data, len(self.segs), Hq, Hkv, out.ctypes.data, n)
            self._fwd[key] = torch.from_numpy(out[:n]).to(device)
        return self._fwd[key]

    def bwd_work(self, Hkv: int, device):
        key = (Hkv, str(device))
        if key not in self._bwd:
            rt = _lib.rt_lib()
            fn = rt.apb_rt_attn_bwd_work
            fn.restype = ctypes.c_int32
            fn.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64,
                           ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
            counts = np.zeros(2, dtype=np.int64)
            rc = fn(self.segs.ctypes.data, len(self.segs), Hkv, None, 0, None, 0, counts.ctypes.data)
            if rc != 0:
                raise ValueError("attention layout has overlapping key ranges with different extents")
            cta = np.empty((max(counts[0], 1), 8), dtype=np.int32)
            lst = np.empty((max(counts[1], 1), 4), dtype=np.int32)
            fn(self.segs.ctypes.data, len(self.segs), Hkv, cta.ctypes.data, counts[0], lst.ctypes.data, counts[1],
               counts.ctypes.data)
            self._bwd[key] = (torch.from_numpy(cta[:counts[0]]).to(device),
                              torch.from_numpy(lst[:counts[1]]).to(device))
        return self._bwd[key]


def attention_ref(q, k, v, layout: AttnLayout, scale: Optional[float] = None, return_lse: bool = False):
    """Dense fp32 reference.  q [T,Hq,D], k/v [T,Hkv,D] -> o [T,Hq,D] (differentiable)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros((T, Hq, D), dtype=torch.float32, device=q.device)
    lse = torch.full((Hq, T), float("-inf"), dtype=torch.float32, device=q.device)
    pieces = []
    for qs, ql, ps, pl, os_, ol in layout.segs.tolist():
        qq = q[qs:qs + ql].float()
        kk = torch.cat([k[ps:ps + pl], k[os_:os_ + ol]], 0).float().repeat_interleave(rep, 1)
        vv = torch.cat([v[ps:ps + pl], v[os_:os_ + ol]], 0).float().repeat_interleave(rep, 1)
        s = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        rows = torch.arange(ql, device=q.device)[:, None]
        cols = torch.arange(ol, device=q.device)[None, :]
        own_mask = cols <= rows + (ol - ql)
        mask = torch.cat([torch.ones((ql, pl), dtype=torch.bool, device=q.device), own_mask], 1)
        s = s.masked_fill(~mask[None], float("-inf"))
        l = torch.logsumexp(s, -1)
        p = torch.exp(s - l[..., None])
        p = torch.nan_to_num(p, nan=0.0)
        o = torch.einsum("hqk,khd->qhd", p, vv)
        pieces.append((qs, ql, o, l))
    for qs, ql, o, l in pieces:
        out = out.index_put((torch.arange(qs, qs + ql, device=q.device),), o)
        lse[:, qs:qs + ql] = l.detach()
    out = out.to(q.dtype)
    return (out, lse) if return_lse else out


_FWD = None
_BWD = None
_DELTA = None


def _fwd_fn():
    global _FWD
    if _FWD is None:
        c = ctypes
        _FWD = _lib.declare("apb_attn_fwd", [c.c_void_p] * 6 + [c.c_int] * 5 + [c.c_longlong] * 4 + [c.c_float, c.c_void_p])
    return _FWD


def attention_fwd_cuda(q, k, v, layout: AttnLayout, scale: float, need_lse: bool = True):
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.stride(2) != 1 or t.stride(1) != D:
            raise ValueError(f"{name} must be [T,H,D] with contiguous heads")
    work = layout.fwd_work(Hq, Hkv, q.device)
    o = torch.empty((T, Hq, D), device=q.device, dtype=q.dtype)
    lse = torch.empty((Hq, T), device=q.device, dtype=torch.float32) if need_lse else None
    code = _fwd_fn()(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(work),
                     work.shape[0], T, Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), o.stride(0),
                     scale, _lib.stream_ptr())
    _lib.check(code, "apb_attn_fwd")
    return o, lse


def _bwd_fn():
    global _BWD
    if _BWD is None:
        c = ctypes
        _BWD = _lib.declare("apb_attn_bwd", [c.c_void_p] * 11 + [c.c_int, c.c_void_p] + [c.c_int] * 4 +
                            [c.c_longlong] * 8 + [c.c_float, c.c_void_p])
    return _BWD


def attention_bwd_cuda(q, k, v, o, d_o, lse, layout: AttnLayout, scale: float):
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    if D != 128:
        raise NotImplementedError("the tcgen05 attention backward supports head_dim 128")
    cta, lst = layout.bwd_work(Hkv, q.device)
    d_o = d_o.contiguous()
    delta = torch.empty((Hq, T), device=q.device, dtype=torch.float32)
    dq_acc = torch.zeros((T, Hq * D), device=q.device, dtype=torch.float32)
    dk = torch.zeros((T, Hkv, D), device=q.device, dtype=q.dtype)
    dv = torch.zeros((T, Hkv, D), device=q.device, dtype=q.dtype)
    code = _bwd_fn()(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(d_o), _lib.ptr(lse),
                     _lib.ptr(delta), _lib.ptr(dq_acc), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(cta), cta.shape[0],
                     _lib.ptr(lst), T, Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), o.stride(0),
                     d_o.stride(0), dq_acc.stride(0), dk.stride(0), dv.stride(0), scale, _lib.stream_ptr())
    _lib.check(code, "apb_attn_bwd")
    return dq_acc.view(T, Hq, D).to(q.dtype), dk, dv


class _SegmentAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, layout, scale):
        o, lse = attention_fwd_cuda(q, k, v, layout, scale, need_lse=True)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.layout = layout
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = attention_bwd_cuda(q, k, v, o, d_o, lse, ctx.layout, ctx.scale)
        return dq, dk, dv, None, None


def segment_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout: AttnLayout,
                      scale: Optional[float] = None) -> torch.Tensor:
    """q [T,Hq,D], k/v [T,Hkv,D] on the packed token axis -> o [T,Hq,D]."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if not q.is_cuda or q.shape[-1] != 128:
        # the tcgen05 kernels are written for head_dim 128 (the Qwen3 family); other head sizes (64: test presets,
        # 256: Qwen3.5 hybrids) run the dense PyTorch expression, on either device
        return attention_ref(q, k, v, layout, scale)
    return _SegmentAttentionFn.apply(q, k, v, layout, scale)
