"""lm_head + log-softmax + label gather (+ entropy) without a ``[N, V]`` logits tensor.

``lm_head_logprobs(hidden, weight, labels, inv_temperature)`` returns, per row,
``log softmax(hidden @ weight^T * inv_temperature)[label]`` and optionally the entropy
of that distribution.  On CUDA the forward runs the vocabulary GEMM on tcgen05 with an
epilogue that reduces every 128-column tile to (max, sum-exp, sum p*logit, label
logit) partials (``lmhead_logprob.cu``) followed by a small combine kernel; the
backward recomputes logits one row-chunk at a time, forms d(logits) in bf16 and feeds
two GEMMs (dH and dW).  The reference has three variants of this: full logits then a
Triton cross-entropy (arctic_platform/common/utils/tiled_logits.py:74-139), chunked
(``:178-237``) and a recompute-in-backward autograd function (``:240-378``).

CPU tensors use the chunked fp32 expression below (the oracle for the GPU tests).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib, gemm


def logprobs_entropy_ref(hidden, weight, labels, inv_temperature=1.0, with_entropy=True, chunk: int = 4096):
    """Differentiable fp32 reference, chunked over rows so memory stays bounded."""
    lps, ents = [], []
    it = inv_temperature
    for s in range(0, hidden.shape[0], chunk):
        h = hidden[s:s + chunk].float()
        logits = h @ weight.float().t()
        if torch.is_tensor(it):
            logits = logits * it[s:s + chunk].float()[:, None]
        else:
            logits = logits * float(it)
        lse = torch.logsumexp(logits, -1)
        lab = labels[s:s + chunk].long()
        lps.append(logits.gather(-1, lab[:, None]).squeeze(-1) - lse)
        if with_entropy:
            p = torch.softmax(logits, -1)
            ents.append(lse - (p * logits).sum(-1))
    lp = torch.cat(lps) if lps else hidden.new_zeros(0, dtype=torch.float32)
    ent = (torch.cat(ents) if ents else hidden.new_zeros(0, dtype=torch.float32)) if with_entropy else None
    return lp, ent


_FWD = None
_DLOGITS = None


def _fns():
    global _FWD, _DLOGITS
    if _FWD is None:
        c = ctypes
        _FWD = _lib.declare("apb_lmhead_logprob_fwd",
                            [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p,
                             c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_longlong, c.c_longlong, c.c_float,
                             c.c_void_p])
        _DLOGITS = _lib.declare("apb_lmhead_dlogits",
                                [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p,
                                 c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_longlong, c.c_longlong,
                                 c.c_longlong, c.c_float, c.c_void_p])
    return _FWD, _DLOGITS


def _fwd_cuda(hidden, weight, labels, inv_temp_t, inv_temp_s):
    """Returns logprob, entropy, lse (all fp32 [N]); lse is of the temperature-scaled logits."""
    N, H = hidden.shape
    V = weight.shape[0]
    fwd, _ = _fns()
    tiles = (V + 127) // 128
    partial = torch.empty((N, tiles, 4), device=hidden.device, dtype=torch.float32)
    lp = torch.empty(N, device=hidden.device, dtype=torch.float32)
    ent = torch.empty(N, device=hidden.device, dtype=torch.float32)
    lse = torch.empty(N, device=hidden.device, dtype=torch.float32)
    code = fwd(_lib.ptr(hidden), _lib.ptr(weight), _lib.ptr(labels), _lib.ptr(inv_temp_t), _lib.ptr(partial),
               _lib.ptr(lp), _lib.ptr(ent), _lib.ptr(lse), N, V, H, hidden.stride(0), weight.stride(0),
               float(inv_temp_s), _lib.stream_ptr())
    _lib.check(code, "apb_lmhead_logprob_fwd")
    return lp, ent, lse


class _LmHeadLogprobFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, inv_temp_t, inv_temp_s, with_entropy, bwd_chunk):
        hidden = hidden.contiguous()
        labels = labels.to(torch.int32).contiguous()
        lp, ent, lse = _fwd_cuda(hidden, weight, labels, inv_temp_t, inv_temp_s)
        ctx.save_for_backward(hidden, weight, labels, lse, ent, inv_temp_t)
        ctx.inv_temp_s = inv_temp_s
        ctx.bwd_chunk = bwd_chunk
        ctx.with_entropy = with_entropy
        ctx.mark_non_differentiable(lse)
        return lp, (ent if with_entropy else lp.new_zeros(0)), lse

    @staticmethod
    def backward(ctx, g_lp, g_ent, _g_lse):
        hidden, weight, labels, lse, ent, inv_temp_t = ctx.saved_tensors
        _, dlog = _fns()
        N, H = hidden.shape
        V = weight.shape[0]
        g_lp = g_lp.float().contiguous()
        g_ent = g_ent.float().contiguous() if (ctx.with_entropy and g_ent is not None and g_ent.numel()) else None
        d_hidden = torch.empty_like(hidden)
        acc = getattr(weight, "grad_f32", None)
        dw32 = acc if acc is not None else torch.zeros((V, H), device=hidden.device, dtype=torch.float32)
        chunk = ctx.bwd_chunk
        buf = torch.empty((min(chunk, N), V), device=hidden.device, dtype=torch.bfloat16)
        for s in range(0, N, chunk):
            n = min(chunk, N - s)
            h = hidden[s:s + n]
            dl = buf[:n]
            it = inv_temp_t[s:s + n] if inv_temp_t is not None else None
            code = dlog(_lib.ptr(h), _lib.ptr(weight), _lib.ptr(labels[s:s + n]), _lib.ptr(it), _lib.ptr(lse[s:s + n]),
                        _lib.ptr(ent[s:s + n]), _lib.ptr(g_lp[s:s + n]),
                        _lib.ptr(g_ent[s:s + n]) if g_ent is not None else None, _lib.ptr(dl), n, V, H, h.stride(0),
                        weight.stride(0), dl.stride(0), float(ctx.inv_temp_s), _lib.stream_ptr())
            _lib.check(code, "apb_lmhead_dlogits")
            gemm.matmul_nn(dl, weight, out=d_hidden[s:s + n])
            gemm.matmul_tn(dl, h, out=dw32, accumulate=True)
        dw = None if acc is not None else dw32.to(weight.dtype)
        return d_hidden, dw, None, None, None, None, None


def lm_head_logprobs(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                     inv_temperature=1.0, with_entropy: bool = True, bwd_chunk: int = 4096
                     ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``hidden [N,H]``, ``weight [V,H]``, ``labels [N]`` -> ``(logprob [N] fp32, entropy [N] fp32 or None)``.
    ``inv_temperature`` is a float or a per-row tensor ``[N]`` multiplying the logits."""
    if not hidden.is_cuda:
        return logprobs_entropy_ref(hidden, weight, labels, inv_temperature, with_entropy)
    if hidden.shape[0] == 0:
        z = hidden.new_zeros(0, dtype=torch.float32)
        return z, (z if with_entropy else None)
    it_t = inv_temperature.float().contiguous() if torch.is_tensor(inv_temperature) else None
    it_s = 1.0 if it_t is not None else float(inv_temperature)
    lp, ent, _ = _LmHeadLogprobFn.apply(hidden, weight, labels, it_t, it_s, with_entropy, bwd_chunk)
    return lp, (ent if with_entropy else None)
