"""RMSNorm (with fused residual add), per-head q/k norm + rotary embedding, SwiGLU.

CUDA tensors run the kernels of ``elementwise.cu``; CPU tensors evaluate the
plain PyTorch expressions below, which double as the test oracle.  These take
the place of the Liger kernels patched in by the reference
(arctic_platform/model/patches/liger.py:25-36) and of its own (1+w) RMSNorm
(arctic_platform/model/implementations/qwen35/models/qwen3_5_moe/modeling_qwen3_5_moe.py:73-87).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib


# ----------------------------------------------------------------- references
def rmsnorm_ref(x, w, eps: float, res=None, w_offset: float = 0.0):
    xs = x.float() + (res.float() if res is not None else 0.0)
    if res is not None:
        xs = xs.to(x.dtype).float()
    rstd = torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + eps)
    y = xs * rstd * (w.float() + w_offset)
    return y.to(x.dtype), xs.to(x.dtype)


def rope_tables(max_pos: int, dim: int, theta: float, device) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


def qknorm_rope_ref(q, k, wq, wk, cos_t, sin_t, pos, eps: float):
    """q [T,Hq,D], k [T,Hkv,D]; rotate-half RoPE over the full head dim."""
    def one(x, w):
        xf = x.float()
        if w is not None:
            xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        D = x.shape[-1]
        c = cos_t[pos.long()][:, None, :]
        s = sin_t[pos.long()][:, None, :]
        a, b = xf[..., : D // 2], xf[..., D // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype)
    return one(q, wq), one(k, wk)


def swiglu_ref(gu):
    g = gu[..., 0::2].float()
    u = gu[..., 1::2].float()
    return (torch.nn.functional.silu(g) * u).to(gu.dtype)


# ----------------------------------------------------------------- RMSNorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, w, eps, w_offset):
        T = x.numel() // x.shape[-1]
        H = x.shape[-1]
        y = torch.empty_like(x)
        res_out = torch.empty_like(x) if res is not None else None
        rstd = torch.empty(T, device=x.device, dtype=torch.float32)
        lib = _lib.cuda_lib()
        _lib.check(lib.apb_rmsnorm_fwd(_lib.ptr(x), _lib.ptr(res), _lib.ptr(w), _lib.ptr(y), _lib.ptr(res_out),
                                       _lib.ptr(rstd), T, H, eps, w_offset, _lib.stream_ptr()), "rmsnorm_fwd")
        ctx.save_for_backward(res_out if res is not None else x, w, rstd)
        ctx.w_offset = w_offset
        ctx.has_res = res is not None
        return y, res_out

    @staticmethod
    def backward(ctx, dy, dres):
        xs, w, rstd = ctx.saved_tensors
        T = xs.numel() // xs.shape[-1]
        H = xs.shape[-1]
        dy = dy.contiguous()
        dx = torch.empty_like(xs)
        acc = getattr(w, "grad_f32", None)
        dw32 = acc if acc is not None else torch.zeros(H, device=xs.device, dtype=torch.float32)
        lib = _lib.cuda_lib()
        dres_c = dres.contiguous() if dres is not None else None
        _lib.check(lib.apb_rmsnorm_bwd(_lib.ptr(dy), _lib.ptr(xs), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres_c),
                                       _lib.ptr(dx), _lib.ptr(dw32), T, H, ctx.w_offset, _lib.stream_ptr()),
                   "rmsnorm_bwd")
        dw = None if acc is not None else dw32.to(w.dtype)
        return dx, (dx if ctx.has_res else None), dw, None, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, res: Optional[torch.Tensor] = None,
            w_offset: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(normed, stream)`` where ``stream = x + res`` (or ``x``) is the residual
    stream to carry forward.  ``w_offset=1`` gives the (1+w) parameterisation."""
    if not x.is_cuda:
        return rmsnorm_ref(x, w, eps, res, w_offset)
    if not x.is_contiguous():
        x = x.contiguous()
    if res is not None and not res.is_contiguous():
        res = res.contiguous()
    y, stream = _RMSNormFn.apply(x, res, w, eps, w_offset)
    return y, (stream if res is not None else x)


# ------------------------------------------------------------ q/k norm + RoPE
class _QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, wq, wk, cos_t, sin_t, pos, Hq, Hkv, D, eps):
        T = qkv.shape[0]
        q = torch.empty((T, Hq, D), device=qkv.device, dtype=qkv.dtype)
        k = torch.empty((T, Hkv, D), device=qkv.device, dtype=qkv.dtype)
        lib = _lib.cuda_lib()
        _lib.check(lib.apb_qknorm_rope_fwd(_lib.ptr(qkv), qkv.stride(0), _lib.ptr(wq), _lib.ptr(wk),
                                           _lib.ptr(cos_t), _lib.ptr(sin_t), _lib.ptr(pos), _lib.ptr(q),
                                           _lib.ptr(k), T, Hq, Hkv, D, D, eps, _lib.stream_ptr()),
                   "qknorm_rope_fwd")
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        ctx.save_for_backward(qkv, wq, wk, cos_t, sin_t, pos)
        ctx.dims = (Hq, Hkv, D, eps)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, wq, wk, cos_t, sin_t, pos = ctx.saved_tensors
        Hq, Hkv, D, eps = ctx.dims
        T = qkv.shape[0]
        dqkv = torch.empty_like(qkv)
        # dv may already live in dqkv's tail (attention backward writes there); else copy.
        dqkv[:, (Hq + Hkv) * D:].view(T, Hkv, D).copy_(dv)
        dq = dq.contiguous()
        dk = dk.contiguous()
        accq = getattr(wq, "grad_f32", None) if wq is not None else None
        acck = getattr(wk, "grad_f32", None) if wk is not None else None
        dwq = accq if accq is not None else torch.zeros(D, device=qkv.device, dtype=torch.float32)
        dwk = acck if acck is not None else torch.zeros(D, device=qkv.device, dtype=torch.float32)
        lib = _lib.cuda_lib()
        _lib.check(lib.apb_qknorm_rope_bwd(_lib.ptr(qkv), qkv.stride(0), _lib.ptr(wq), _lib.ptr(wk),
                                           _lib.ptr(cos_t), _lib.ptr(sin_t), _lib.ptr(pos), _lib.ptr(dq),
                                           _lib.ptr(dk), _lib.ptr(dqkv), dqkv.stride(0), _lib.ptr(dwq),
                                           _lib.ptr(dwk), T, Hq, Hkv, D, D, eps, _lib.stream_ptr()),
                   "qknorm_rope_bwd")
        gq = None if (wq is None or accq is not None) else dwq.to(wq.dtype)
        gk = None if (wk is None or acck is not None) else dwk.to(wk.dtype)
        return dqkv, gq, gk, None, None, None, None, None, None, None


def qknorm_rope(qkv: torch.Tensor, wq, wk, cos_t, sin_t, pos, Hq: int, Hkv: int, D: int, eps: float = 1e-6):
    """Splits ``qkv [T,(Hq+2Hkv)*D]`` into q/k/v, applies per-head RMSNorm (if weights given)
    and rotate-half RoPE to q and k.  Returns ``q [T,Hq,D], k [T,Hkv,D], v [T,Hkv,D]`` (v is a view)."""
    T = qkv.shape[0]
    if not qkv.is_cuda:
        q = qkv[:, : Hq * D].reshape(T, Hq, D)
        k = qkv[:, Hq * D: (Hq + Hkv) * D].reshape(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
        q, k = qknorm_rope_ref(q, k, wq, wk, cos_t, sin_t, pos, eps)
        return q, k, v
    return _QKNormRopeFn.apply(qkv, wq, wk, cos_t, sin_t, pos.to(torch.int32), Hq, Hkv, D, eps)


# ------------------------------------------------------------------- SwiGLU
class _SwiGLUFn(torch.autograd.Function):
    """act = silu(gate) * up on an interleaved ``gu``; forward is normally produced by the
    GEMM epilogue, this Function only attaches the backward."""

    @staticmethod
    def forward(ctx, gu, act_precomputed):
        ctx.save_for_backward(gu)
        if act_precomputed is not None:
            return act_precomputed
        T = gu.numel() // gu.shape[-1]
        I = gu.shape[-1] // 2
        act = torch.empty((*gu.shape[:-1], I), device=gu.device, dtype=gu.dtype)
        _lib.check(_lib.cuda_lib().apb_swiglu_fwd(_lib.ptr(gu), _lib.ptr(act), T, I, _lib.stream_ptr()),
                   "swiglu_fwd")
        return act

    @staticmethod
    def backward(ctx, dact):
        (gu,) = ctx.saved_tensors
        T = gu.numel() // gu.shape[-1]
        I = gu.shape[-1] // 2
        dact = dact.contiguous()
        dgu = torch.empty_like(gu)
        _lib.check(_lib.cuda_lib().apb_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dact), _lib.ptr(dgu), T, I,
                                                  _lib.stream_ptr()), "swiglu_bwd")
        return dgu, None


def swiglu(gu: torch.Tensor, act_precomputed: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not gu.is_cuda:
        return swiglu_ref(gu)
    return _SwiGLUFn.apply(gu.contiguous(), act_precomputed)
