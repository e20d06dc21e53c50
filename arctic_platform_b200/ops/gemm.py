"""bf16 GEMM on tcgen05 tensor cores and the autograd ``linear`` built on it.

On CUDA tensors every product runs in ``gemm_tcgen05.cu``; on CPU tensors (the
fp32 plumbing/oracle configuration) the same functions evaluate the plain
PyTorch expression, which is also the reference the GPU tests compare with.
The reference keeps these products on cuBLAS via ``nn.Linear``
(arctic_platform/model/loaders/huggingface.py:26-43).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

EPI_BF16 = 0
EPI_F32 = 1
EPI_F32_ATOMIC = 2
EPI_F32_ACCUM = 3
EPI_SWIGLU = 4


def _check2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit inner stride, got {tuple(t.shape)} {t.stride()}")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16, got {t.dtype}")


BN_X2 = 1000   # add to a tile width (64 / 128): 3-stage ring, two CTAs per SM -- for skinny problems between one and two waves


def gemm_raw(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor], *, M: int, N: int, K: int,
             a_mn: bool = False, b_mn: bool = False, epi: int = EPI_BF16, splits: int = 1,
             alpha: float = 1.0, bias: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None,
             tile_map: Optional[torch.Tensor] = None, b_rows: int = 0, bn: int = 0, max_ctas: int = 0,
             stream=None) -> None:
    """Launches the kernel on already validated tensors (see ``apb_gemm_bf16``)."""
    lib = _lib.cuda_lib()
    code = lib.apb_gemm_bf16(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0),
        out.stride(0) if out is not None else 0, int(a_mn), int(b_mn), epi, splits, float(alpha),
        _lib.ptr(bias), _lib.ptr(out2), out2.stride(0) if out2 is not None else 0,
        _lib.ptr(tile_map), 0 if tile_map is None else tile_map.shape[0], b_rows, bn, max_ctas,
        _lib.stream_ptr(stream))
    _lib.check(code, "apb_gemm_bf16")


def matmul_nt(a: torch.Tensor, b: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
              accumulate: bool = False, alpha: float = 1.0, bn: int = 0) -> torch.Tensor:
    """``a[M,K] @ b[N,K]^T`` (the forward of a linear layer)."""
    if not a.is_cuda:
        r = alpha * (a.float() @ b.float().t())
        if bias is not None:
            r = r + bias.float()
        if out is not None:
            if accumulate:
                out.add_(r.to(out.dtype))
            else:
                out.copy_(r.to(out.dtype))
            return out
        return r.to(out_dtype if a.dtype == torch.bfloat16 else a.dtype)
    _check2d(a, "a")
    _check2d(b, "b")
    M, K = a.shape
    N = b.shape[0]
    if b.shape[1] != K:
        raise ValueError("inner dimensions differ")
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype)
        accumulate = False
    if out.dtype == torch.bfloat16:
        if accumulate:
            raise ValueError("accumulation needs an fp32 output")
        epi = EPI_BF16
    else:
        epi = EPI_F32_ACCUM if accumulate else EPI_F32
    gemm_raw(a, b, out, M=M, N=N, K=K, epi=epi, alpha=alpha, bias=bias, bn=bn)
    return out


def matmul_nn(a: torch.Tensor, b: torch.Tensor, *, out: Optional[torch.Tensor] = None,
              out_dtype: torch.dtype = torch.bfloat16, bn: int = 0) -> torch.Tensor:
    """``a[M,K] @ b[K,N]`` with b row-major (the data gradient dX = dY @ W)."""
    if not a.is_cuda:
        r = a.float() @ b.float()
        return r.to(out_dtype if a.dtype == torch.bfloat16 else a.dtype)
    _check2d(a, "a")
    _check2d(b, "b")
    M, K = a.shape
    N = b.shape[1]
    if b.shape[0] != K:
        raise ValueError("inner dimensions differ")
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype)
    epi = EPI_BF16 if out.dtype == torch.bfloat16 else EPI_F32
    gemm_raw(a, b, out, M=M, N=N, K=K, b_mn=True, epi=epi, bn=bn)
    return out


def matmul_tn(a: torch.Tensor, b: torch.Tensor, *, out: Optional[torch.Tensor] = None,
              out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False, bn: int = 0) -> torch.Tensor:
    """``a[K,M]^T @ b[K,N]`` (the weight gradient dW = dY^T @ X), optionally accumulated into fp32 ``out``."""
    if not a.is_cuda:
        r = a.float().t() @ b.float()
        if out is not None:
            if accumulate:
                out.add_(r.to(out.dtype))
            else:
                out.copy_(r.to(out.dtype))
            return out
        return r.to(out_dtype if a.dtype == torch.bfloat16 else a.dtype)
    _check2d(a, "a")
    _check2d(b, "b")
    K, M = a.shape
    N = b.shape[1]
    if b.shape[0] != K:
        raise ValueError("inner dimensions differ")
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype)
        accumulate = False
    if out.dtype == torch.bfloat16:
        if accumulate:
            raise ValueError("accumulation needs an fp32 output")
        epi = EPI_BF16
    else:
        epi = EPI_F32_ACCUM if accumulate else EPI_F32
    gemm_raw(a, b, out, M=M, N=N, K=K, a_mn=True, b_mn=True, epi=epi, bn=bn)
    return out


def gate_up_swiglu(x: torch.Tensor, w_gu: torch.Tensor, *, keep_gu: bool = True):
    """``gu = x @ w_gu^T`` with gate/up rows interleaved in ``w_gu`` and ``act = silu(gate) * up``
    produced in the GEMM epilogue.  Returns ``(gu or None, act)``."""
    if not x.is_cuda:
        gu = (x.float() @ w_gu.float().t())
        act = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]
        return (gu.to(x.dtype) if keep_gu else None), act.to(x.dtype)
    _check2d(x, "x")
    _check2d(w_gu, "w_gu")
    M, K = x.shape
    N = w_gu.shape[0]
    gu = torch.empty((M, N), device=x.device, dtype=torch.bfloat16) if keep_gu else None
    act = torch.empty((M, N // 2), device=x.device, dtype=torch.bfloat16)
    gemm_raw(x, w_gu, gu, M=M, N=N, K=K, epi=EPI_SWIGLU, out2=act)
    return gu, act


class _LinearFn(torch.autograd.Function):
    """y = x @ w^T.  The weight gradient is written to ``w.grad_f32`` (fp32 accumulation
    buffer owned by the ZeRO partitioner) when that attribute exists, else returned."""

    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        x2 = x.reshape(-1, x.shape[-1])
        y = matmul_nt(x2, w, bias=bias)
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = matmul_nn(dy2, w).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            acc = getattr(w, "grad_f32", None)
            if acc is not None:
                matmul_tn(dy2, x2, out=acc, accumulate=True)
                dw = None
            else:
                dw = matmul_tn(dy2, x2, out_dtype=w.dtype if not w.is_cuda else torch.bfloat16)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.is_cuda and (w.shape[0] % 8 or w.shape[1] % 8):
        # the TMA-fed kernel needs 16-byte rows on both sides; a projection this narrow (a 4-expert router, a
        # per-head scalar gate) is a few hundred FLOPs per token and goes through the library
        return torch.nn.functional.linear(x, w, bias)
    return _LinearFn.apply(x, w, bias)
