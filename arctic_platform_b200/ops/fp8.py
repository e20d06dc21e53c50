"""Block-scaled fp8 (e4m3) linear layers for the sampler.

Weights: ``quantize_fp8_block128`` (one fp32 scale per 128 x 128 block, produced by the trainer -> sampler sync).
Activations: ``quant_act_fp8`` (one scale per token and 128-wide K block).  ``fp8_linear`` multiplies the two on the
tensor cores with the scales folded in per K block (``csrc/gemm_fp8_blockscale.cu``).  CPU tensors run the same
arithmetic on de-quantised values, which is also the oracle of the GPU test."""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from . import _lib

_FN = {}


def _fns():
    if not _FN:
        c = ctypes
        vp, i, ll = c.c_void_p, c.c_int, c.c_longlong
        _FN["qa"] = _lib.declare("apb_quant_act_fp8", [vp, ll, i, i, vp, ll, vp, vp])
        _FN["gemm"] = _lib.declare("apb_gemm_fp8_blockscale", [vp, vp, vp, vp, vp, i, i, i, ll, ll, ll, vp])
    return _FN


def quant_act_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [M, K]`` bf16 (K % 128 == 0) -> ``(q [M, K] float8_e4m3fn, scales [M, K/128] fp32)``."""
    M, K = x.shape
    if K % 128:
        raise ValueError("fp8 activations need K to be a multiple of 128")
    if not x.is_cuda:
        blocks = x.float().view(M, K // 128, 128)
        amax = blocks.abs().amax(-1)
        scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
        return (blocks / scale[..., None]).view(M, K).to(torch.float8_e4m3fn), scale
    x = x.contiguous()
    q = torch.empty((M, K), device=x.device, dtype=torch.float8_e4m3fn)
    scales = torch.empty((M, K // 128), device=x.device, dtype=torch.float32)
    _lib.check(_fns()["qa"](_lib.ptr(x), x.stride(0), M, K, _lib.ptr(q), q.stride(0), _lib.ptr(scales), _lib.stream_ptr()),
               "apb_quant_act_fp8")
    return q, scales


def dequant_weight(wq: torch.Tensor, sw: torch.Tensor) -> torch.Tensor:
    N, K = wq.shape
    s = sw.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    return wq.float() * s


def fp8_gemm(xq: torch.Tensor, sa: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor) -> torch.Tensor:
    """``(xq * sa) @ (wq * sw)^T`` -> bf16 ``[M, N]``."""
    M, K = xq.shape
    N = wq.shape[0]
    if not xq.is_cuda:
        xa = xq.float().view(M, K // 128, 128) * sa[..., None]
        return (xa.view(M, K) @ dequant_weight(wq, sw).t()).to(torch.bfloat16)
    out = torch.empty((M, N), device=xq.device, dtype=torch.bfloat16)
    _lib.check(_fns()["gemm"](_lib.ptr(xq), _lib.ptr(sa), _lib.ptr(wq), _lib.ptr(sw), _lib.ptr(out), M, N, K, xq.stride(0),
                              wq.stride(0), out.stride(0), _lib.stream_ptr()), "apb_gemm_fp8_blockscale")
    return out


def fp8_linear(x: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor) -> torch.Tensor:
    """``x [M, K]`` bf16 times a block-scaled fp8 weight ``wq [N, K]`` / ``sw``: quantises ``x`` per token, then GEMM."""
    xq, sa = quant_act_fp8(x)
    return fp8_gemm(xq, sa, wq, sw)
