"""Fused kernels of the RL step that are not GEMM shaped (``csrc/rl_ops.cu``): the token-mean GRPO objective with its
gradient in one pass, and the mixture-of-experts routing decision (scores, top-k, tokens-per-expert histogram).

Both have PyTorch twins in this package -- ``rl/processors/functional.py`` and ``models/moe.route_topk`` -- which are
what runs on CPU and what the GPU tests compare against."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib

_FN = {}
KL_KINDS = {"low_var_kl": 1, "k3": 1, "kl": 2, "k1": 2, "mse": 3, "k2": 3, "abs": 4}


def _fn(name: str):
    if not _FN:
        c = ctypes
        vp, i, ll, f = c.c_void_p, c.c_int, c.c_longlong, c.c_float
        _FN["grpo"] = _lib.declare("apb_grpo_token_loss", [vp, vp, vp, vp, vp, vp, vp, vp, ll, f, f, f, i, f, f, vp])
        _FN["route"] = _lib.declare("apb_moe_route", [vp, ll, vp, i, i, i, i, vp, vp, vp])
    return _FN[name]


class _GrpoTokenLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lp, old_lp, adv, ref_lp, weight, mask, clip_low, clip_high, clip_c, kl_kind, kl_coef, scale):
        n = lp.numel()
        f32 = lambda t: None if t is None else t.detach().to(torch.float32).contiguous()
        lp32, old32, adv32, ref32, w32 = f32(lp), f32(old_lp), f32(adv), f32(ref_lp), f32(weight)
        m8 = mask.detach().to(torch.uint8).contiguous()
        grad = torch.empty(n, device=lp.device, dtype=torch.float32)
        sums = torch.zeros(8, device=lp.device, dtype=torch.float64)
        _lib.check(_fn("grpo")(_lib.ptr(lp32), _lib.ptr(old32), _lib.ptr(adv32), _lib.ptr(ref32), _lib.ptr(w32),
                               _lib.ptr(m8), _lib.ptr(grad), _lib.ptr(sums), n, float(clip_low), float(clip_high),
                               float(clip_c), int(kl_kind), float(kl_coef), float(scale), _lib.stream_ptr()),
                   "apb_grpo_token_loss")
        ctx.save_for_backward(grad)
        ctx.lp_dtype = lp.dtype
        loss = ((sums[4] + kl_coef * sums[5]) * scale).to(torch.float32)
        ctx.mark_non_differentiable(sums)
        return loss, sums

    @staticmethod
    def backward(ctx, g_loss, _g_sums):
        (grad,) = ctx.saved_tensors
        return ((grad * g_loss).to(ctx.lp_dtype),) + (None,) * 11


def grpo_token_loss(lp: torch.Tensor, old_lp: torch.Tensor, adv: torch.Tensor, mask: torch.Tensor, scale: float,
                    ref_lp: Optional[torch.Tensor] = None, kl_kind: Optional[str] = None, kl_coef: float = 0.0,
                    weight: Optional[torch.Tensor] = None, clip_low: float = 0.2, clip_high: float = 0.2,
                    clip_c: float = 3.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """``loss = scale * sum_t mask_t (w_t * dualclip(lp_t, old_t, adv_t) + kl_coef * KL(lp_t, ref_t))`` on CUDA
    tensors, differentiable in ``lp``.  Returns ``(loss, sums)`` with ``sums = [tokens, clipped, sum(-log ratio),
    lower-clipped, sum(policy loss), sum(KL), 0, 0]`` (fp64, no gradient)."""
    kind = 0
    if ref_lp is not None and kl_kind is not None and kl_coef:
        if kl_kind not in KL_KINDS:
            raise NotImplementedError(f"kl penalty {kl_kind!r}")
        kind = KL_KINDS[kl_kind]
    return _GrpoTokenLoss.apply(lp, old_lp, adv, ref_lp if kind else None, weight, mask, clip_low, clip_high, clip_c,
                                kind, kl_coef if kind else 0.0, scale)


def fused_grpo_supported(lp: torch.Tensor, agg_mode: str, batch_num_tokens, kl_kind: Optional[str], has_entropy: bool) -> bool:
    return bool(lp.is_cuda and agg_mode == "token-mean" and batch_num_tokens is not None and not has_entropy
                and (kl_kind is None or kl_kind in KL_KINDS))


@torch.no_grad()
def moe_route(logits: torch.Tensor, k: int, score_func: str = "softmax", bias: Optional[torch.Tensor] = None,
              counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Top-``k`` expert indices ``[T, k]`` (int64, best first) of every token from router ``logits [T, E]``: softmax or
    sigmoid scores, plus ``bias [E]`` for the selection.  ``counts [E]`` (int32), when given, receives +1 per routed
    (token, expert) pair.  No host synchronisation."""
    T, E = logits.shape
    x = logits.detach().to(torch.float32)
    if x.stride(1) != 1:
        x = x.contiguous()
    idx = torch.empty((T, k), device=logits.device, dtype=torch.int64)
    b = None if bias is None else bias.detach().to(torch.float32).contiguous()
    _lib.check(_fn("route")(_lib.ptr(x), x.stride(0), _lib.ptr(b), T, E, k, 1 if score_func == "sigmoid" else 0,
                            _lib.ptr(idx), _lib.ptr(counts), _lib.stream_ptr()), "apb_moe_route")
    return idx
