"""Loss building blocks on per-token tensors.

All functions take ``values`` and a ``mask`` of the same shape -- either the padded ``[B, R]`` response
grid or the packed 1-D token axis with ``seq_ids`` naming each token's sequence -- so the same code
serves the padded client contract and the packed kernels.  Semantics follow
arctic_platform/integrations/verl/grpo_loss.py:93-210,345-407 and
arctic_platform/rl/processors/functional.py:41-303 in the reference.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def masked_sum(values: torch.Tensor, mask: torch.Tensor, axis=None) -> torch.Tensor:
    picked = torch.where(mask.bool(), values, torch.zeros((), dtype=values.dtype, device=values.device))
    return picked.sum() if axis is None else picked.sum(axis)


def masked_mean(values: torch.Tensor, mask: torch.Tensor, axis=None) -> torch.Tensor:
    cnt = mask.sum() if axis is None else mask.sum(axis)
    return masked_sum(values, mask, axis) / (cnt + 1e-8)


def _per_sequence(values, mask, seq_ids, num_seqs):
    """Token sums and token counts per sequence for either layout."""
    if values.dim() == 2:
        m = mask.to(values.dtype)
        return (values * m).sum(-1), m.sum(-1)
    m = mask.to(values.dtype)
    sums = torch.zeros(num_seqs, dtype=values.dtype, device=values.device).index_add_(0, seq_ids, values * m)
    cnts = torch.zeros(num_seqs, dtype=values.dtype, device=values.device).index_add_(0, seq_ids, m)
    return sums, cnts


def agg_loss(loss_mat: torch.Tensor, loss_mask: torch.Tensor, loss_agg_mode: str = "token-mean", dp_size: int = 1,
             batch_num_tokens: Optional[float] = None, global_batch_size: Optional[float] = None,
             loss_scale_factor: Optional[float] = None, seq_ids: Optional[torch.Tensor] = None,
             num_seqs: Optional[int] = None) -> torch.Tensor:
    """Scalar loss that is invariant to how the global batch was split over ranks and micro-batches:
    every mode divides by a GLOBAL denominator and multiplies by ``dp_size`` (gradients are averaged over
    ranks afterwards)."""
    if loss_agg_mode == "token-mean":
        if batch_num_tokens is None:
            if dp_size > 1:
                raise ValueError("(global) batch_num_tokens is required when dp_size > 1")
            batch_num_tokens = loss_mask.sum()
        return masked_sum(loss_mat, loss_mask) / batch_num_tokens * dp_size
    if loss_agg_mode not in ("seq-mean-token-sum", "seq-mean-token-sum-norm", "seq-mean-token-mean"):
        raise ValueError(f"Invalid loss_agg_mode: {loss_agg_mode}")
    if loss_mat.dim() == 1 and seq_ids is None:
        raise ValueError("sequence-level aggregation of packed tokens needs seq_ids")
    sums, cnts = _per_sequence(loss_mat, loss_mask, seq_ids, num_seqs)
    present = (cnts > 0).to(sums.dtype)
    per_seq = sums / (cnts + 1e-8) if loss_agg_mode == "seq-mean-token-mean" else sums
    if global_batch_size is None:
        if dp_size > 1:
            raise ValueError("global_batch_size is required when dp_size > 1")
        global_batch_size = present.sum()
    loss = (per_seq * present).sum() / global_batch_size * dp_size
    if loss_agg_mode == "seq-mean-token-sum-norm":
        horizon = loss_scale_factor if loss_scale_factor is not None else loss_mask.shape[-1]
        loss = loss / horizon
    return loss


def kl_penalty_forward(logprob: torch.Tensor, ref_logprob: torch.Tensor, kind: str) -> torch.Tensor:
    kind = kind.rstrip("+")
    d = logprob - ref_logprob
    if kind in ("kl", "k1"):
        return d
    if kind == "abs":
        return d.abs()
    if kind in ("mse", "k2"):
        return 0.5 * d.square()
    if kind in ("low_var_kl", "k3"):
        k = torch.clamp(-d, min=-20, max=20)
        return torch.clamp(torch.exp(k) - k - 1, min=-10, max=10)
    raise NotImplementedError(f"kl penalty {kind!r}")


def kl_penalty(logprob: torch.Tensor, ref_logprob: torch.Tensor, kind: str) -> torch.Tensor:
    """KL estimate per token.  A trailing ``+`` keeps the estimator's value but routes the gradient through
    the k2 estimator (straight-through), whose expected gradient is the true KL gradient."""
    fwd = kl_penalty_forward(logprob, ref_logprob, kind)
    if not kind.endswith("+") or kind in ("mse", "k2"):
        return fwd
    bwd = 0.5 * (logprob - ref_logprob).square()
    return bwd - bwd.detach() + fwd.detach()


def ppo_clip_token_loss(log_probs, old_log_probs, advantages, clip_low: float = 0.2, clip_high: float = 0.2,
                        clip_c: float = 3.0):
    """Dual-clip PPO per token.  Returns ``(loss, neg_approx_kl, clipped_mask, lower_clipped_mask)``."""
    d = torch.clamp(log_probs - old_log_probs, min=-20.0, max=20.0)
    ratio = torch.exp(d)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1 - clip_low, 1 + clip_high)
    c1 = torch.maximum(l1, l2)
    l3 = -advantages * clip_c
    c2 = torch.minimum(l3, c1)
    loss = torch.where(advantages < 0, c2, c1)
    return loss, d, (l2 > l1), (c1 > l3) & (advantages < 0)


def masked_normalization(x: torch.Tensor, mask: Optional[torch.Tensor] = None, unbiased: bool = False,
                         eps: float = 1e-5, group=None, all_reduce: bool = True) -> torch.Tensor:
    """Whitening with statistics over the masked elements of ALL ranks (three fp64 all-reduces: count, sum,
    sum of squares), as advantage normalisation needs."""
    xf = x.double()
    m = torch.ones_like(xf) if mask is None else mask.double()
    stats = torch.stack([m.sum(), (xf * m).sum(), (xf.square() * m).sum()])
    if all_reduce and dist.is_initialized():
        dist.all_reduce(stats, group=group)
    n, s, ss = stats.unbind()
    mean = s / n.clamp_min(1)
    var = ss / n.clamp_min(1) - mean.square()
    if unbiased:
        var = var * n / (n - 1).clamp_min(1)
    out = (xf - mean) / (var.clamp_min(0).sqrt() + eps)
    return (out * m).to(x.dtype) if mask is not None else out.to(x.dtype)
