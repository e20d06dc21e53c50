"""The verl-shaped GRPO / PPO objective registered as ``"verl_grpo"`` (clamped log-ratio, clip 0.2 / 0.2, dual clip
c = 3, ``agg_loss`` with the global token count) and the helper names verl recipes import beside it.  The loss itself
lives with the other losses (``rl/processors/losses.py``); the pieces here are its building blocks under the
reference's names (arctic_platform/integrations/verl/grpo_loss.py:41-522), expressed with this build's functional ops.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch

from ...rl.processors.functional import (agg_loss, kl_penalty, kl_penalty_forward, masked_mean, masked_sum,  # noqa: F401
                                         ppo_clip_token_loss)
from ...rl.processors.losses import verl_grpo_loss  # noqa: F401

__all__ = ["VerlPolicyConfig", "agg_loss", "compute_policy_loss_vanilla", "kl_penalty", "kl_penalty_forward",
           "mask_and_pad_for_log_probs", "masked_mean", "masked_sum", "shift_log_probs_left", "verl_grpo_loss"]


class VerlPolicyConfig:
    """The actor settings the objective reads, with verl's defaults."""

    def __init__(self, actor_config_dict: Optional[dict] = None, policy_loss_config_dict: Optional[dict] = None):
        a, p = actor_config_dict or {}, policy_loss_config_dict or {}
        self.loss_agg_mode = a.get("loss_agg_mode", "token-mean")
        self.kl_loss_coef = a.get("kl_loss_coef", 0.001)
        self.kl_loss_type = a.get("kl_loss_type", "low_var_kl")
        self.clip_ratio = a.get("clip_ratio", 0.2)
        self.clip_ratio_low = a.get("clip_ratio_low", self.clip_ratio)
        self.clip_ratio_high = a.get("clip_ratio_high", self.clip_ratio)
        self.clip_ratio_c = a.get("clip_ratio_c", 3.0)
        self.entropy_coeff = a.get("entropy_coeff", 0.0)
        self.use_kl_loss = a.get("use_kl_loss", False)
        self.loss_mode = p.get("loss_mode", "vanilla")
        if self.clip_ratio_c <= 1.0:
            raise ValueError(f"clip_ratio_c must be greater than 1 for dual-clip PPO, got {self.clip_ratio_c}")


def compute_policy_loss_vanilla(old_log_probs: torch.Tensor, log_probs: torch.Tensor, advantages: torch.Tensor,
                                response_mask: torch.Tensor, loss_agg_mode: str = "token-mean",
                                global_batch_info: Optional[Dict[str, Any]] = None,
                                rollout_is_weights: Optional[torch.Tensor] = None,
                                config: Optional[VerlPolicyConfig] = None) -> Tuple[torch.Tensor, Dict[str, float]]:
    """Dual-clip PPO over ``[B, R]`` grids -> ``(loss, metrics)`` with paired ``{name}.sum`` / ``{name}.tokens``
    metrics (one device -> host read).  ``global_batch_info`` carries ``dp_size`` / ``batch_num_tokens`` /
    ``global_batch_size`` for ``agg_loss``; ``rollout_is_weights`` multiplies the per-token losses."""
    cfg = config or VerlPolicyConfig()
    per_tok, log_ratio, clipped, lower = ppo_clip_token_loss(log_probs, old_log_probs, advantages, cfg.clip_ratio_low,
                                                             cfg.clip_ratio_high, cfg.clip_ratio_c)
    if rollout_is_weights is not None:
        per_tok = per_tok * rollout_is_weights
    loss = agg_loss(per_tok, response_mask, loss_agg_mode, **(global_batch_info or {}))
    m = response_mask.to(per_tok.dtype)
    stats = torch.stack([m.sum(), (clipped.to(m.dtype) * m).sum(), (-log_ratio * m).sum(), (lower.to(m.dtype) * m).sum(),
                         (per_tok * m).sum()]).detach().cpu().tolist()
    n = stats[0]
    return loss, {"actor/pg_clipfrac.sum": stats[1], "actor/pg_clipfrac.tokens": n, "actor/ppo_kl.sum": stats[2],
                  "actor/ppo_kl.tokens": n, "actor/pg_clipfrac_lower.sum": stats[3], "actor/pg_clipfrac_lower.tokens": n,
                  "actor/pg_loss.sum": stats[4], "actor/pg_loss.tokens": n}


def mask_and_pad_for_log_probs(tensor: torch.Tensor, batch: Dict[str, Any]) -> torch.Tensor:
    """Per-token values of a packed ``[total tokens]`` buffer moved to the predict-next convention: inside every
    response window (``sequence_offsets[i] - response_lens[i] .. sequence_offsets[i]``) position ``t`` receives the
    value of position ``t - 1``; everything outside the windows is zero.  No loop over sequences."""
    values = tensor.values() if getattr(tensor, "is_nested", False) else tensor
    n = values.shape[0]
    ends = torch.as_tensor(batch["sequence_offsets"], device=values.device, dtype=torch.long).reshape(-1)
    starts = ends - torch.as_tensor(batch["response_lens"], device=values.device, dtype=torch.long).reshape(-1)
    delta = torch.zeros(n + 1, dtype=torch.int32, device=values.device)
    delta.index_add_(0, starts, torch.ones_like(starts, dtype=torch.int32))
    delta.index_add_(0, ends, torch.full_like(ends, -1, dtype=torch.int32))
    inside = delta[:n].cumsum(0) > 0
    shifted = torch.zeros_like(values)
    shifted[1:] = values[:-1]
    return torch.where(inside, shifted, torch.zeros_like(values))


def shift_log_probs_left(tensor: torch.Tensor, batch: Optional[Dict[str, Any]] = None) -> torch.Tensor:
    """Response-aligned values (what the prompt-deduplicated path produces) need no shift: the flat values as they are."""
    return tensor.values() if getattr(tensor, "is_nested", False) else tensor
