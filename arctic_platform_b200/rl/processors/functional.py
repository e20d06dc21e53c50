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
             num_seqs: Optional[int] = None, count_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
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
    if count_mask is not None:
        # this rank holds only part of every sequence's tokens (sequence parallelism): the per-sequence token counts
        # come from the complete mask, so that the ranks' partial sums add up to the sequence's mean
        _s, cnts = _per_sequence(torch.zeros_like(loss_mat), count_mask, seq_ids, num_seqs)
        if global_batch_size is None:
            raise ValueError("global_batch_size is required when a rank holds partial sequences")
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


# ----------------------------------------------------------------------------- off-policy / asynchronous RL pieces
def proximal_logp_approximations(old_logp: torch.Tensor, logprobs: torch.Tensor, versions: torch.Tensor,
                                 current_version: int, method: Optional[str] = None) -> dict:
    """Log-probs of the proximal policy (the policy one version before the one being trained) estimated from the
    behaviour policy's and the current policy's log-probs by how stale each token is.

    A token generated by version ``v`` while training version ``V`` lies ``(V-1-v) / (V-v)`` of the way from the
    behaviour policy to the current one (0 for fresh tokens, -> 1 for very old ones; prompt tokens carry version
    ``< 0`` and get 0).  ``loglinear`` interpolates log-probs, ``linear`` probabilities, ``rollout`` keeps the
    behaviour policy (arctic_platform/rl/processors/grpo.py:88-117)."""
    v = versions.float()
    diff = float(current_version) - v
    alpha = torch.where((diff > 0) & (versions >= 0), (float(current_version) - 1.0 - v) / diff.clamp_min(1e-12),
                        torch.zeros_like(v)).clamp(0.0, 1.0)
    out = {}
    for m in ([method] if method else ["loglinear", "linear", "rollout"]):
        if m == "loglinear":
            out[m] = old_logp + alpha * (logprobs - old_logp)
        elif m == "linear":
            out[m] = torch.log((1 - alpha) * old_logp.exp() + alpha * logprobs.exp() + 1e-10)
        elif m == "rollout":
            out[m] = old_logp.clone()
        else:
            raise ValueError(f"unknown proximal approximation {m!r}")
    return out


def resolve_proximal_logp(prox_logp: Optional[torch.Tensor], method: str, old_logp: torch.Tensor,
                          logprobs: torch.Tensor, versions: Optional[torch.Tensor],
                          current_version: Optional[int]) -> torch.Tensor:
    """``recompute``: the client sent the proximal log-probs (or is on-policy: proximal == behaviour);
    ``loglinear``: no extra forward pass, interpolate by staleness; ``metrics``: client-sent values are required."""
    if method not in ("recompute", "loglinear", "metrics"):
        raise ValueError(f"unknown prox_logp_method {method!r}")
    if prox_logp is None:
        if method == "recompute":
            return old_logp
        if method == "metrics":
            raise ValueError("prox_logp is missing but prox_logp_method='metrics' needs it")
        if versions is None or current_version is None:
            raise ValueError("prox_logp_method='loglinear' needs per-token versions and current_version")
        prox_logp = proximal_logp_approximations(old_logp, logprobs, versions, int(current_version), "loglinear")["loglinear"]
    if not torch.isfinite(prox_logp).all():
        raise RuntimeError(f"proximal log-probs contain NaN or Inf (prox_logp_method={method!r})")
    return prox_logp


def m2po_mask(old_logp: torch.Tensor, prox_logp: torch.Tensor, loss_mask: torch.Tensor, m2_threshold: float) -> torch.Tensor:
    """Second-moment trust region: drops the tokens with the largest squared behaviour/proximal log-ratio until the
    mean of what is left falls under ``m2_threshold``; at least one token survives
    (arctic_platform/rl/processors/grpo.py:168-192)."""
    flat = loss_mask.reshape(-1).bool()
    m2 = (old_logp - prox_logp).square().reshape(-1)[flat]
    n = m2.numel()
    if n == 0:
        return loss_mask
    srt, order = torch.sort(m2, descending=True)
    suffix_mean = srt.flip(0).cumsum(0).flip(0) / torch.arange(n, 0, -1, device=srt.device, dtype=srt.dtype)
    ok = torch.nonzero(suffix_mean < m2_threshold)
    drop = int(ok[0]) if ok.numel() else n - 1
    keep_sorted = torch.ones(n, dtype=torch.bool, device=srt.device)
    keep_sorted[:drop] = False
    keep = torch.empty_like(keep_sorted)
    keep[order] = keep_sorted
    out = torch.zeros_like(flat)
    out[flat] = keep
    return out.view_as(loss_mask)


def sequence_level_ratio_and_advantages(log_ratio: torch.Tensor, advantages: torch.Tensor, loss_mask: torch.Tensor,
                                        seq_ids: Optional[torch.Tensor] = None, num_seqs: Optional[int] = None):
    """GSPO-style importance: every token of a sequence gets ``exp(mean log-ratio of the sequence)`` and the
    sequence's mean advantage.  Packed 1-D tensors need ``seq_ids`` / ``num_seqs``; 2-D tensors are ``[B, R]``."""
    if log_ratio.dim() == 1:
        if seq_ids is None or num_seqs is None:
            raise ValueError("sequence-level importance on packed tokens needs seq_ids and num_seqs")
        lr_sum, cnt = _per_sequence(log_ratio, loss_mask, seq_ids, num_seqs)
        adv_sum, _ = _per_sequence(advantages, loss_mask, seq_ids, num_seqs)
        cnt = cnt.clamp_min(1)
        ratio = torch.exp(lr_sum / cnt)[seq_ids]
        adv = (adv_sum / cnt)[seq_ids]
    else:
        m = loss_mask.to(log_ratio.dtype)
        cnt = m.sum(-1, keepdim=True).clamp_min(1)
        ratio = torch.exp((log_ratio * m).sum(-1, keepdim=True) / cnt).expand_as(log_ratio)
        adv = ((advantages * m).sum(-1, keepdim=True) / cnt).expand_as(log_ratio)
    zero = torch.zeros((), dtype=ratio.dtype, device=ratio.device)
    return torch.where(loss_mask.bool(), ratio, zero), torch.where(loss_mask.bool(), adv, zero)


def ppo_actor_loss_fn(logprobs, proximal_logprobs, old_logprobs, advantages, eps_clip: float, loss_mask,
                      eps_clip_higher: Optional[float] = None, c_clip: Optional[float] = None,
                      behav_imp_weight_cap: Optional[float] = None, importance_sampling_level: str = "token",
                      loss_agg_mode: str = "token-mean", rollout_is_weights: Optional[torch.Tensor] = None,
                      seq_ids: Optional[torch.Tensor] = None, num_seqs: Optional[int] = None, **agg_kwargs):
    """Decoupled PPO: clip against the proximal policy, weight by the (capped) behaviour importance
    ``exp(proximal - behaviour)``; optional dual clip and token- or sequence-level ratios.  Returns the scalar loss
    and per-token statistics (arctic_platform/rl/processors/functional.py:186-262)."""
    loss_mask = loss_mask.bool()
    log_ratio = logprobs - proximal_logprobs
    if importance_sampling_level == "sequence":
        ratio, advantages = sequence_level_ratio_and_advantages(log_ratio, advantages, loss_mask, seq_ids, num_seqs)
    elif importance_sampling_level == "token":
        ratio = torch.where(loss_mask, torch.exp(log_ratio), torch.zeros((), dtype=log_ratio.dtype, device=log_ratio.device))
    else:
        raise ValueError(f"Invalid importance_sampling_level: {importance_sampling_level}.")
    clipped = torch.clamp(ratio, 1.0 - eps_clip, 1.0 + (eps_clip if eps_clip_higher is None else eps_clip_higher))
    l1, l2 = -advantages * ratio, -advantages * clipped
    clip_mask = l1.detach() < l2.detach()
    pg = torch.maximum(l1, l2)
    if c_clip is not None:
        if c_clip <= 1.0:
            raise ValueError(f"c_clip must exceed 1, got {c_clip}")
        l3 = torch.sign(advantages) * c_clip * advantages
        dual_mask = l3.detach() < pg.detach()
        pg = torch.minimum(pg, l3)
    else:
        dual_mask = torch.zeros_like(clip_mask)
    behav_kl = proximal_logprobs - old_logprobs
    behav_w = behav_kl.exp()
    behav_mask = (behav_w <= behav_imp_weight_cap) & loss_mask if behav_imp_weight_cap is not None else loss_mask
    zero = torch.zeros((), dtype=behav_w.dtype, device=behav_w.device)
    behav_w = torch.where(behav_mask, behav_w, zero)
    pg = pg * behav_w.detach()
    if rollout_is_weights is not None:
        pg = pg * rollout_is_weights
    loss = agg_loss(pg, loss_mask, loss_agg_mode, seq_ids=seq_ids, num_seqs=num_seqs, **agg_kwargs)
    stat = {"loss": pg.detach(), "importance_weight": ratio.detach(), "approx_kl": log_ratio.detach(),
            "clip_mask": clip_mask & loss_mask, "dual_clip_mask": dual_mask & loss_mask,
            "behave_imp_weight": behav_w, "behave_approx_kl": torch.where(behav_mask, behav_kl, zero),
            "behave_mask": behav_mask}
    return loss, stat


def sapo_loss_fn(logprobs, old_logprobs, advantages, tau_pos: float, tau_neg: float, loss_mask,
                 importance_sampling_level: str = "token", seq_ids: Optional[torch.Tensor] = None,
                 num_seqs: Optional[int] = None):
    """Soft adaptive policy optimisation: the hard clip is replaced by a sigmoid gate on the ratio,
    ``4 / tau * sigmoid(tau * (ratio - 1))`` with one temperature for positive and one for negative advantages (the
    factor 4 / tau gives unit slope at ratio 1).  Local token mean
    (arctic_platform/rl/processors/functional.py:265-303)."""
    if tau_pos <= 0 or tau_neg <= 0:
        raise ValueError("SAPO temperatures must be positive.")
    loss_mask = loss_mask.bool()
    advantages = advantages.detach()
    log_ratio = logprobs - old_logprobs
    if importance_sampling_level == "sequence":
        ratio, advantages = sequence_level_ratio_and_advantages(log_ratio, advantages, loss_mask, seq_ids, num_seqs)
    elif importance_sampling_level == "token":
        ratio = torch.exp(log_ratio)
    else:
        raise ValueError(f"Invalid importance_sampling_level: {importance_sampling_level}.")
    gate_pos = torch.sigmoid(tau_pos * (ratio - 1.0)) * (4.0 / tau_pos)
    gate_neg = torch.sigmoid(tau_neg * (ratio - 1.0)) * (4.0 / tau_neg)
    gate = torch.where(advantages > 0, gate_pos, gate_neg)
    pg = -gate * advantages
    loss = masked_sum(pg, loss_mask) / loss_mask.sum().clamp_min(1)
    none = torch.zeros_like(loss_mask)
    stat = {"loss": pg.detach(), "importance_weight": ratio.detach(), "approx_kl": log_ratio.detach(),
            "clip_mask": none, "dual_clip_mask": none, "sapo_soft_gate": gate.detach(),
            "sapo_scaled_gate_pos": gate_pos.detach(), "sapo_scaled_gate_neg": gate_neg.detach()}
    return loss, stat


# ------------------------------------------------------------------ names of the proximal-policy options
from enum import Enum  # noqa: E402


class ProxLogpMethod(str, Enum):
    """Where the proximal policy's log-probs come from (``processing.loss_kwargs.prox_logp_method``)."""
    RECOMPUTE = "recompute"      # the client sent them (an extra forward pass), or the data is on-policy
    LOGLINEAR = "loglinear"      # interpolated from behaviour and current log-probs by staleness, no extra pass
    METRICS = "metrics"          # client-sent values are required; approximations are computed for metrics only


class ProxApproxMethod(str, Enum):
    LOGLINEAR = "loglinear"      # interpolate log-probs
    LINEAR = "linear"            # interpolate probabilities
    ROLLOUT = "rollout"          # keep the behaviour policy's values


PROX_LOGP_METHOD_RECOMPUTE = ProxLogpMethod.RECOMPUTE.value
PROX_LOGP_METHOD_LOGLINEAR = ProxLogpMethod.LOGLINEAR.value
PROX_LOGP_METHOD_METRICS = ProxLogpMethod.METRICS.value
PROX_APPROX_METHOD_LOGLINEAR = ProxApproxMethod.LOGLINEAR.value
PROX_APPROX_METHOD_LINEAR = ProxApproxMethod.LINEAR.value
PROX_APPROX_METHOD_ROLLOUT = ProxApproxMethod.ROLLOUT.value
PROX_APPROX_METHODS_ALL = [m.value for m in ProxApproxMethod]

# the reference's spellings of three helpers
compute_prox_logp_approximations = proximal_logp_approximations
_resolve_proximal_logp = resolve_proximal_logp
_compute_sequence_level_ratio_and_advantages = sequence_level_ratio_and_advantages
