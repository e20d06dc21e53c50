"""Registered loss functions.

Each loss has the signature ``fn(model_outputs, batch, meta, config, device) -> (loss, metrics)``:
``model_outputs`` carries per-token ``logprobs`` (and ``entropy``) on the packed axis together with the
:class:`PackedBatch` that maps tokens back to the padded ``[B, R]`` response grid; ``batch`` holds the
client's padded tensors.  Metrics are emitted as ``{name}.sum`` / ``{name}.tokens`` pairs so that the
server can form global token means (see ``common/utils/metrics.py``).

* ``verl_grpo`` -- verl-shaped PPO/GRPO actor loss (dual-clip, optional entropy bonus and KL-to-reference
  penalty), the loss the reference runs in production
  (arctic_platform/integrations/verl/grpo_loss.py:415-522).
* ``grpo``      -- decoupled-PPO variant with a proximal policy, behaviour-importance cap and the same
  aggregation modes (arctic_platform/rl/processors/grpo.py:195-394).
* ``sft`` / ``sft_ce`` -- next-token cross entropy with global-token normalisation
  (arctic_platform/sft/processor.py:95-292).
"""
from __future__ import annotations

from typing import Any, Dict, Tuple

import torch

from ...common.registry import register_loss_fn
from ...utils.transfer_stats import to_device, to_host
from .functional import (agg_loss, kl_penalty, m2po_mask, masked_sum, ppo_actor_loss_fn, ppo_clip_token_loss,
                         resolve_proximal_logp, sapo_loss_fn)


def _global_info(meta: dict, model_outputs: dict = None) -> dict:
    info = {"dp_size": int(meta.get("dp_size", 1) or 1), "batch_num_tokens": meta.get("batch_num_tokens"),
            "global_batch_size": meta.get("global_batch_size")}
    if model_outputs is not None and model_outputs.get("_full_mask") is not None:
        info["count_mask"] = model_outputs["_full_mask"]
    # the "-norm" aggregation divides by the response horizon of the padded grid, not by the packed token count
    horizon = meta.get("loss_scale_factor")
    if horizon is None and model_outputs is not None and model_outputs.get("packed") is not None:
        horizon = model_outputs["packed"].response_length
    info["loss_scale_factor"] = horizon
    return info


def _token_views(model_outputs: dict, batch: dict, device):
    """Per-token views (packed order) of the padded client tensors."""
    packed = model_outputs["packed"]
    R = packed.response_length

    def take(name, default=None):
        t = batch.get(name)
        if t is None:
            return default
        return packed.gather_from_grid(to_device(t, device)).float()

    mask_grid = batch.get("response_mask")
    if mask_grid is None:
        mask = torch.ones_like(model_outputs["logprobs"], dtype=torch.bool)
    else:
        mask = packed.gather_from_grid(to_device(mask_grid, device)).bool()
    if model_outputs.get("owned") is not None:          # sequence parallelism: this rank's share of the rows
        model_outputs["_full_mask"] = mask
        mask = mask & model_outputs["owned"].to(mask.device)
    seq_ids = torch.div(packed.out_index.to(device), R, rounding_mode="floor")
    return packed, take, mask, seq_ids


def _verl_grpo_fused(lp, old, adv, mask, take, actor, agg_mode, info, meta, model_outputs, packed, device):
    """The token-mean objective on a GPU: ONE kernel produces the loss statistics and the gradient with respect to
    the log-probs (``csrc/rl_ops.cu``) instead of some thirty element-wise kernels plus their autograd graph.  Returns
    ``None`` when the configuration needs the general path (sequence-mean aggregation, an entropy bonus, sequence
    parallelism, no global token count)."""
    from ...ops import rl_ops
    use_kl = bool(actor.get("use_kl_loss", False))
    kl_kind = actor.get("kl_loss_type", "low_var_kl") if use_kl else None
    if (model_outputs.get("owned") is not None or info.get("count_mask") is not None
            or not rl_ops.fused_grpo_supported(lp, agg_mode, info.get("batch_num_tokens"), kl_kind,
                                               model_outputs.get("entropy") is not None)):
        return None
    ref = take("ref_log_prob") if use_kl else None
    if use_kl and ref is None:
        raise KeyError("use_kl_loss needs batch['ref_log_prob']")
    kl_coef = float(actor.get("kl_loss_coef", 0.001)) if use_kl else 0.0
    is_w = meta.get("rollout_is_weights")
    weight = packed.gather_from_grid(to_device(is_w, device)).float() if is_w is not None else None
    scale = float(info["dp_size"]) / float(info["batch_num_tokens"])
    loss, sums = rl_ops.grpo_token_loss(lp, old, adv, mask, scale, ref_lp=ref, kl_kind=kl_kind, kl_coef=kl_coef,
                                        weight=weight, clip_low=0.2, clip_high=0.2, clip_c=3.0)
    ntok, clip_s, kl_s, lower_s, pg_s, kld_s = to_host(sums).tolist()[:6]      # the one device->host sync of the loss
    metrics: Dict[str, Any] = {}
    for name, v in (("actor/pg_clipfrac", clip_s), ("actor/ppo_kl", kl_s), ("actor/pg_clipfrac_lower", lower_s),
                    ("actor/pg_loss", pg_s)):
        metrics[name + ".sum"] = v
        metrics[name + ".tokens"] = ntok
    loss_sum = pg_s
    if use_kl:
        metrics["kl_loss.sum"] = kld_s
        metrics["kl_loss.tokens"] = ntok
        metrics["kl_coef"] = kl_coef
        loss_sum += kl_coef * kld_s
    metrics["loss.sum"] = loss_sum
    metrics["loss.tokens"] = ntok
    return loss, metrics


@register_loss_fn("verl_grpo")
def verl_grpo_loss(model_outputs: dict, batch: dict, meta: dict, config: dict, device) -> Tuple[torch.Tensor, dict]:
    actor = meta.get("actor_config", {}) or {}
    agg_mode = actor.get("loss_agg_mode", "token-mean")
    entropy_coeff = float(actor.get("entropy_coeff", 0.0) or 0.0)
    packed, take, mask, seq_ids = _token_views(model_outputs, batch, device)
    info = _global_info(meta, model_outputs)
    info.update(seq_ids=seq_ids, num_seqs=packed.batch_size)
    lp = model_outputs["logprobs"].float()
    old = take("old_log_probs")
    adv = take("advantages")
    if old is None or adv is None:
        raise KeyError("verl_grpo needs batch['old_log_probs'] and batch['advantages']")
    fused = _verl_grpo_fused(lp, old, adv, mask, take, actor, agg_mode, info, meta, model_outputs, packed, device)
    if fused is not None:
        return fused
    # the clip constants are fixed in the reference implementation (0.2 / 0.2 / 3.0) whatever the config says
    tok_loss, neg_kl, clipped, lower = ppo_clip_token_loss(lp, old, adv, 0.2, 0.2, 3.0)
    is_w = meta.get("rollout_is_weights")
    if is_w is not None:
        tok_loss = tok_loss * packed.gather_from_grid(to_device(is_w, device)).float()
    loss = agg_loss(tok_loss, mask, agg_mode, **info)
    mf = mask.float()
    sums = torch.stack([mf.sum(), (clipped.float() * mf).sum(), (-neg_kl * mf).sum(), (lower.float() * mf).sum(),
                        (tok_loss * mf).sum()]).detach()
    extra = []
    entropy = model_outputs.get("entropy")
    if entropy is not None:
        entropy = entropy.float()
        loss = loss - entropy_coeff * agg_loss(entropy, mask, agg_mode, **info)
        extra.append((entropy * mf).sum().detach())
    use_kl = bool(actor.get("use_kl_loss", False))
    if use_kl:
        ref = take("ref_log_prob")
        if ref is None:
            raise KeyError("use_kl_loss needs batch['ref_log_prob']")
        kld = kl_penalty(lp, ref, actor.get("kl_loss_type", "low_var_kl"))
        kl_coef = float(actor.get("kl_loss_coef", 0.001))
        loss = loss + kl_coef * agg_loss(kld, mask, agg_mode, **info)
        extra.append((kld * mf).sum().detach())
    vals = torch.cat([sums, torch.stack(extra)]) if extra else sums
    vals = to_host(vals).tolist()                   # the one device->host sync of the loss
    ntok, clip_s, kl_s, lower_s, pg_s = vals[:5]
    metrics: Dict[str, Any] = {}
    for name, v in (("actor/pg_clipfrac", clip_s), ("actor/ppo_kl", kl_s), ("actor/pg_clipfrac_lower", lower_s),
                    ("actor/pg_loss", pg_s)):
        metrics[name + ".sum"] = v
        metrics[name + ".tokens"] = ntok
    loss_sum = pg_s
    k = 5
    if entropy is not None:
        metrics["actor/entropy_loss.sum"] = vals[k]
        metrics["actor/entropy_loss.tokens"] = ntok
        loss_sum -= entropy_coeff * vals[k]
        k += 1
    if use_kl:
        metrics["kl_loss.sum"] = vals[k]
        metrics["kl_loss.tokens"] = ntok
        metrics["kl_coef"] = kl_coef
        loss_sum += kl_coef * vals[k]
    metrics["loss.sum"] = loss_sum
    metrics["loss.tokens"] = ntok
    return loss, metrics


@register_loss_fn("grpo")
def grpo_loss(model_outputs: dict, batch: dict, meta: dict, config: dict, device) -> Tuple[torch.Tensor, dict]:
    """Decoupled PPO for synchronous and asynchronous RL.

    The clip is taken against a proximal policy and the behaviour mismatch enters as a capped importance weight.
    Optional pieces, all off by default (config keys in brackets):

    * proximal log-probs sent by the client (``prox_log_probs`` / ``prox_logp`` in the batch) or interpolated from
      per-token ``versions`` and ``current_version`` without an extra forward pass [``prox_logp_method``:
      ``recompute`` | ``loglinear`` | ``metrics``];
    * M2PO second-moment masking of the most off-policy tokens [``m2_threshold``];
    * SAPO soft gate instead of the hard clip [``use_sapo_loss``, ``sapo_tau_pos``, ``sapo_tau_neg``];
    * token- or sequence-level importance ratios [``importance_sampling_level``];
    * dual clip [``c_clip``], behaviour-importance cap [``behav_imp_weight_cap``], per-token correction weights
      (``rollout_is_weights`` in the batch), entropy bonus [``entropy_coeff``], KL penalty to a reference policy
      [``use_kl_loss`` or a non-zero ``kl_ctl``, ``kl_loss_coef``, ``kl_loss_type``], four aggregation modes
      [``loss_agg_mode``]."""
    cfg = {**(meta.get("actor_config") or {}), **(config or {})}
    eps = float(cfg.get("eps_clip", cfg.get("clip_ratio", 0.2)))
    eps_hi = cfg.get("eps_clip_higher")
    eps_hi = float(eps_hi) if eps_hi else None
    c_clip = cfg.get("c_clip")
    cap = cfg.get("behav_imp_weight_cap")
    agg_mode = cfg.get("loss_agg_mode", "token-mean")
    level = cfg.get("importance_sampling_level", "token")
    packed, take, mask, seq_ids = _token_views(model_outputs, batch, device)
    info = _global_info(meta, model_outputs)
    seq_kw = {"seq_ids": seq_ids, "num_seqs": packed.batch_size}
    if model_outputs.get("owned") is not None and (level == "sequence" or cfg.get("use_sapo_loss") or cfg.get("m2_threshold") is not None):
        raise NotImplementedError("sequence-level importance, SAPO and M2PO masking need whole sequences on a rank; "
                                  "they are not available together with sequence parallelism")
    lp = model_outputs["logprobs"].float()
    old = take("old_log_probs")
    if old is None:
        old = lp.detach()                                  # strictly on-policy client: behaviour == current
    adv = take("advantages")
    prox_sent = take("prox_log_probs")
    if prox_sent is None:
        prox_sent = take("prox_logp")
    versions = batch.get("versions")
    if versions is not None:
        versions = packed.gather_from_grid(to_device(versions, device))
    prox = resolve_proximal_logp(prox_sent, cfg.get("prox_logp_method", "recompute"), old, lp.detach(), versions,
                                 cfg.get("current_version"))
    if cfg.get("m2_threshold") is not None:
        mask = m2po_mask(old, prox, mask, float(cfg["m2_threshold"]))
    if cfg.get("use_sapo_loss"):
        if cfg.get("use_decoupled_loss"):
            raise ValueError("SAPO is not compatible with use_decoupled_loss=True.")
        loss, stat = sapo_loss_fn(lp, old, adv, float(cfg.get("sapo_tau_pos", 1.0)), float(cfg.get("sapo_tau_neg", 1.05)),
                                  mask, level, **seq_kw)
    else:
        loss, stat = ppo_actor_loss_fn(lp, prox, old, adv, eps, mask, eps_clip_higher=eps_hi,
                                       c_clip=float(c_clip) if c_clip is not None else None,
                                       behav_imp_weight_cap=float(cap) if cap is not None else None,
                                       importance_sampling_level=level, loss_agg_mode=agg_mode,
                                       rollout_is_weights=take("rollout_is_weights"), **seq_kw, **info)
    ent_coef = float(cfg.get("entropy_coeff", 0.0) or 0.0)
    entropy = model_outputs.get("entropy")
    if entropy is not None and ent_coef:
        loss = loss - ent_coef * agg_loss(entropy.float().detach() if cfg.get("detach_entropy") else entropy.float(),
                                          mask, agg_mode, **seq_kw, **info)
    kl_coef = float(cfg.get("kl_ctl", 0.0) or 0.0) or (float(cfg.get("kl_loss_coef", 0.001)) if cfg.get("use_kl_loss") else 0.0)
    ref = take("ref_log_prob")
    if ref is None:
        ref = take("ref_log_probs")
    if kl_coef:
        if ref is None:
            raise ValueError("a KL penalty is configured but the batch has no ref_log_prob")
        loss = loss + kl_coef * agg_loss(kl_penalty(lp, ref, cfg.get("kl_loss_type", "k3")), mask, agg_mode, **seq_kw, **info)
    mf = mask.float()
    behav = stat.get("behave_imp_weight")
    vals = torch.stack([mf.sum(), (stat["loss"] * mf).sum(), (stat["clip_mask"].float() * mf).sum(),
                        (stat["approx_kl"] * mf).sum(), (stat["importance_weight"] * mf).sum(),
                        (behav * mf).sum() if behav is not None else mf.sum(),
                        (stat["dual_clip_mask"].float() * mf).sum(),
                        ((entropy.float().detach() if entropy is not None else -lp.detach()) * mf).sum()]).detach()
    vals = to_host(vals).tolist()
    n = vals[0]
    metrics = {"loss.sum": vals[1], "loss.tokens": n, "actor/pg_loss.sum": vals[1], "actor/pg_loss.tokens": n,
               "actor/pg_clipfrac.sum": vals[2], "actor/pg_clipfrac.tokens": n,
               "actor/approx_kl.sum": vals[3], "actor/approx_kl.tokens": n,
               "actor/importance_weight.sum": vals[4], "actor/importance_weight.tokens": n,
               "actor/behav_imp_weight.sum": vals[5], "actor/behav_imp_weight.tokens": n,
               "actor/pg_clipfrac_lower.sum": vals[6], "actor/pg_clipfrac_lower.tokens": n,
               "actor/entropy.sum": vals[7], "actor/entropy.tokens": n}
    return loss, metrics


def _sft_core(model_outputs: dict, batch: dict, meta: dict, device):
    packed = model_outputs["packed"]
    lp = model_outputs["logprobs"].float()
    lm = batch.get("loss_mask")
    if lm is None and batch.get("labels") is not None:
        lm = (batch["labels"] != -100)
    mask = (packed.gather_from_grid(to_device(lm, device)).bool() if lm is not None
            else torch.ones_like(lp, dtype=torch.bool))
    if model_outputs.get("owned") is not None:
        mask = mask & model_outputs["owned"].to(mask.device)
    ce_sum = -masked_sum(lp, mask)
    ntok = mask.sum()
    return ce_sum, ntok


@register_loss_fn("sft_ce")
def sft_ce_loss(model_outputs: dict, batch: dict, meta: dict, config: dict, device):
    """Cross entropy summed over this shard's tokens, divided by the GLOBAL token count and multiplied by
    ``dp_size`` (gradients are averaged over ranks afterwards); all-masked shards contribute zero."""
    ce_sum, ntok = _sft_core(model_outputs, batch, meta, device)
    dp = int(meta.get("dp_size", 1) or 1)
    t_global = meta.get("batch_num_tokens")
    denom = float(t_global) if t_global else ntok.clamp_min(1).float()
    loss = ce_sum / denom * dp
    s, n = to_host(torch.stack([ce_sum.detach(), ntok.float()])).tolist()
    return loss, {"loss.sum": s, "loss.tokens": n}


@register_loss_fn("sft")
def sft_loss(model_outputs: dict, batch: dict, meta: dict, config: dict, device):
    """Mean next-token cross entropy of the shard (the Hugging Face ``outputs.loss`` convention)."""
    ce_sum, ntok = _sft_core(model_outputs, batch, meta, device)
    loss = ce_sum / ntok.clamp_min(1).float()
    s, n = to_host(torch.stack([ce_sum.detach(), ntok.float()])).tolist()
    return loss, {"loss.sum": s, "loss.tokens": n}


SFT_LOSS_FNS = {"sft", "sft_ce"}
