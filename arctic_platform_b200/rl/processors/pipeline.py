"""One forward (and backward) pass of a worker over its shard of the batch.

``run_pipeline`` takes the client's padded tensors, builds the packed (optionally prompt-deduplicated)
layout on the host in one pass, runs the model once, evaluates the registered loss and, when asked,
back-propagates into the engine's flat gradient buffer.  Outputs go back padded to ``[B, R]``.

The reference's pipeline (arctic_platform/rl/processors/pipeline.py:222-499) un-pads 2-D side tensors to
1-D, calls a monkey-patched HF model, collects logits/log-probs through post-processors and re-pads; here
the model is packed-native and log-probs/entropy come straight out of the fused lm-head kernel, so the
post-processors reduce to the entropy switch and the temperature.
"""
from __future__ import annotations

import time
from typing import Any, Dict, List, Optional

import torch

from ...utils import sft_profile
from ...utils.transfer_stats import to_device, to_host
from ...common.registry import LOSS_FNS, POST_PROCESSORS, register_post_processor, resolve_fn
from ...models.decoder import token_logprobs
from ..zorro_train.layout import PackedBatch, build_packed_batch, build_plain_packed
from . import losses as _losses  # noqa: F401  (registers the built-in losses)
from .padding import *  # noqa: F401,F403  (padded grid <-> packed row helpers, importable from here as well)
from ...common.utils.batch import dump_dict_payload  # noqa: F401
from ...common.utils.tiled_logits import (chunked_logprobs_and_entropy_from_logits,  # noqa: F401
                                          fast_logprobs_and_entropy_from_logits, logprobs_from_logits)

DEFAULT_PROCESSING = {"pre": [], "post": ["compute_entropy_and_logprobs"], "loss_fn": "verl_grpo", "loss_kwargs": {}}


@register_post_processor("identity")
def _identity(model_outputs, batch, meta, config, device):
    return model_outputs


@register_post_processor("compute_entropy_and_logprobs")
def _entropy_and_logprobs(model_outputs, batch, meta, config, device):
    """Log-probs and entropy are produced by the fused lm-head kernel; nothing left to compute."""
    return model_outputs


@register_post_processor("compute_entropy")
def _entropy(model_outputs, batch, meta, config, device):
    return model_outputs


@register_post_processor("apply_temperature")
def _temperature(model_outputs, batch, meta, config, device):
    """Temperature is folded into the lm-head epilogue (``meta['temperature']``)."""
    return model_outputs


def response_length_of(batch: dict, meta: dict) -> int:
    for key in ("responses", "response_mask", "old_log_probs", "advantages"):
        t = batch.get(key)
        if torch.is_tensor(t) and t.dim() == 2:
            return int(t.shape[1])
    if meta.get("response_length"):
        return int(meta["response_length"])
    raise KeyError("cannot infer the response length: send 'responses'/'response_mask' or meta['response_length']")


def pack_for_model(batch: dict, meta: dict, sft: bool) -> PackedBatch:
    ids = batch["input_ids"]
    mask = batch.get("attention_mask")
    if mask is None:
        mask = torch.ones_like(ids)
    if sft:
        cu = batch.get("cu_seqlens")
        pos = batch.get("position_ids")
        prepacked = ids.dim() == 2 and ids.shape[0] == 1 and (
            cu is not None or (torch.is_tensor(pos) and pos.numel() == ids.numel() and bool((pos.reshape(-1)[1:] == 0).any())))
        if prepacked:
            from ..zorro_train.layout import build_prepacked
            return build_prepacked(ids, pos, cu)              # the client packed several documents into one row
        return build_plain_packed(ids, mask)
    return build_packed_batch(ids, mask, response_length_of(batch, meta),
                              dedup=bool(meta.get("zorro_train_enable", True)))


def action_masks_of(batch: Dict[str, Any], packed):
    """Token-set constraints of the batch, one row per prediction of ``packed``.  The batch carries them densely on
    the response grid: ``action_mask_tokens [B, R, K]`` (padded with -1) and ``action_mask_allow [B, R]`` (1 = the
    listed tokens are the legal set, 0 = they are illegal, -1 = unconstrained position)."""
    toks = batch.get("action_mask_tokens")
    if toks is None:
        return None
    from ...utils.action_masks import ActionMasks
    allow = batch.get("action_mask_allow")
    B, R, K = toks.shape
    if allow is None:
        allow = torch.where((toks >= 0).any(-1), 1, -1)
    rows = packed.out_index.to("cpu")
    return ActionMasks.from_grid(toks.reshape(B * R, K).to("cpu")[rows], allow.reshape(B * R).to("cpu")[rows])


def _sp_logprobs(model, packed, sp_group, inv_temperature, want_entropy: bool, batch):
    """Ulysses sequence parallelism: this rank runs its row shard of the packed axis and scores the prediction rows
    that fall into it.  Returns full-length ``[N]`` tensors (zero where another rank scores) and the ownership mask."""
    from ...parallel.ulysses import sp_token_logprobs
    if batch.get("action_mask_tokens") is not None:
        raise NotImplementedError("action masks are not supported together with sequence parallelism")
    lp_loc, ent_loc, owned = sp_token_logprobs(model, packed, sp_group, inv_temperature, want_entropy)
    idx = owned.nonzero()[:, 0]
    N = packed.labels.numel()
    lp = torch.zeros(N, dtype=lp_loc.dtype, device=lp_loc.device).index_put((idx,), lp_loc)
    ent = torch.zeros(N, dtype=lp_loc.dtype, device=lp_loc.device).index_put((idx,), ent_loc) if ent_loc is not None else None
    return lp, ent, owned


def run_pipeline(engine, batch: Dict[str, torch.Tensor], meta: Optional[dict] = None,
                 processing: Optional[dict] = None, device=None, backward: bool = True,
                 return_tensors: bool = True) -> Dict[str, Any]:
    meta = dict(meta or {})
    processing = {**DEFAULT_PROCESSING, **(processing or {})}
    model = engine.model
    device = device or next(model.parameters()).device
    loss_name = processing.get("loss_fn")
    sft = loss_name in _losses.SFT_LOSS_FNS or bool(meta.get("plain_packing"))
    t0 = time.perf_counter()
    with sft_profile.timed("h2d"):
        packed = pack_for_model(batch, meta, sft).to(device)
    actor = meta.get("actor_config", {}) or {}
    want_entropy = bool(actor.get("entropy_coeff", 0.0)) or bool(meta.get("compute_entropy", not backward))
    temperature = float(meta.get("temperature", 1.0) or 1.0)
    model.train(backward)
    ctx = torch.enable_grad() if backward else torch.no_grad()
    with ctx:
        sp_group = getattr(model, "sp_group", None)
        owned = None
        with sft_profile.timed("fwd"):
            if sp_group is None:
                # rollout routing replay: the experts the sampler chose, per input token and MoE layer
                routed = batch.get("routed_experts") if packed.src_index is not None else None
                lp, ent = token_logprobs(model, packed, 1.0 / temperature, with_entropy=want_entropy,
                                         action_masks=action_masks_of(batch, packed),
                                         routed_experts=None if routed is None else to_device(routed, device))
            else:
                lp, ent, owned = _sp_logprobs(model, packed, sp_group, 1.0 / temperature, want_entropy, batch)
                # every rank of the sequence-parallel group holds the same batch and scores its own rows; the loss
                # factor dp_size counts data-parallel GROUPS, the gradient mean runs over all ranks
                import torch.distributed as dist
                meta["dp_size"] = int(meta.get("dp_size", 1) or 1) * dist.get_world_size(sp_group)
        outputs: Dict[str, Any] = {"logprobs": lp, "entropy": ent, "packed": packed}
        if owned is not None:
            outputs["owned"] = owned
        for name in processing.get("post") or []:
            outputs = resolve_fn(name, POST_PROCESSORS)(outputs, batch, meta, processing, device)
        loss = None
        metrics: Dict[str, Any] = {}
        if loss_name:
            loss_fn = resolve_fn(loss_name, LOSS_FNS)
            with sft_profile.timed("loss"):
                loss, metrics = loss_fn(outputs, batch, meta, processing.get("loss_kwargs") or {}, device)
        if backward:
            if loss is None:
                raise ValueError("backward needs a loss_fn")
            with sft_profile.timed("bwd"):
                engine.backward(loss)
    result: Dict[str, Any] = {"metrics": metrics,
                              "avg_loss": float(to_host(loss.detach())) if loss is not None else 0.0}
    metrics.setdefault("perf/packed_tokens", float(packed.total_tokens))
    metrics.setdefault("perf/dedup_redundancy", float(packed.redundancy))
    metrics["perf/pipeline_ms"] = (time.perf_counter() - t0) * 1e3
    if return_tensors:
        lp_out = lp.detach().float()
        ent_out = ent.detach().float() if ent is not None else None
        if owned is not None:                     # rows scored by the other ranks of the group are zero here: sum them in
            import torch.distributed as dist
            both = torch.stack([lp_out, ent_out if ent_out is not None else torch.zeros_like(lp_out)])
            dist.all_reduce(both, group=sp_group)
            lp_out, ent_out = both[0], (both[1] if ent_out is not None else None)
        out_batch = {"log_probs": to_host(packed.scatter_to_grid(lp_out))}
        if ent_out is not None:
            out_batch["entropy"] = to_host(packed.scatter_to_grid(ent_out))
        result["batch"] = out_batch
    return result
