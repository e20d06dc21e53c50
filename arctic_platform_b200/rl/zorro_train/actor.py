"""Stand-alone actor harness for ZoRRo Train: a model, a padded RL batch in, log-probs / a PPO step out.

``DeduplicatedActor`` is the smallest complete user of the prompt-deduplicated layout -- no server, no worker:
``forward(batch)`` returns per-token log-probs (and entropy) on the ``[B, R]`` response grid;
``compute_policy_loss_and_backward(batch)`` splits the batch into micro-batches along prompt groups, runs the
clipped PPO objective on the packed response tokens and accumulates gradients.  With ``dedup=False`` the same
class is the plain-packing baseline, which is what the gradient-equivalence tests compare against.

Counterpart of arctic_platform/rl/zorro_train/actor.py:42-252 (which drives a monkey-patched Hugging Face model;
here the layout object alone selects deduplication).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ...models.decoder import DecoderLM, token_logprobs
from ...models.factory import ModelSpec, Patches, build_model
from .layout import build_packed_batch, find_prompt_groups


def packed_ppo_policy_loss(log_prob: torch.Tensor, old_log_prob: torch.Tensor, advantages: torch.Tensor,
                           ref_log_prob: Optional[torch.Tensor] = None, clip_ratio: float = 0.2,
                           kl_loss_coef: float = 0.001) -> Tuple[torch.Tensor, Dict[str, float]]:
    """Clipped PPO surrogate with token-mean reduction over 1-D packed response tokens (+ optional k1 KL to a
    reference policy).  Returns the loss before gradient-accumulation scaling and scalar metrics."""
    log_ratio = log_prob - old_log_prob
    ratio = torch.exp(log_ratio)
    unclipped = -advantages * ratio
    clipped = -advantages * ratio.clamp(1.0 - clip_ratio, 1.0 + clip_ratio)
    pg_loss = torch.maximum(unclipped, clipped).mean()
    loss = pg_loss
    metrics: Dict[str, float] = {}
    if ref_log_prob is not None:
        kl = (log_prob - ref_log_prob).mean()
        loss = loss + kl_loss_coef * kl
        metrics["actor/kl_loss"] = float(kl.detach())
    with torch.no_grad():
        metrics.update({
            "actor/pg_loss": float(pg_loss), "actor/policy_loss": float(loss),
            "actor/pg_clipfrac": float(((ratio - 1.0).abs() > clip_ratio).float().mean()),
            "actor/ppo_kl": float(((ratio - 1.0) - log_ratio).mean()),
        })
    return loss, metrics


class DeduplicatedActor:
    def __init__(self, model_name_or_path: str = "qwen3-tiny", device: str = "cuda", dtype: torch.dtype = torch.bfloat16,
                 dedup: bool = True, max_token_len: int = 16384, model: Optional[DecoderLM] = None, seed: int = 0,
                 gradient_checkpointing: bool = False):
        self.device = torch.device(device)
        if model is None:
            name = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
            spec = ModelSpec(model_name_or_path, dtype=name, patches=Patches(gradient_checkpointing=False))
            model = build_model(spec, device=self.device, seed=seed).model
        self.model = model
        self.model.gradient_checkpointing = gradient_checkpointing
        self.dedup = dedup
        self.max_token_len = max_token_len
        self.last_stats: Dict[str, float] = {}

    def train(self):
        self.model.train()
        return self

    def eval(self):
        self.model.eval()
        return self

    # ------------------------------------------------------------------ batching
    def _micro_batches(self, batch: Dict[str, torch.Tensor], response_len: int) -> List[np.ndarray]:
        """Sample indices per micro-batch: whole prompt groups, greedily filled up to ``max_token_len`` packed tokens."""
        ids, mask = batch["input_ids"], batch["attention_mask"]
        groups = find_prompt_groups(ids, response_len) if self.dedup else np.arange(ids.shape[0])
        P = ids.shape[1] - response_len
        p_len = mask[:, :P].sum(1).cpu().numpy()
        r_len = mask[:, P:].sum(1).cpu().numpy()
        out, cur, cur_tok = [], [], 0
        for g in dict.fromkeys(groups.tolist()):
            members = np.nonzero(groups == g)[0]
            cost = int(p_len[members[0]] + r_len[members].sum()) if self.dedup else int((p_len + r_len)[members].sum())
            if cur and cur_tok + cost > self.max_token_len:
                out.append(np.concatenate(cur))
                cur, cur_tok = [], 0
            cur.append(members)
            cur_tok += cost
        if cur:
            out.append(np.concatenate(cur))
        return out

    def _packed(self, batch, idx, response_len):
        sel = torch.as_tensor(idx, dtype=torch.long)
        pk = build_packed_batch(batch["input_ids"][sel.to(batch["input_ids"].device)],
                                batch["attention_mask"][sel.to(batch["attention_mask"].device)], response_len,
                                dedup=self.dedup)
        return pk.to(self.device), sel

    # ------------------------------------------------------------------ API
    def forward(self, batch: Dict[str, torch.Tensor], response_len: int, temperature: float = 1.0,
                with_entropy: bool = True) -> Dict[str, torch.Tensor]:
        """No-grad scoring: ``{"log_probs": [B, R], "entropy": [B, R]}`` (zeros on padding)."""
        B = batch["input_ids"].shape[0]
        lp = torch.zeros((B, response_len), dtype=torch.float32, device=self.device)
        ent = torch.zeros_like(lp) if with_entropy else None
        tokens = full = 0
        with torch.no_grad():
            for idx in self._micro_batches(batch, response_len):
                pk, sel = self._packed(batch, idx, response_len)
                l, e = token_logprobs(self.model, pk, 1.0 / temperature, with_entropy)
                lp[sel.to(self.device)] = pk.scatter_to_grid(l)
                if with_entropy:
                    ent[sel.to(self.device)] = pk.scatter_to_grid(e)
                tokens += pk.total_tokens
                full += pk.full_tokens
        self.last_stats = {"packed_tokens": tokens, "full_tokens": full, "redundancy": 1.0 - tokens / max(1, full)}
        return {"log_probs": lp, "entropy": ent}

    def compute_policy_loss_and_backward(self, batch: Dict[str, torch.Tensor], response_len: int,
                                         temperature: float = 1.0, clip_ratio: float = 0.2,
                                         kl_loss_coef: float = 0.001) -> Dict[str, float]:
        """One gradient-accumulated PPO pass.  ``batch`` additionally holds ``old_log_probs``, ``advantages``
        (``[B, R]``) and optionally ``ref_log_prob``.  Every micro-batch is weighted by its share of the valid
        response tokens so that the accumulated gradient equals the token-mean loss over the whole batch."""
        mbs = self._micro_batches(batch, response_len)
        P = batch["input_ids"].shape[1] - response_len
        total_valid = float(batch["attention_mask"][:, P:].sum())
        agg: Dict[str, float] = {}
        loss_sum = 0.0
        for idx in mbs:
            pk, sel = self._packed(batch, idx, response_len)
            lp, _ = token_logprobs(self.model, pk, 1.0 / temperature, with_entropy=False)
            pick = lambda name: pk.gather_from_grid(batch[name][sel.to(batch[name].device)].to(self.device).float())
            old, adv = pick("old_log_probs"), pick("advantages")
            ref = pick("ref_log_prob") if "ref_log_prob" in batch else None
            loss, m = packed_ppo_policy_loss(lp, old, adv, ref, clip_ratio, kl_loss_coef)
            w = lp.numel() / max(1.0, total_valid)
            (loss * w).backward()
            loss_sum += float(loss.detach()) * w
            for k, v in m.items():
                agg[k] = agg.get(k, 0.0) + v * w
        agg["actor/loss"] = loss_sum
        agg["actor/num_micro_batches"] = float(len(mbs))
        return agg
