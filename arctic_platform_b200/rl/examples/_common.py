"""Pieces the examples share: synthetic prompts, a toy reward, the padded GRPO batch."""
from __future__ import annotations

from typing import List, Sequence

import torch


def synthetic_prompts(n: int, length: int, vocab: int, seed: int = 0) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, vocab, (length,), generator=g).tolist() for _ in range(n)]


def toy_reward(token_ids: Sequence[int]) -> float:
    """More even tokens = more reward: enough signal for a few optimizer steps to move the policy visibly."""
    return sum(1.0 for t in token_ids if t % 2 == 0) / max(1, len(token_ids))


def grpo_batch(prompts: List[List[int]], outs: List[dict], n: int, max_tokens: int) -> dict:
    """Prompts left-padded to ``P``, responses right-padded to ``R``, group-normalised advantages, sampler log-probs
    as the old policy."""
    P, R, B = max(len(p) for p in prompts), max_tokens, len(outs)
    ids = torch.zeros((B, P + R), dtype=torch.int64)
    mask = torch.zeros_like(ids)
    old = torch.zeros((B, R))
    for i, o in enumerate(outs):
        p, t = prompts[o["prompt_index"]], o["token_ids"][:R]
        ids[i, P - len(p):P] = torch.tensor(p)
        mask[i, P - len(p):P] = 1
        ids[i, P:P + len(t)] = torch.tensor(t)
        mask[i, P:P + len(t)] = 1
        old[i, :len(t)] = torch.tensor(o["logprobs"][:R])
    r = torch.tensor([toy_reward(o["token_ids"]) for o in outs]).view(-1, n)
    adv = ((r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True) + 1e-6)).reshape(B, 1).expand(B, R).contiguous()
    return {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, P:].contiguous(), "advantages": adv,
            "old_log_probs": old, "_reward_mean": float(r.mean())}
