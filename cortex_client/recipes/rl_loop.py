"""GRPO against the hosted service: one job with a training and a sampling sub-job; every step samples ``n`` rollouts
per prompt, scores them with a user reward function, takes one policy update and hands the new weights to the sampler.

    python -m cortex_client.recipes.rl_loop --url https://... --model Qwen/Qwen3-8B --prompts prompts.jsonl

``--prompts`` is a jsonl file of ``{"prompt_ids": [...], "answer": ...}`` rows; the default reward is 1 when the decoded
answer tokens (``answer_ids``) appear in the rollout, else 0 -- replace ``reward_fn`` for real tasks.
Counterpart of cortex-client/recipes/rl_loop.py in the reference."""
from __future__ import annotations

import argparse
import json
from typing import Callable, List, Optional, Sequence

import torch

from ..dss_client import NeutrinoClient, SubJobConfig


def contains_answer(rollout_ids: Sequence[int], row: dict) -> float:
    ans = list(row.get("answer_ids") or [])
    if not ans:
        return 0.0
    r = list(rollout_ids)
    return float(any(r[i:i + len(ans)] == ans for i in range(len(r) - len(ans) + 1)))


def build_batch(prompts: List[List[int]], outs: List[dict], max_tokens: int, rewards: torch.Tensor, n: int) -> dict:
    """verl-shaped padded batch: prompts left-padded, responses right-padded, group-normalised advantages."""
    P, R, B = max(len(p) for p in prompts), max_tokens, len(outs)
    ids = torch.zeros((B, P + R), dtype=torch.int64)
    mask = torch.zeros_like(ids)
    for i, o in enumerate(outs):
        p, t = prompts[o["prompt_index"]], o["token_ids"][:R]
        ids[i, P - len(p):P] = torch.tensor(p)
        mask[i, P - len(p):P] = 1
        ids[i, P:P + len(t)] = torch.tensor(t)
        mask[i, P:P + len(t)] = 1
    g = rewards.view(-1, n)
    adv = ((g - g.mean(1, keepdim=True)) / (g.std(1, keepdim=True) + 1e-6)).reshape(B, 1).expand(B, R).contiguous()
    return {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, P:].contiguous(), "advantages": adv}


def run(client: NeutrinoClient, model: str, rows: List[dict], steps: int = 3, prompts_per_step: int = 4, n: int = 4,
        max_tokens: int = 64, gpus: int = 1, lr: float = 1e-6, reward_fn: Callable[[Sequence[int], dict], float] = contains_answer,
        job_id: Optional[str] = None, log=print) -> List[dict]:
    own = job_id is None
    if own:
        job = client.create_job([SubJobConfig.training_job(model, num_gpus=gpus, learning_rate=lr),
                                 SubJobConfig.sampling_job(model, num_gpus=gpus)])
        job_id = job["job_id"]
        client.wait_for_job(job_id)
    history = []
    try:
        client.weight_sync(job_id)
        for step in range(steps):
            chunk = [rows[(step * prompts_per_step + k) % len(rows)] for k in range(prompts_per_step)]
            prompts = [list(r["prompt_ids"]) for r in chunk]
            outs = client.generate(job_id, prompts, {"n": n, "max_tokens": max_tokens, "temperature": 1.0})["results"]
            rewards = torch.tensor([reward_fn(o["token_ids"], chunk[o["prompt_index"]]) for o in outs])
            batch = build_batch(prompts, outs, max_tokens, rewards, n)
            meta = {"zorro_train_enable": True, "response_length": max_tokens}
            old = client.forward(job_id, batch, meta)
            batch["old_log_probs"] = old["batch"]["log_probs"]
            out = client.forward_backward(job_id, batch, meta, {"loss_fn": "verl_grpo"})
            st = client.step(job_id)
            client.weight_sync(job_id)
            rec = {"step": step, "reward_mean": float(rewards.mean()), "loss": out.get("avg_loss"),
                   "grad_norm": (st.get("metrics") or {}).get("grad_norm")}
            history.append(rec)
            log(json.dumps(rec))
    finally:
        if own:
            client.cancel_job(job_id)
    return history


def main(argv=None, client: Optional[NeutrinoClient] = None) -> int:
    ap = argparse.ArgumentParser(description="GRPO loop against the hosted training service")
    ap.add_argument("--url")
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompts", required=True)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--prompts-per-step", type=int, default=4)
    ap.add_argument("--n", type=int, default=4)
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--lr", type=float, default=1e-6)
    ap.add_argument("--job")
    args = ap.parse_args(argv)
    if client is None:
        from ..dss_client.dss_neutrino_cli import _client
        client = _client(args)
    with open(args.prompts, encoding="utf-8") as f:
        rows = [json.loads(ln) for ln in f if ln.strip()]
    run(client, args.model, rows, args.steps, args.prompts_per_step, args.n, args.max_tokens, args.gpus, args.lr,
        job_id=args.job)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
