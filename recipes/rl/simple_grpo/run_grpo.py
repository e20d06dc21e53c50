"""Minimal GRPO loop on the platform client: generate -> reward -> advantages -> reference / old log-probs ->
forward_backward -> step -> sync_weights.  No dataset download: the task is synthetic arithmetic ("a+b=" with the
answer scored by the GSM8K reward), tokenised with a byte-level toy tokenizer, so the recipe runs offline and on
any preset model (random init).  With a real checkpoint directory and tokenizer the same loop is a GSM8K run.

    python -m recipes.rl.simple_grpo.run_grpo --model qwen3-tiny --steps 3 --prompts 4 --samples 4 --device cpu

Counterpart of recipes/rl/skyrl/simple_gsm8k and recipes/rl/verl/simple in the reference (which launch verl /
SkyRL with the platform as remote backend).
"""
from __future__ import annotations

import argparse
import json
import random
from typing import List

import torch

from arctic_platform_b200.rl import ArcticRLClientConfig, create_arctic_rl_client
from recipes.rl.rewards import gsm8k_reward


def encode(text: str, vocab: int) -> List[int]:
    return [3 + (b % (vocab - 3)) for b in text.encode()]


def decode(ids: List[int]) -> str:
    return bytes((i - 3) % 256 for i in ids).decode("latin-1")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-tiny")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--prompts", type=int, default=4)
    ap.add_argument("--samples", type=int, default=4)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--lr", type=float, default=1e-5)
    ap.add_argument("--zorro", action="store_true", default=True)
    args = ap.parse_args()
    cfg = ArcticRLClientConfig(comm_protocol="local", model_name=args.model, training_gpus=1, sampling_gpus=1,
                               log_prob_gpus=1, colocate=True,
                               ds_config={"zero_optimization": {"stage": 2}, "gradient_clipping": 1.0,
                                          "optimizer": {"type": "AdamW", "params": {"lr": args.lr}}},
                               vllm_config={"max_model_len": 64 + args.max_tokens})
    client = create_arctic_rl_client(cfg)
    from arctic_platform_b200.models.config import resolve_config
    vocab = resolve_config(args.model).vocab_size
    rng = random.Random(0)
    for step in range(args.steps):
        tasks = [(rng.randint(1, 99), rng.randint(1, 99)) for _ in range(args.prompts)]
        prompts = [encode(f"What is {a}+{b}? Finish with '#### <answer>'.\n", vocab) for a, b in tasks]
        P = max(len(p) for p in prompts)
        client.call("sync_weights")
        outs = client.call("generate", prompts, {"n": args.samples, "temperature": 1.0, "max_tokens": args.max_tokens})
        R = args.max_tokens
        B = len(outs)
        ids = torch.zeros((B, P + R), dtype=torch.int64)
        mask = torch.zeros_like(ids)
        rewards = torch.zeros(B)
        for i, o in enumerate(outs):
            p = prompts[o["prompt_index"]]
            t = o["token_ids"]
            ids[i, P - len(p):P] = torch.tensor(p)
            mask[i, P - len(p):P] = 1
            ids[i, P:P + len(t)] = torch.tensor(t)
            mask[i, P:P + len(t)] = 1
            a, b = tasks[o["prompt_index"]]
            rewards[i] = gsm8k_reward(decode(t), f"#### {a + b}", method="flexible", format_score=0.1)
        grp = rewards.view(args.prompts, args.samples)
        adv = ((grp - grp.mean(1, keepdim=True)) / (grp.std(1, keepdim=True) + 1e-6)).reshape(B, 1).expand(B, R)
        batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, P:].contiguous(),
                 "advantages": adv.contiguous()}
        meta = {"zorro_train_enable": bool(args.zorro), "temperature": 1.0}
        batch["old_log_probs"] = client.call("fwd_no_grad", {"batch": batch, "meta": meta})["batch"]["log_probs"]
        batch["ref_log_prob"] = client.call("fwd_no_grad", {"batch": batch, "meta": meta}, reference_model=True)["batch"]["log_probs"]
        out = client.call("fwd_bwd", {"batch": batch, "meta": meta}, {"loss_fn": "verl_grpo"})
        st = client.call("step")
        print(json.dumps({"step": step, "reward_mean": float(rewards.mean()), "loss": out["avg_loss"],
                          "grad_norm": st["metrics"]["grad_norm"], "lr": st["metrics"]["last_lr"]}), flush=True)
    client.call("shutdown")


if __name__ == "__main__":
    main()
