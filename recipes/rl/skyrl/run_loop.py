"""Dataset-driven GRPO loop on the platform backend with the recipe environments -- what the SkyRL launchers run,
without needing the SkyRL checkout: prompts come from a parquet / jsonl file of verl- or SkyRL-format rows, every
prompt gets ``n`` rollouts, each rollout is scored by the row's environment, advantages are group-normalised and one
policy update is taken per batch.

    python -m recipes.rl.skyrl.run_loop --data train.parquet --env bird_sql_arctic --model Qwen/Qwen3-8B \\
        --training-gpus 8 --sampling-gpus 8 --batch-prompts 64 --n 16 --max-tokens 4096

A tokenizer directory (``--tokenizer``) is needed for real checkpoints; without one a byte-level codec is used,
which is enough for the tiny presets and the tests.  The reference drives the same loop through SkyRL's trainer
(recipes/rl/skyrl/*/arctic_rl/entrypoint.py and the ``run_qwen3_*_grpo_arl.sh`` launchers beside them)."""
from __future__ import annotations

import argparse
import json
from typing import Any, Dict, Iterator, List, Optional

import torch

from .arctic_backend import SkyRLArcticBackend
from .envs import make


def read_rows(path: str) -> List[Dict[str, Any]]:
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq
        return pq.read_table(path).to_pylist()
    with open(path, encoding="utf-8") as f:
        return [json.loads(ln) for ln in f if ln.strip()]


class ByteCodec:
    """Byte-level stand-in for a tokenizer: ids 3..258 are bytes (0-2 are reserved)."""

    def __init__(self, vocab_size: int):
        self.vocab_size = vocab_size

    def encode(self, text: str) -> List[int]:
        return [3 + b % max(1, min(256, self.vocab_size - 3)) for b in text.encode("utf-8")]

    def decode(self, ids: List[int]) -> str:
        return bytes(max(0, min(255, i - 3)) for i in ids).decode("utf-8", "replace")


def load_codec(tokenizer: Optional[str], vocab_size: int):
    if tokenizer:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(tokenizer)
    return ByteCodec(vocab_size)


def prompt_text(row: Dict[str, Any], codec) -> str:
    p = row.get("prompt")
    if isinstance(p, str):
        return p
    if hasattr(codec, "apply_chat_template"):
        return codec.apply_chat_template(p, tokenize=False, add_generation_prompt=True)
    return "\n".join(f"{m['role']}: {m['content']}" for m in p) + "\nassistant: "


def batches(rows: List[Dict[str, Any]], size: int, epochs: int, rank: int = 0, world: int = 1) -> Iterator[List[Dict[str, Any]]]:
    """``size`` prompts per rank and step: a global batch is ``size * world`` consecutive rows, rank ``r`` takes the
    ``r``-th block of it (every rank runs this loop under ``torchrun``)."""
    g = size * world
    for _ in range(epochs):
        for i in range(0, len(rows) - g + 1, g):
            yield rows[i + rank * size:i + (rank + 1) * size]


def grpo_advantages(rewards: torch.Tensor, n: int, eps: float = 1e-6) -> torch.Tensor:
    """Group-normalised advantages; a group whose rollouts all got the same reward contributes zeros."""
    g = rewards.view(-1, n)
    return ((g - g.mean(1, keepdim=True)) / (g.std(1, keepdim=True) + eps)).reshape(-1)


def run(args, backend: Optional[SkyRLArcticBackend] = None, log=print) -> List[Dict[str, float]]:
    from arctic_platform_b200.models.config import resolve_config
    rows = read_rows(args.data)
    vocab = resolve_config(args.model).vocab_size
    codec = load_codec(args.tokenizer, vocab)
    own = backend is None
    backend = backend or SkyRLArcticBackend(
        args.model, training_gpus=args.training_gpus, sampling_gpus=args.sampling_gpus, log_prob_gpus=args.log_prob_gpus,
        lr=args.lr, zero_stage=args.zero_stage, zorro=not args.no_zorro, max_model_len=args.max_prompt_tokens + args.max_tokens,
        kl_loss_coef=args.kl_loss_coef, sampler_tp=getattr(args, "sampler_tp", 1),
        sequence_parallel=getattr(args, "sequence_parallel", 1), offload_optimizer=getattr(args, "offload_optimizer", False))
    history = []
    try:
        backend.client.call("sync_weights")
        import os
        rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        for step, rows_b in enumerate(batches(rows, args.batch_prompts, args.epochs, rank, world)):
            if args.max_steps and step >= args.max_steps:
                break
            prompts = [codec.encode(prompt_text(r, codec))[-args.max_prompt_tokens:] for r in rows_b]
            outs = backend.generate(prompts, n=args.n, max_tokens=args.max_tokens, temperature=args.temperature)
            P, R, B = max(len(p) for p in prompts), args.max_tokens, len(outs)
            ids = torch.zeros((B, P + R), dtype=torch.int64)
            mask = torch.zeros_like(ids)
            rewards = torch.zeros(B)
            for i, o in enumerate(outs):
                p, t = prompts[o["prompt_index"]], o["token_ids"]
                ids[i, P - len(p):P] = torch.tensor(p)
                mask[i, P - len(p):P] = 1
                ids[i, P:P + len(t)] = torch.tensor(t)
                mask[i, P:P + len(t)] = 1
                rewards[i] = make(args.env, rows_b[o["prompt_index"]]).step(codec.decode(t)).reward
            adv = grpo_advantages(rewards, args.n).view(B, 1).expand(B, R).contiguous()
            m = backend.train_on_batch(ids, mask, R, adv, temperature=args.temperature)
            rec = {"step": step, "reward_mean": float(rewards.mean()), "reward_max": float(rewards.max()),
                   "loss": float(m["loss"]), "grad_norm": float(m["grad_norm"])}
            history.append(rec)
            if rank == 0:
                log(json.dumps(rec))
    finally:
        if own:
            backend.shutdown()
    return history


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="GRPO over a prompt dataset with the recipe environments")
    ap.add_argument("--data", required=True)
    ap.add_argument("--env", required=True)
    ap.add_argument("--model", default="qwen3-tiny")
    ap.add_argument("--tokenizer")
    ap.add_argument("--training-gpus", type=int, default=1)
    ap.add_argument("--sampling-gpus", type=int, default=1)
    ap.add_argument("--log-prob-gpus", type=int, default=1)
    ap.add_argument("--batch-prompts", type=int, default=4)
    ap.add_argument("--n", type=int, default=4)
    ap.add_argument("--max-prompt-tokens", type=int, default=2048)
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--lr", type=float, default=1e-6)
    ap.add_argument("--zero-stage", type=int, default=3)
    ap.add_argument("--kl-loss-coef", type=float, default=0.001)
    ap.add_argument("--no-zorro", action="store_true")
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--max-steps", type=int, default=0)
    ap.add_argument("--sampler-tp", type=int, default=1, help="tensor-parallel width of each sampler replica")
    ap.add_argument("--sequence-parallel", type=int, default=1, help="Ulysses degree of the trainer (long prompts)")
    ap.add_argument("--offload-optimizer", action="store_true", help="fp32 master weights and Adam moments in host memory")
    return ap


if __name__ == "__main__":
    run(build_parser().parse_args())
