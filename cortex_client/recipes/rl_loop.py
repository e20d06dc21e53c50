"""GRPO against the hosted service: one job with a training and a sampling sub-job; every step samples ``n`` rollouts
per prompt, scores them with a user reward function, takes one policy update and hands the new weights to the sampler.

    python -m cortex_client.recipes.rl_loop --url https://... --model Qwen/Qwen3-8B --prompts prompts.jsonl

    python -m cortex_client.recipes.rl_loop config=conn.json model_name=Qwen/Qwen3-8B prompts=math.jsonl lora_rank=32 \
        training_gpus=4 sampling_gpus=4 max_tokens=512 eval_prompts=math500.jsonl eval_every=10 log_path=/tmp/rl

``--prompts`` is a jsonl file of token rows ``{"prompt_ids": [...], "answer_ids": [...]}`` (reward 1 when the answer
tokens appear in the rollout) or of text rows ``{"prompt": "..." | "messages": [...], "answer": "..."}``, which are
rendered through the chat template and scored by the boxed-answer math reward on the decoded rollout -- replace
``reward_fn`` for other tasks.  With ``eval_prompts`` a held-out set is sampled greedily every ``eval_every`` steps and
its mean reward logged as ``eval/reward_mean``.  The second calling form takes ``key=value`` settings
(``RLSettings``) and writes ``config.json`` + ``metrics.jsonl`` under ``log_path``.
Counterpart of cortex-client/recipes/rl_loop.py in the reference."""
from __future__ import annotations

import argparse
import dataclasses
import json
from typing import Any, Callable, List, Optional, Sequence

import torch

from ..dss_client import NeutrinoClient, SubJobConfig
from .common import MetricsLogger, apply_overrides, client_from_settings, math_reward


@dataclasses.dataclass
class RLSettings:
    config: Optional[str] = None
    url: Optional[str] = None
    model_name: str = "Qwen/Qwen3-8B"
    prompts: str = "prompts.jsonl"
    eval_prompts: Optional[str] = None
    tokenizer: Optional[str] = None
    steps: int = 50
    prompts_per_step: int = 16
    group_size: int = 8
    max_tokens: int = 512
    max_seq_len: int = 2048
    training_gpus: int = 4
    sampling_gpus: int = 4
    learning_rate: float = 1e-6
    lora_rank: int = 0
    eval_every: int = 10
    log_path: Optional[str] = None
    wandb_project: Optional[str] = None
    wandb_name: Optional[str] = None
    job_id: Optional[str] = None


def read_rows(path: str) -> List[dict]:
    with open(path, encoding="utf-8") as f:
        return [json.loads(ln) for ln in f if ln.strip()]


def prepare_rows(rows: List[dict], tokenizer: Any = None) -> List[dict]:
    """Text rows get ``prompt_ids`` (chat template + generation prompt); token rows pass through."""
    out = []
    for r in rows:
        if "prompt_ids" in r:
            out.append(r)
            continue
        if tokenizer is None:
            raise ValueError("text prompts need a tokenizer")
        msgs = r.get("messages") or [{"role": "user", "content": r["prompt"]}]
        ids = tokenizer.apply_chat_template(msgs, tokenize=True, add_generation_prompt=True)
        out.append({**r, "prompt_ids": list(ids["input_ids"] if isinstance(ids, dict) else ids)})
    return out


def make_reward(tokenizer: Any = None) -> Callable[[Sequence[int], dict], float]:
    """Token rows: the answer tokens appear in the rollout.  Text rows: boxed answer of the decoded rollout."""
    def reward(rollout_ids: Sequence[int], row: dict) -> float:
        if "answer" in row and tokenizer is not None:
            return math_reward(tokenizer.decode(list(rollout_ids), skip_special_tokens=True), str(row["answer"]))
        return contains_answer(rollout_ids, row)
    return reward


def evaluate(client: NeutrinoClient, job_id: str, rows: List[dict], reward_fn, max_tokens: int) -> dict:
    """Greedy, one sample per held-out prompt."""
    prompts = [list(r["prompt_ids"]) for r in rows]
    outs = client.generate(job_id, prompts, {"n": 1, "max_tokens": max_tokens, "temperature": 0.0})["results"]
    scores = [reward_fn(o["token_ids"], rows[o["prompt_index"]]) for o in outs]
    return {"eval/reward_mean": sum(scores) / max(1, len(scores)), "eval/prompts": len(scores)}


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
        job_id: Optional[str] = None, log=print, sampling_gpus: Optional[int] = None, extra: Optional[dict] = None,
        max_seq_len: Optional[int] = None, eval_rows: Optional[List[dict]] = None, eval_every: int = 0,
        logger: Optional[MetricsLogger] = None) -> List[dict]:
    own = job_id is None
    if own:
        tkw = {"max_seq_len": max_seq_len} if max_seq_len else {}
        skw = {"max_model_len": max_seq_len} if max_seq_len else {}
        job = client.create_job([SubJobConfig.training_job(model, num_gpus=gpus, learning_rate=lr, extra=dict(extra or {}), **tkw),
                                 SubJobConfig.sampling_job(model, num_gpus=sampling_gpus or gpus, **skw)])
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
            solved = (rewards.view(-1, n) > 0).any(1).float().mean()
            rec = {"step": step, "reward_mean": float(rewards.mean()), "loss": out.get("avg_loss"),
                   "grad_norm": (st.get("metrics") or {}).get("grad_norm"), "prompts_solved": float(solved),
                   "response_tokens_mean": sum(len(o["token_ids"]) for o in outs) / max(1, len(outs))}
            if eval_rows and eval_every and (step + 1) % eval_every == 0:
                rec.update(evaluate(client, job_id, eval_rows, reward_fn, max_tokens))     # on the weights just synced
            history.append(rec)
            if logger is not None:
                logger.log(step, {k: v for k, v in rec.items() if k != "step"})
            else:
                log(json.dumps(rec))
    finally:
        if own:
            client.cancel_job(job_id)
    return history


def run_settings(st: RLSettings, client: Optional[NeutrinoClient] = None, tokenizer: Any = None, echo=print) -> List[dict]:
    client = client or client_from_settings(st.config, st.url)
    rows, eval_rows = read_rows(st.prompts), (read_rows(st.eval_prompts) if st.eval_prompts else None)
    needs_text = any("prompt_ids" not in r or "answer" in r for r in rows + (eval_rows or []))
    if tokenizer is None and needs_text:
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(st.tokenizer or st.model_name)
    rows = prepare_rows(rows, tokenizer)
    eval_rows = prepare_rows(eval_rows, tokenizer) if eval_rows else None
    too_long = [i for i, r in enumerate(rows) if len(r["prompt_ids"]) + st.max_tokens > st.max_seq_len]
    if too_long:
        raise ValueError(f"{len(too_long)} prompt(s) do not fit max_seq_len={st.max_seq_len} with max_tokens={st.max_tokens} "
                         f"(first: row {too_long[0]})")
    logger = MetricsLogger(st.log_path, dataclasses.asdict(st), st.wandb_project, st.wandb_name, echo=echo)
    try:
        return run(client, st.model_name, rows, st.steps, st.prompts_per_step, st.group_size, st.max_tokens,
                   st.training_gpus, st.learning_rate, make_reward(tokenizer), st.job_id,
                   sampling_gpus=st.sampling_gpus, extra={"lora_rank": st.lora_rank} if st.lora_rank > 0 else None,
                   max_seq_len=st.max_seq_len, eval_rows=eval_rows, eval_every=st.eval_every, logger=logger)
    finally:
        logger.close()


def main(argv=None, client: Optional[NeutrinoClient] = None) -> int:
    import sys
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and all("=" in a and not a.startswith("-") for a in argv):       # key=value settings
        run_settings(apply_overrides(RLSettings(), argv), client)
        return 0
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
