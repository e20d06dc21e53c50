"""Supervised fine-tuning against the hosted service: create a training job, stream token batches to it, step, save.

    python -m cortex_client.recipes.sft_loop --url https://... --model Qwen/Qwen3-8B --data train.jsonl --steps 100

    python -m cortex_client.recipes.sft_loop config=conn.json model_name=Qwen/Qwen3-8B data=chat.jsonl lora_rank=32 \
        n_gpus=8 batch_size=16 micro_batch_size=2 max_length=4096 log_path=/tmp/sft wandb_project=dss

``--data`` is a jsonl file of ``{"input_ids": [...], "labels": [...]?}`` rows (labels default to the inputs; ``-100``
marks tokens without loss) or of chat rows ``{"messages": [{"role", "content"}, ...]}``, which are rendered through the
model's chat template with the loss on the assistant turns (``tokenizer=`` names the tokenizer, default the model).
The loop is the local ``model(batch); optimizer.step()`` shape through ``NeutrinoTrainingEngine``; a batch larger than
``micro_batch_size * n_gpus`` is sent in slices that accumulate on the service before the step.  The second calling
form takes ``key=value`` settings (``SFTSettings``), writes ``config.json`` + ``metrics.jsonl`` under ``log_path`` and
mirrors metrics to Weights & Biases when ``wandb_project`` is set.  Counterpart of cortex-client/recipes/sft_loop.py
in the reference."""
from __future__ import annotations

import argparse
import dataclasses
import json
from typing import Any, Iterator, List, Optional

import torch

from ..dss_client import NeutrinoClient, NeutrinoTrainingEngine, SubJobConfig
from .common import MetricsLogger, apply_overrides, client_from_settings, render_chat


@dataclasses.dataclass
class SFTSettings:
    config: Optional[str] = None           # connection file
    url: Optional[str] = None
    model_name: str = "Qwen/Qwen3-8B"
    data: str = "train.jsonl"
    tokenizer: Optional[str] = None        # for chat rows; default: model_name
    steps: int = 100
    batch_size: int = 8
    micro_batch_size: int = 0              # rows per GPU and slice; 0 = the whole batch in one call
    n_gpus: int = 8
    learning_rate: float = 1e-5
    max_length: int = 4096
    lora_rank: int = 32                    # 0 = full fine-tuning
    model_provider: Optional[str] = None
    ep_size: int = 1
    save_every: int = 0
    log_path: Optional[str] = None
    wandb_project: Optional[str] = None
    wandb_name: Optional[str] = None
    job_id: Optional[str] = None

    def validate(self) -> None:
        if self.micro_batch_size and self.batch_size % (self.micro_batch_size * self.n_gpus):
            raise ValueError("batch_size must be a multiple of micro_batch_size * n_gpus")
        if self.ep_size > 1 and self.n_gpus % self.ep_size:
            raise ValueError("n_gpus must be a multiple of ep_size")

    def training_extra(self) -> dict:
        extra: dict = {}
        if self.lora_rank > 0:
            extra["lora_rank"] = self.lora_rank
        if self.model_provider:
            extra["model_provider"] = self.model_provider
        if self.ep_size > 1:
            extra["ep_size"] = self.ep_size
        return extra


def read_rows(path: str) -> List[dict]:
    with open(path, encoding="utf-8") as f:
        return [json.loads(ln) for ln in f if ln.strip()]


def tokenize_rows(rows: List[dict], tokenizer: Any, max_length: Optional[int] = None) -> List[dict]:
    """Chat rows (``messages``) -> ``input_ids`` + ``labels`` with the loss on the assistant turns; token rows are cut
    to ``max_length`` and otherwise pass through."""
    out = []
    for r in rows:
        if "messages" in r:
            ids, mask = render_chat(r["messages"], tokenizer, max_length)
            out.append({"input_ids": ids, "labels": [t if m else -100 for t, m in zip(ids, mask)]})
        else:
            n = max_length or len(r["input_ids"])
            out.append({**r, "input_ids": r["input_ids"][:n], **({"labels": r["labels"][:n]} if r.get("labels") else {})})
    return out


def slices(batch: dict, rows_per_call: int) -> List[dict]:
    n = batch["input_ids"].shape[0]
    if rows_per_call <= 0 or rows_per_call >= n:
        return [batch]
    return [{k: v[i:i + rows_per_call] for k, v in batch.items()} for i in range(0, n, rows_per_call)]


def collate(rows: List[dict], pad_id: int = 0) -> dict:
    """Right-padded ``input_ids`` / ``attention_mask`` / ``labels`` (``-100`` on padding)."""
    S = max(len(r["input_ids"]) for r in rows)
    ids = torch.full((len(rows), S), pad_id, dtype=torch.int64)
    mask = torch.zeros_like(ids)
    labels = torch.full_like(ids, -100)
    for i, r in enumerate(rows):
        n = len(r["input_ids"])
        ids[i, :n] = torch.tensor(r["input_ids"])
        mask[i, :n] = 1
        labels[i, :n] = torch.tensor(r.get("labels") or r["input_ids"])
    return {"input_ids": ids, "attention_mask": mask, "labels": labels}


def batches(rows: List[dict], size: int, steps: int) -> Iterator[List[dict]]:
    i = 0
    for _ in range(steps):
        yield [rows[(i + k) % len(rows)] for k in range(size)]
        i += size


def run(client: NeutrinoClient, model: str, data: str, steps: int = 10, batch_size: int = 8, gpus: int = 1,
        lr: float = 1e-5, save_every: int = 0, job_id: Optional[str] = None, log=print, micro_batch_size: int = 0,
        max_length: Optional[int] = None, tokenizer: Any = None, extra: Optional[dict] = None,
        max_seq_len: Optional[int] = None, logger: Optional[MetricsLogger] = None) -> List[dict]:
    own = job_id is None
    if own:
        kw = {"max_seq_len": max_seq_len} if max_seq_len else {}
        sub = SubJobConfig.training_job(model, num_gpus=gpus, learning_rate=lr, extra=dict(extra or {}), **kw)
        job_id = client.create_job([sub])["job_id"]
        client.wait_for_job(job_id)
    engine = NeutrinoTrainingEngine(client, job_id, loss_fn="sft_ce")
    rows_all = read_rows(data)
    if any("messages" in r for r in rows_all):
        if tokenizer is None:
            raise ValueError("chat rows need a tokenizer")
        if isinstance(tokenizer, str):
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(tokenizer)
    rows_all = tokenize_rows(rows_all, tokenizer, max_length)
    history = []
    try:
        for step, rows in enumerate(batches(rows_all, batch_size, steps)):
            parts = slices(collate(rows), micro_batch_size * gpus)
            tokens = [int((p["labels"] != -100).sum()) for p in parts]
            losses = [engine(p) for p in parts]                        # gradients accumulate on the service
            loss = sum(l * t for l, t in zip(losses, tokens)) / max(1, sum(tokens))
            m = engine.step()
            rec = {"step": step, "loss": loss, "train_mean_nll": loss, "loss_tokens": sum(tokens),
                   "grad_norm": m.get("grad_norm"), "lr": m.get("last_lr")}
            history.append(rec)
            if logger is not None:
                logger.log(step, {k: v for k, v in rec.items() if k != "step"})
            else:
                log(json.dumps(rec))
            if save_every and (step + 1) % save_every == 0:
                engine.save()
    finally:
        if own:
            client.cancel_job(job_id)
    return history


def run_settings(st: SFTSettings, client: Optional[NeutrinoClient] = None, echo=print) -> List[dict]:
    st.validate()
    client = client or client_from_settings(st.config, st.url)
    logger = MetricsLogger(st.log_path, dataclasses.asdict(st), st.wandb_project, st.wandb_name, echo=echo)
    try:
        return run(client, st.model_name, st.data, st.steps, st.batch_size, st.n_gpus, st.learning_rate, st.save_every,
                   st.job_id, micro_batch_size=st.micro_batch_size, max_length=st.max_length,
                   tokenizer=st.tokenizer or st.model_name, extra=st.training_extra(), max_seq_len=st.max_length,
                   logger=logger)
    finally:
        logger.close()


def main(argv=None, client: Optional[NeutrinoClient] = None) -> int:
    import sys
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and all("=" in a and not a.startswith("-") for a in argv):       # key=value settings
        run_settings(apply_overrides(SFTSettings(), argv), client)
        return 0
    ap = argparse.ArgumentParser(description="SFT loop against the hosted training service")
    ap.add_argument("--url")
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", required=True)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--lr", type=float, default=1e-5)
    ap.add_argument("--save-every", type=int, default=0)
    ap.add_argument("--job")
    args = ap.parse_args(argv)
    if client is None:
        from ..dss_client.dss_neutrino_cli import _client
        client = _client(args)
    run(client, args.model, args.data, args.steps, args.batch_size, args.gpus, args.lr, args.save_every, args.job)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
