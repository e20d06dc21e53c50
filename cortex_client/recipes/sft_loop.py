"""Supervised fine-tuning against the hosted service: create a training job, stream token batches to it, step, save.

    python -m cortex_client.recipes.sft_loop --url https://... --model Qwen/Qwen3-8B --data train.jsonl --steps 100

``--data`` is a jsonl file of ``{"input_ids": [...], "labels": [...]?}`` rows (labels default to the inputs; ``-100``
marks tokens without loss).  The loop is the local ``model(batch); optimizer.step()`` shape through
``NeutrinoTrainingEngine``.  Counterpart of cortex-client/recipes/sft_loop.py in the reference."""
from __future__ import annotations

import argparse
import json
from typing import Iterator, List, Optional

import torch

from ..dss_client import NeutrinoClient, NeutrinoTrainingEngine, SubJobConfig


def read_rows(path: str) -> List[dict]:
    with open(path, encoding="utf-8") as f:
        return [json.loads(ln) for ln in f if ln.strip()]


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
        lr: float = 1e-5, save_every: int = 0, job_id: Optional[str] = None, log=print) -> List[dict]:
    own = job_id is None
    if own:
        job_id = client.create_job([SubJobConfig.training_job(model, num_gpus=gpus, learning_rate=lr)])["job_id"]
        client.wait_for_job(job_id)
    engine = NeutrinoTrainingEngine(client, job_id, loss_fn="sft_ce")
    history = []
    try:
        for step, rows in enumerate(batches(read_rows(data), batch_size, steps)):
            loss = engine(collate(rows))
            m = engine.step()
            rec = {"step": step, "loss": loss, "grad_norm": m.get("grad_norm"), "lr": m.get("last_lr")}
            history.append(rec)
            log(json.dumps(rec))
            if save_every and (step + 1) % save_every == 0:
                engine.save()
    finally:
        if own:
            client.cancel_job(job_id)
    return history


def main(argv=None, client: Optional[NeutrinoClient] = None) -> int:
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
