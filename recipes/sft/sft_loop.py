"""Supervised fine-tuning loop on the SFT client: tokenised (prompt, answer) pairs -> ``fwd_bwd`` with labels masked
on the prompt -> ``step`` -> periodic checkpoint.  Synthetic copy task so it runs offline:

    python -m recipes.sft.sft_loop --model qwen3-tiny --steps 5 --batch 4 --ckpt /tmp/sft_ckpt

Counterpart of cortex-client/recipes/sft_loop.py in the reference."""
from __future__ import annotations

import argparse
import json

import torch

from arctic_platform_b200.sft import ArcticSFTClient, ArcticSFTClientConfig


def make_batch(batch: int, seq: int, vocab: int, gen: torch.Generator):
    half = seq // 2
    src = torch.randint(3, min(vocab, 200), (batch, half), generator=gen)
    ids = torch.cat([src, src], 1)                                  # the answer repeats the prompt
    labels = ids.clone()
    labels[:, :half] = -100                                         # loss only on the answer half
    return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": labels}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-tiny")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=32)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--ckpt", default="/tmp/apb200_sft_ckpt")
    ap.add_argument("--save-every", type=int, default=0)
    args = ap.parse_args()
    cfg = ArcticSFTClientConfig(comm_protocol="local", model_name=args.model, training_gpus=1, checkpoint_path=args.ckpt,
                                max_seq_len=args.seq,
                                ds_config={"optimizer": {"type": "AdamW", "params": {"lr": args.lr}},
                                           "gradient_clipping": 1.0})
    from arctic_platform_b200.models.config import resolve_config
    vocab = resolve_config(args.model).vocab_size
    gen = torch.Generator().manual_seed(0)
    with ArcticSFTClient(cfg) as client:
        for step in range(args.steps):
            out = client.fwd_bwd(make_batch(args.batch, args.seq, vocab, gen))
            st = client.step()
            print(json.dumps({"step": step, "loss": out["avg_loss"], "grad_norm": st["metrics"]["grad_norm"]}), flush=True)
            if args.save_every and (step + 1) % args.save_every == 0:
                client.save_checkpoint(step=step + 1)


if __name__ == "__main__":
    main()
