"""The SFT loop in one file, over any transport.

    python -m arctic_platform_b200.sft.examples.sft_example --steps 20                            # in process, CPU
    python -m arctic_platform_b200.sft.examples.sft_example --comm-protocol http --launch-local-server \
        --model /models/Qwen3-4B --training-gpus 8 --server-cuda-visible-devices 0,1,2,3,4,5,6,7

``fwd_bwd`` (loss ``sft_ce``: every loss token of the global batch weighs the same) -> ``step`` -> periodic
``save_checkpoint``; with ``--accumulate k`` each step sends ``k`` micro-batches that accumulate on the engine.
Counterpart of arctic_platform/sft/examples/sft_example.py in the reference.
"""
from __future__ import annotations

import argparse
import json
import tempfile
from typing import List, Optional

from .. import ArcticSFTClient, ArcticSFTClientConfig
from ._common import batches


def build_config(a) -> ArcticSFTClientConfig:
    kw = {"host": a.host, "port": a.port} if a.comm_protocol != "local" else {}
    return ArcticSFTClientConfig(
        model_name=a.model, training_gpus=a.training_gpus, comm_protocol=a.comm_protocol, max_seq_len=a.seq_len,
        checkpoint_path=a.checkpoint_path or tempfile.mkdtemp(prefix="sft-example-"),
        launch_local_server=a.launch_local_server, server_cuda_visible_devices=a.server_cuda_visible_devices,
        ds_config={"zero_optimization": {"stage": a.zero_stage}, "gradient_clipping": 1.0,
                   "optimizer": {"type": "AdamW", "params": {"lr": a.lr, "weight_decay": 0.0}}}, **kw)


def run(a, log=print) -> List[dict]:
    history = []
    with ArcticSFTClient(build_config(a)) as client:
        data = batches(a.batch_size, a.seq_len, a.vocab)
        for step in range(a.steps):
            mbs = [next(data) for _ in range(a.accumulate)]
            out = client.fwd_bwd(mbs if a.accumulate > 1 else mbs[0])
            st = client.step()
            rec = {"step": step, "loss": out["avg_loss"], "grad_norm": st["metrics"]["grad_norm"], "lr": st["metrics"]["last_lr"]}
            history.append(rec)
            log(json.dumps(rec))
            if a.save_every and (step + 1) % a.save_every == 0:
                saved = client.save_checkpoint(step=step + 1)
                log(json.dumps({"saved": saved["path"]}))
    return history


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--model", default="qwen3-tiny")
    ap.add_argument("--vocab", type=int, default=200, help="synthetic token range (must not exceed the model's vocabulary)")
    ap.add_argument("--training-gpus", type=int, default=1)
    ap.add_argument("--comm-protocol", default="local", choices=["local", "http", "ray"])
    ap.add_argument("--host", default="localhost")
    ap.add_argument("--port", type=int, default=8765)
    ap.add_argument("--launch-local-server", action="store_true")
    ap.add_argument("--server-cuda-visible-devices")
    ap.add_argument("--checkpoint-path")
    ap.add_argument("--zero-stage", type=int, default=0)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=24)
    ap.add_argument("--accumulate", type=int, default=1)
    ap.add_argument("--lr", type=float, default=3e-3)
    ap.add_argument("--save-every", type=int, default=0)
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    run(parser().parse_args(argv))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
