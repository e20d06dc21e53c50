"""Train -> sync -> sample: the cycle that keeps a sampler on the trainer's weights.

    python -m arctic_platform_b200.rl.examples.weight_sync_example                         # tiny model, CPU
    python -m arctic_platform_b200.rl.examples.weight_sync_example --model /models/Qwen3-4B \
        --training-gpus 1 --sampling-gpus 1 --colocate --steps 4

1. create the client (starts a training and a sampling job), 2. sample from the initial policy, 3. take a few GRPO
steps with a large learning rate so that the weights move, 4. hand the weights to the sampler, 5. sample again: greedy
continuations change, and ``weight_norm`` reports the same norm on both engines, 6. shut down.
Counterpart of arctic_platform/rl/examples/weight_sync_example.py in the reference.
"""
from __future__ import annotations

import argparse
import json
from typing import List, Optional

from .. import ArcticRLClientConfig, create_arctic_rl_client
from ._common import grpo_batch, synthetic_prompts


def run(model: str = "qwen3-tiny", training_gpus: int = 1, sampling_gpus: int = 1, colocate: bool = True, steps: int = 3,
        n: int = 4, max_tokens: int = 8, lr: float = 5e-3, comm_protocol: str = "local", host: Optional[str] = None,
        port: Optional[int] = None, log=print) -> dict:
    kw = {"host": host, "port": port} if comm_protocol != "local" else {}
    client = create_arctic_rl_client(ArcticRLClientConfig(
        comm_protocol=comm_protocol, model_name=model, training_gpus=training_gpus, sampling_gpus=sampling_gpus,
        log_prob_gpus=0, colocate=colocate, vllm_config={"max_model_len": 64 + max_tokens},
        ds_config={"gradient_clipping": 1.0, "optimizer": {"type": "AdamW", "params": {"lr": lr}}}, **kw))
    try:
        prompts = synthetic_prompts(4, 12, 200)
        greedy = {"n": 1, "temperature": 0.0, "max_tokens": max_tokens}
        client.call("sync_weights")
        before = [o["token_ids"] for o in client.call("generate", prompts, greedy)]
        norms0 = client.call("weight_norm")
        for step in range(steps):
            outs = client.call("generate", prompts, {"n": n, "temperature": 1.0, "max_tokens": max_tokens, "seed": step})
            batch = grpo_batch(prompts, outs, n, max_tokens)
            reward = batch.pop("_reward_mean")
            out = client.call("fwd_bwd", {"batch": batch, "meta": {"zorro_train_enable": True}}, {"loss_fn": "verl_grpo"})
            st = client.call("step")
            log(json.dumps({"step": step, "reward_mean": reward, "loss": out["avg_loss"], "grad_norm": st["metrics"]["grad_norm"]}))
            client.call("sync_weights")
        after = [o["token_ids"] for o in client.call("generate", prompts, greedy)]
        norms1 = client.call("weight_norm")
        result = {"changed_prompts": sum(a != b for a, b in zip(before, after)),
                  "training_norm_before": norms0["training_norm"], "training_norm_after": norms1["training_norm"],
                  "sampling_norm_after": norms1["sampling_norm"]}
        log(json.dumps(result))
        return result
    finally:
        client.call("shutdown")


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--model", default="qwen3-tiny")
    ap.add_argument("--training-gpus", type=int, default=1)
    ap.add_argument("--sampling-gpus", type=int, default=1)
    ap.add_argument("--colocate", action="store_true")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--lr", type=float, default=5e-3)
    ap.add_argument("--comm-protocol", default="local", choices=["local", "http", "ray"])
    ap.add_argument("--host")
    ap.add_argument("--port", type=int)
    a = ap.parse_args(argv)
    run(a.model, a.training_gpus, a.sampling_gpus, a.colocate, a.steps, lr=a.lr, comm_protocol=a.comm_protocol,
        host=a.host, port=a.port)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
