"""Asynchronous RL in miniature: a rollout thread and a trainer thread share one client.

    python -m arctic_platform_b200.rl.examples.local_server_example --updates 4

The rollout thread keeps generating groups with whatever weights the sampler holds and queues them, tagged with the
policy version it sampled from; the trainer thread takes groups off the queue, trains on them with the decoupled loss
(``loss_fn: grpo`` -- the sampler's log-probs are the behaviour policy, ``versions`` says how stale each token is),
steps, and every ``--sync-every`` updates hands the new weights to the sampler.  The hand-over and a generation never
overlap (one lock): a sampler must not read weights that are being replaced.
Counterpart of arctic_platform/rl/examples/local_server_example.py in the reference.
"""
from __future__ import annotations

import argparse
import json
import queue
import threading
from typing import List, Optional

import torch

from .. import ArcticRLClientConfig, create_arctic_rl_client
from ._common import grpo_batch, synthetic_prompts


def run(model: str = "qwen3-tiny", updates: int = 3, sync_every: int = 1, n: int = 4, max_tokens: int = 8,
        queue_depth: int = 2, training_gpus: int = 1, sampling_gpus: int = 1, log=print) -> List[dict]:
    client = create_arctic_rl_client(ArcticRLClientConfig(
        comm_protocol="local", model_name=model, training_gpus=training_gpus, sampling_gpus=sampling_gpus, log_prob_gpus=0,
        colocate=True, vllm_config={"max_model_len": 64 + max_tokens},
        ds_config={"gradient_clipping": 1.0, "optimizer": {"type": "AdamW", "params": {"lr": 1e-3}}}))
    rollouts: "queue.Queue" = queue.Queue(maxsize=queue_depth)
    stop = threading.Event()
    sampler_lock = threading.Lock()
    version = {"sampler": 0, "trainer": 0}
    errors: List[BaseException] = []
    history: List[dict] = []

    def rollout_worker():
        k = 0
        try:
            while not stop.is_set():
                prompts = synthetic_prompts(2, 10, 200, seed=k)
                with sampler_lock:
                    v = version["sampler"]
                    outs = client.call("generate", prompts, {"n": n, "temperature": 1.0, "max_tokens": max_tokens, "seed": k})
                item = (prompts, outs, v)
                while not stop.is_set():
                    try:
                        rollouts.put(item, timeout=0.2)
                        break
                    except queue.Full:
                        continue
                k += 1
        except BaseException as exc:                      # surfaced by the main thread
            errors.append(exc)
            stop.set()

    def trainer_worker():
        try:
            for u in range(updates):
                while True:
                    if stop.is_set():
                        return
                    try:
                        prompts, outs, v = rollouts.get(timeout=0.2)
                        break
                    except queue.Empty:
                        continue
                batch = grpo_batch(prompts, outs, n, max_tokens)
                reward = batch.pop("_reward_mean")
                R = batch["response_mask"].shape[1]
                batch["versions"] = torch.full((len(outs), R), v, dtype=torch.int64)
                meta = {"zorro_train_enable": True, "current_version": version["trainer"]}
                out = client.call("fwd_bwd", {"batch": batch, "meta": meta}, {"loss_fn": "grpo"})
                st = client.call("step")
                version["trainer"] += 1
                if (u + 1) % sync_every == 0:
                    with sampler_lock:
                        client.call("sync_weights")
                        version["sampler"] = version["trainer"]
                rec = {"update": u, "sampled_at_version": v, "staleness": version["trainer"] - 1 - v, "reward_mean": reward,
                       "loss": out["avg_loss"], "grad_norm": st["metrics"]["grad_norm"]}
                history.append(rec)
                log(json.dumps(rec))
        except BaseException as exc:
            errors.append(exc)
        finally:
            stop.set()

    try:
        client.call("sync_weights")
        threads = [threading.Thread(target=rollout_worker, name="rollout"), threading.Thread(target=trainer_worker, name="trainer")]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
        return history
    finally:
        stop.set()
        client.call("shutdown")


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--model", default="qwen3-tiny")
    ap.add_argument("--updates", type=int, default=3)
    ap.add_argument("--sync-every", type=int, default=1)
    ap.add_argument("--training-gpus", type=int, default=1)
    ap.add_argument("--sampling-gpus", type=int, default=1)
    a = ap.parse_args(argv)
    run(a.model, a.updates, a.sync_every, training_gpus=a.training_gpus, sampling_gpus=a.sampling_gpus)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
