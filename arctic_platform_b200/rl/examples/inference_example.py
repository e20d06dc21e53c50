"""Sampling only: a client that owns no trainer, against a job server that is already running (or in process).

    python -m arctic_platform_b200.rl.http_server --port 7000 &                      # on the GPU node
    python -m arctic_platform_b200.rl.examples.inference_example --host gpu-node --port 7000 --model /models/Qwen3-4B
    python -m arctic_platform_b200.rl.examples.inference_example                     # tiny model in this process

Shows per-request sampling parameters (``n``, temperature, top-k / top-p, stop tokens, seed), the fields of a result
record, scoring of given completions (``log_probs``) and a second client attaching to the same sampling job.
Counterpart of arctic_platform/rl/examples/inference_example.py in the reference.
"""
from __future__ import annotations

import argparse
import json
from typing import List, Optional

from .. import ArcticRLClientConfig, create_arctic_rl_client
from ._common import synthetic_prompts


def run(model: str = "qwen3-tiny", host: Optional[str] = None, port: Optional[int] = None, sampling_gpus: int = 1,
        log=print) -> dict:
    proto = "http" if host else "local"
    kw = {"host": host, "port": port or 7000} if host else {}
    cfg = ArcticRLClientConfig(comm_protocol=proto, model_name=model, training_gpus=0, sampling_gpus=sampling_gpus,
                               log_prob_gpus=0, vllm_config={"max_model_len": 96, "max_num_seqs": 16}, **kw)
    client = create_arctic_rl_client(cfg)
    try:
        prompts = synthetic_prompts(2, 10, 200)
        greedy = client.call("generate", prompts, {"n": 1, "temperature": 0.0, "max_tokens": 6})
        sampled = client.call("generate", prompts, {"n": 3, "temperature": 0.8, "top_k": 50, "top_p": 0.95, "max_tokens": 6,
                                                    "seed": 11})
        stop_tok = greedy[0]["token_ids"][2]
        stopped = client.call("generate", prompts[:1], {"n": 1, "temperature": 0.0, "max_tokens": 6, "stop_token_ids": [stop_tok]})
        log(json.dumps({"fields": sorted(greedy[0]), "greedy": [o["token_ids"] for o in greedy]}))
        log(json.dumps({"sampled_per_prompt": [sum(o["prompt_index"] == i for o in sampled) for i in range(len(prompts))],
                        "stopped_after": len(stopped[0]["token_ids"]), "finish_reason": stopped[0]["finish_reason"]}))
        scored = client.call("log_probs", prompts, [o["token_ids"] for o in greedy])
        again = create_arctic_rl_client(client.reconnect_config())            # attaches: no second sampling job
        same = again.call("generate", prompts, {"n": 1, "temperature": 0.0, "max_tokens": 6})
        return {"greedy": greedy, "sampled": sampled, "stopped": stopped, "scored": scored,
                "reattached_equal": [o["token_ids"] for o in same] == [o["token_ids"] for o in greedy]}
    finally:
        client.call("shutdown")


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--model", default="qwen3-tiny")
    ap.add_argument("--host")
    ap.add_argument("--port", type=int)
    ap.add_argument("--sampling-gpus", type=int, default=1)
    a = ap.parse_args(argv)
    run(a.model, a.host, a.port, a.sampling_gpus)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
