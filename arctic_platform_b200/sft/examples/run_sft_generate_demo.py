"""SFT with a sampler beside the trainer: fine-tune, hand the weights over, watch greedy generations change.

    python -m arctic_platform_b200.sft.examples.run_sft_generate_demo --steps 30

The synthetic task is "continue the arithmetic progression"; before training the model continues the prompts with
noise, after a few dozen steps most continuations follow the rule.  ``sampling_gpus=1`` + ``colocate`` puts trainer
and sampler on the same device; ``sync_weights`` is the hand-over.
Counterpart of arctic_platform/sft/examples/run_sft_generate_demo.py in the reference.
"""
from __future__ import annotations

import json
from typing import List, Optional

import torch

from .. import ArcticSFTClient
from . import sft_example
from ._common import batches


def rule_accuracy(prompts: List[List[int]], outs: List[dict], vocab: int) -> float:
    """Fraction of generated tokens that continue their prompt's progression."""
    hit = tot = 0
    for o in outs:
        p = prompts[o["prompt_index"]]
        stride, prev = p[-1] - p[-2], p[-1]
        for t in o["token_ids"]:
            want = (prev - 3 + stride) % (vocab - 3) + 3
            hit += int(t == want)
            tot += 1
            prev = t
    return hit / max(1, tot)


def main(argv: Optional[List[str]] = None, log=print) -> int:
    ap = sft_example.parser()
    ap.set_defaults(steps=30, batch_size=16)
    a = ap.parse_args(argv)
    cfg = sft_example.build_config(a).model_copy(update={"sampling_gpus": 1, "colocate": True,
                                                         "vllm_config": {"max_model_len": a.seq_len + 16}})
    g = torch.Generator().manual_seed(5)
    start = torch.randint(3, a.vocab // 2, (4,), generator=g)
    prompts = [[int(s) + k * 2 for k in range(6)] for s in start]         # stride 2
    sp = {"n": 1, "temperature": 0.0, "max_tokens": 6}
    with ArcticSFTClient(cfg) as c:
        c.sync_weights()
        before = rule_accuracy(prompts, c.generate(prompts, sp), a.vocab)
        data = batches(a.batch_size, a.seq_len, a.vocab, seed=2)
        for step in range(a.steps):
            loss = c.fwd_bwd(next(data))["avg_loss"]
            c.step()
            if step % 10 == 9:
                log(json.dumps({"step": step, "loss": loss}))
        c.sync_weights()
        after = rule_accuracy(prompts, c.generate(prompts, sp), a.vocab)
    log(json.dumps({"rule_accuracy_before": before, "rule_accuracy_after": after}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
