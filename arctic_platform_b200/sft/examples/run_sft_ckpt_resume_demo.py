"""Checkpoint and resume: train, save, start a NEW job from the checkpoint, and continue exactly where it stopped.

    python -m arctic_platform_b200.sft.examples.run_sft_ckpt_resume_demo --steps 6

Phase 1 trains ``--steps`` steps and saves.  Phase 2 starts a fresh client on the same ``checkpoint_path``, loads the
checkpoint (weights, optimizer state, step counter, learning rate) and trains ``--steps`` more.  A third run trains
``2 x steps`` without interruption on the same data; the demo checks that the resumed losses equal the uninterrupted
ones.  Counterpart of arctic_platform/sft/examples/run_sft_ckpt_resume_demo.py in the reference.
"""
from __future__ import annotations

import json
import tempfile
from typing import List, Optional

from .. import ArcticSFTClient
from . import sft_example
from ._common import batches


def _train(client, data, steps: int) -> List[float]:
    out = []
    for _ in range(steps):
        out.append(float(client.fwd_bwd(next(data))["avg_loss"]))
        client.step()
    return out


def main(argv: Optional[List[str]] = None, log=print) -> int:
    ap = sft_example.parser()
    ap.set_defaults(steps=4)
    a = ap.parse_args(argv)
    a.checkpoint_path = a.checkpoint_path or tempfile.mkdtemp(prefix="sft-resume-")
    data = batches(a.batch_size, a.seq_len, a.vocab, seed=1)
    with ArcticSFTClient(sft_example.build_config(a)) as c:
        first = _train(c, data, a.steps)
        saved = c.save_checkpoint(step=a.steps)
    log(json.dumps({"phase": 1, "losses": first, "saved": saved["path"]}))
    with ArcticSFTClient(sft_example.build_config(a)) as c:
        loaded = c.load_checkpoint()                                   # follows <checkpoint_path>/latest
        second = _train(c, data, a.steps)
    log(json.dumps({"phase": 2, "resumed_at": loaded["global_steps"], "losses": second}))
    a.checkpoint_path = tempfile.mkdtemp(prefix="sft-straight-")
    data = batches(a.batch_size, a.seq_len, a.vocab, seed=1)
    with ArcticSFTClient(sft_example.build_config(a)) as c:
        straight = _train(c, data, 2 * a.steps)
    worst = max(abs(x - y) for x, y in zip(first + second, straight))
    log(json.dumps({"phase": 3, "uninterrupted": straight, "max_abs_difference": worst}))
    return 0 if loaded["global_steps"] == a.steps and worst < 1e-4 else 1


if __name__ == "__main__":
    raise SystemExit(main())
