"""One training micro-batch (forward + backward) of a Qwen3 decoder on the packed, prompt-deduplicated layout.

    python benchmarks/bench_train_step.py [--model qwen3-4b] [--layers 4] [--prompt-len 2048] [--response-len 2048]
                                          [--rollouts 4] [--iters 3]

CUDA-event timing after warm-up; every iteration uses fresh random tokens (inputs far larger than L2 stream through).
For the per-kernel launch list of a training step, run a small case (``--layers 4 --iters 1``) plainly first and,
where the profiler is open on the box, again under
``ncu --metrics gpu__time_duration.sum --clock-control none -c 4000 --csv --log-file train_launches.csv``
(always with ``--clock-control none``: without it the profiler locks the GPU clocks, a setting that outlives the
process on a shared GPU)."""
import argparse
import dataclasses
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from arctic_platform_b200.models.config import PRESETS  # noqa: E402
from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs  # noqa: E402
from arctic_platform_b200.ops import _lib  # noqa: E402
from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-4b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--response-len", type=int, default=2048)
    ap.add_argument("--rollouts", type=int, default=4)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--no-dedup", action="store_true")
    args = ap.parse_args()
    cfg = PRESETS[args.model]
    if args.layers:
        cfg = dataclasses.replace(cfg, num_layers=args.layers)
    model = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=0)
    for p in model.parameters():
        p.grad_f32 = torch.zeros(p.shape, device="cuda", dtype=torch.float32)   # fp32 accumulation like the trainer
    g = torch.Generator().manual_seed(0)
    P, R, n = args.prompt_len, args.response_len, args.rollouts

    def batch():
        prompt = torch.randint(1, cfg.vocab_size, (1, P), generator=g).expand(n, P)
        ids = torch.cat([prompt, torch.randint(1, cfg.vocab_size, (n, R), generator=g)], 1)
        return build_packed_batch(ids, torch.ones_like(ids), R, dedup=not args.no_dedup).to("cuda")

    def step(pk):
        lp, _ = token_logprobs(model, pk, 1.0, with_entropy=False)
        (-lp.mean()).backward()

    for _ in range(2):
        step(batch())
    torch.cuda.synchronize()
    times, fwd_times = [], []
    for _ in range(args.iters):
        pk = batch()
        torch.cuda.synchronize()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        lp, _ = token_logprobs(model, pk, 1.0, with_entropy=False)
        loss = -lp.mean()
        e1.record()
        loss.backward()
        e2.record()
        torch.cuda.synchronize()
        fwd_times.append(e0.elapsed_time(e1))
        times.append(e0.elapsed_time(e2))
    _lib.check_status("bench_train_step")
    T = pk.total_tokens
    params = sum(p.numel() for n_, p in model.named_parameters() if "embed" not in n_)
    flops = 6.0 * params * T + 6.0 * cfg.vocab_size * cfg.hidden_size * pk.labels.numel()
    ms = min(times)
    print(json.dumps({"model": args.model, "layers": cfg.num_layers, "packed_tokens": T, "pred_tokens": int(pk.labels.numel()),
                      "ms_fwd_bwd": round(ms, 2), "ms_fwd": round(min(fwd_times), 2),
                      "gemm_tflops_equiv": round(flops / ms / 1e9, 1)}))


if __name__ == "__main__":
    main()
