"""Stand-alone harness for the prompt-de-duplicated training path: synthetic GRPO batches, a gradient-equivalence
check against the plain (every rollout carries its own prompt copy) computation, and a timing loop.

    python -m arctic_platform_b200.rl.zorro_train.harness --model qwen3-tiny --prompts 4 --rollouts 8

prints the largest log-prob / gradient differences between the two paths and their step times.  On a GPU the timing
uses CUDA events on the current stream; on CPU, wall-clock.  Counterpart of the reference's in-tree scripts
(arctic_platform/rl/zorro_train/tests.py:46-749, demo.py, test_perf.py:122-564)."""
from __future__ import annotations

import argparse
import json
import time
from typing import Callable, Dict, Optional, Tuple

import torch

from ...models.config import resolve_config
from ...models.decoder import DecoderLM, token_logprobs
from .layout import build_packed_batch


def create_dummy_batch(num_prompts: int = 4, rollouts: int = 8, prompt_len: Tuple[int, int] = (16, 64),
                       response_len: Tuple[int, int] = (4, 32), vocab_size: int = 32000, seed: int = 0,
                       shuffle: bool = True) -> Dict[str, torch.Tensor]:
    """A GRPO batch in the verl padding convention: prompts LEFT-padded to the longest prompt, responses RIGHT-padded
    to the longest response, ``rollouts`` samples per prompt (not necessarily adjacent when ``shuffle``)."""
    g = torch.Generator().manual_seed(seed)
    P, R, B = prompt_len[1], response_len[1], num_prompts * rollouts
    ids = torch.zeros((B, P + R), dtype=torch.int64)
    mask = torch.zeros_like(ids)
    for p in range(num_prompts):
        pl = int(torch.randint(prompt_len[0], P + 1, (1,), generator=g))
        prompt = torch.randint(3, vocab_size, (pl,), generator=g)
        for s in range(rollouts):
            b = p * rollouts + s
            rl = int(torch.randint(response_len[0], R + 1, (1,), generator=g))
            ids[b, P - pl:P], mask[b, P - pl:P] = prompt, 1
            ids[b, P:P + rl], mask[b, P:P + rl] = torch.randint(3, vocab_size, (rl,), generator=g), 1
    if shuffle:
        perm = torch.randperm(B, generator=g)
        ids, mask = ids[perm], mask[perm]
    adv = torch.randn(B, 1, generator=g).expand(B, R).contiguous()
    return {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, P:].contiguous(), "advantages": adv,
            "response_length": R}


def policy_step(model: DecoderLM, batch: Dict[str, torch.Tensor], dedup: bool, temperature: float = 1.0):
    """Forward + backward of an advantage-weighted log-likelihood; returns ``(log_probs [B, R], packed batch)``."""
    R = int(batch["response_length"])
    dev = next(model.parameters()).device
    pk = build_packed_batch(batch["input_ids"], batch["attention_mask"], R, dedup=dedup).to(dev)
    lp, _ = token_logprobs(model, pk, 1.0 / temperature, with_entropy=False)
    adv = pk.gather_from_grid(batch["advantages"].to(dev)).float()
    (-(lp * adv).sum() / max(1, lp.numel())).backward()
    return pk.scatter_to_grid(lp.detach().float()), pk


def compare_gradients(a: Dict[str, torch.Tensor], b: Dict[str, torch.Tensor]) -> Dict[str, float]:
    """Largest absolute difference, largest difference relative to the tensor's scale, and the smallest cosine
    similarity over all parameters."""
    worst_abs = worst_rel = 0.0
    worst_cos, worst_name = 1.0, ""
    for name, ga in a.items():
        gb = b[name].float()
        ga = ga.float()
        d = float((ga - gb).abs().max())
        scale = float(gb.abs().max()) + 1e-12
        cos = float(torch.nn.functional.cosine_similarity(ga.flatten(), gb.flatten(), dim=0)) if gb.abs().sum() > 0 else 1.0
        if d / scale > worst_rel:
            worst_rel, worst_name = d / scale, name
        worst_abs, worst_cos = max(worst_abs, d), min(worst_cos, cos)
    return {"max_abs": worst_abs, "max_rel": worst_rel, "min_cosine": worst_cos, "worst_param": worst_name}


def _grads(model: DecoderLM) -> Dict[str, torch.Tensor]:
    out = {}
    for n, p in model.named_parameters():
        g = getattr(p, "grad_f32", None)
        g = g if g is not None else p.grad
        if g is not None:
            out[n] = g.detach().clone()
    return out


def gradient_correctness(model: DecoderLM, batch: Dict[str, torch.Tensor]) -> Dict[str, float]:
    """Runs the same step with and without de-duplication and reports how far log-probs and gradients are apart."""
    res = {}
    for dedup in (False, True):
        model.zero_grad(set_to_none=True)
        lp, pk = policy_step(model, batch, dedup)
        res[dedup] = (lp, _grads(model), pk)
    m = batch["response_mask"].bool()
    out = compare_gradients(res[True][1], res[False][1])
    out["max_logprob_diff"] = float((res[True][0].cpu() - res[False][0].cpu())[m].abs().max())
    out["tokens_plain"], out["tokens_dedup"] = res[False][2].total_tokens, res[True][2].total_tokens
    return out


def timed(fn: Callable[[], None], warmup: int = 1, iters: int = 3, device: Optional[torch.device] = None) -> float:
    """Mean milliseconds per call: CUDA events on the current stream on a GPU, wall-clock otherwise."""
    for _ in range(warmup):
        fn()
    if device is not None and device.type == "cuda":
        torch.cuda.synchronize(device)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            fn()
        end.record()
        torch.cuda.synchronize(device)
        return start.elapsed_time(end) / iters
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t0) * 1e3 / iters


def benchmark_performance(model: DecoderLM, batch: Dict[str, torch.Tensor], warmup: int = 1, iters: int = 3) -> Dict[str, float]:
    dev = next(model.parameters()).device
    out = {}
    for dedup in (False, True):
        def step(d=dedup):
            model.zero_grad(set_to_none=True)
            policy_step(model, batch, d)
        out["dedup_ms" if dedup else "plain_ms"] = timed(step, warmup, iters, dev)
    out["speedup"] = out["plain_ms"] / max(out["dedup_ms"], 1e-9)
    return out


def main(argv=None) -> Dict[str, float]:
    ap = argparse.ArgumentParser(description="de-duplicated vs plain training step: equivalence and timing")
    ap.add_argument("--model", default="qwen3-tiny")
    ap.add_argument("--prompts", type=int, default=4)
    ap.add_argument("--rollouts", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=64)
    ap.add_argument("--response-len", type=int, default=32)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    cfg = resolve_config(args.model)
    dev = torch.device(args.device)
    model = DecoderLM(cfg, dev, torch.bfloat16 if dev.type == "cuda" else torch.float32).init_weights(seed=0)
    batch = create_dummy_batch(args.prompts, args.rollouts, (max(4, args.prompt_len // 2), args.prompt_len),
                               (max(2, args.response_len // 4), args.response_len), cfg.vocab_size)
    report = {**gradient_correctness(model, batch), **benchmark_performance(model, batch, iters=args.iters)}
    print(json.dumps(report, indent=2))
    return report


if __name__ == "__main__":
    main()
