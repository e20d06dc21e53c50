"""Training-FLOPs and wall-time estimator for dense, MoE and gated (partially active) models.

    python -m arctic_platform_b200.cli.flops_estimator --params 10 --tokens 1e12 --moe-experts 128 --moe-topk 8 \
        --ffn-fraction 0.9 --gpu-tflops 1400 --num-gpus 64 --mfu 0.45 --json

``total = per_token_factor * active_params * tokens`` with ``active = params * ((1 - ffn_fraction) + ffn_fraction *
topk / experts)`` (or ``--active-fraction`` directly).  Counterpart of scripts/gated_deltanet_estimator.py in the
reference."""
from __future__ import annotations

import argparse
import json
from typing import Optional

_SUFFIX = [(1e24, "Y"), (1e21, "Z"), (1e18, "E"), (1e15, "P"), (1e12, "T"), (1e9, "G"), (1e6, "M"), (1e3, "k")]


def human(x: float) -> str:
    for scale, s in _SUFFIX:
        if abs(x) >= scale:
            return f"{x / scale:.3g}{s}"
    return f"{x:.3g}"


def active_fraction(ffn_fraction: Optional[float], experts: Optional[int], topk: Optional[int],
                    explicit: Optional[float]) -> float:
    if explicit is not None:
        if not 0 < explicit <= 1:
            raise ValueError("--active-fraction must be in (0, 1]")
        return explicit
    if experts and topk:
        if topk > experts:
            raise ValueError("--moe-topk cannot exceed --moe-experts")
        f = 0.67 if ffn_fraction is None else ffn_fraction
        return (1 - f) + f * topk / experts
    return 1.0


def estimate(params_b: float, tokens: float, per_token_factor: float = 6.0, act: float = 1.0,
             gpu_tflops: Optional[float] = None, num_gpus: int = 1, mfu: float = 1.0) -> dict:
    active = params_b * 1e9 * act
    total = per_token_factor * active * tokens
    out = {"active_params": active, "flops_per_token": per_token_factor * active, "total_flops": total}
    if gpu_tflops:
        sec = total / (gpu_tflops * 1e12 * num_gpus * mfu)
        out.update({"seconds": sec, "gpu_hours": sec * num_gpus / 3600, "days": sec / 86400})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=float, default=10.0, help="model size in billions")
    ap.add_argument("--tokens", type=float, default=1e12)
    ap.add_argument("--per-token-factor", type=float, default=6.0)
    ap.add_argument("--active-fraction", type=float)
    ap.add_argument("--ffn-fraction", type=float)
    ap.add_argument("--moe-experts", type=int)
    ap.add_argument("--moe-topk", type=int)
    ap.add_argument("--gpu-tflops", type=float)
    ap.add_argument("--num-gpus", type=int, default=1)
    ap.add_argument("--mfu", type=float, default=1.0)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    act = active_fraction(a.ffn_fraction, a.moe_experts, a.moe_topk, a.active_fraction)
    res = estimate(a.params, a.tokens, a.per_token_factor, act, a.gpu_tflops, a.num_gpus, a.mfu)
    if a.json:
        print(json.dumps({"active_fraction": act, **res}))
    else:
        print(f"active fraction {act:.3f}  active params {human(res['active_params'])}  "
              f"FLOPs/token {human(res['flops_per_token'])}  total {human(res['total_flops'])}FLOP")
        if "seconds" in res:
            print(f"{a.num_gpus} GPUs x {a.gpu_tflops} TFLOP/s at MFU {a.mfu}: {res['days']:.2f} days, {human(res['gpu_hours'])} GPU-hours")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
