"""Times the tcgen05 segment attention forward/backward against flash-attn 2 (the reference's
default attention, arctic_platform/integrations/verl/adapter.py:442-444) on packed causal sequences
and on a ZoRRo group layout.  CUDA events, 3 warm-up + N timed launches; q/k/v rotate through a pool
larger than L2.

    python benchmarks/bench_attention.py [--seqlen 4096] [--batch 8] [--iters 10]
"""
import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from arctic_platform_b200.ops import _lib  # noqa: E402
from arctic_platform_b200.ops.attention import AttnLayout, attention_bwd_cuda, attention_fwd_cuda  # noqa: E402


def timeit(fn, nv, iters, warmup=3):
    for i in range(warmup):
        fn(i % nv)
    torch.cuda.synchronize()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for i in range(iters):
        fn(i % nv)
    en.record()
    torch.cuda.synchronize()
    return st.elapsed_time(en) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqlen", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    Hq, Hkv, D = 32, 8, 128
    S, B = args.seqlen, args.batch
    T = S * B
    scale = D ** -0.5
    layout = AttnLayout.from_cu_seqlens(np.arange(B + 1) * S)
    nv = 3
    qs = [torch.randn(T, Hq, D, device="cuda").bfloat16() for _ in range(nv)]
    ks = [torch.randn(T, Hkv, D, device="cuda").bfloat16() for _ in range(nv)]
    vs = [torch.randn(T, Hkv, D, device="cuda").bfloat16() for _ in range(nv)]
    dos = [torch.randn(T, Hq, D, device="cuda").bfloat16() for _ in range(nv)]
    flops_fwd = 4.0 * B * Hq * D * S * S / 2
    res = {}
    t = timeit(lambda i: attention_fwd_cuda(qs[i], ks[i], vs[i], layout, scale), nv, args.iters)
    res["ours_fwd_ms"], res["ours_fwd_tflops"] = round(t, 3), round(flops_fwd / t / 1e9, 1)
    outs = [attention_fwd_cuda(qs[i], ks[i], vs[i], layout, scale) for i in range(nv)]
    t = timeit(lambda i: attention_bwd_cuda(qs[i], ks[i], vs[i], outs[i][0], dos[i], outs[i][1], layout, scale),
               nv, args.iters)
    res["ours_bwd_ms"], res["ours_bwd_tflops"] = round(t, 3), round(2.5 * flops_fwd / t / 1e9, 1)
    _lib.check_status("attention bench")
    try:
        from flash_attn import flash_attn_varlen_func
        cu = torch.arange(B + 1, device="cuda", dtype=torch.int32) * S
        t = timeit(lambda i: flash_attn_varlen_func(qs[i], ks[i], vs[i], cu, cu, S, S, causal=True), nv, args.iters)
        res["fa2_fwd_ms"], res["fa2_fwd_tflops"] = round(t, 3), round(flops_fwd / t / 1e9, 1)
        qg = [x.clone().requires_grad_() for x in qs]
        kg = [x.clone().requires_grad_() for x in ks]
        vg = [x.clone().requires_grad_() for x in vs]
        og = [flash_attn_varlen_func(qg[i], kg[i], vg[i], cu, cu, S, S, causal=True) for i in range(nv)]
        t = timeit(lambda i: torch.autograd.grad(og[i], (qg[i], kg[i], vg[i]), dos[i], retain_graph=True), nv,
                   args.iters)
        res["fa2_bwd_ms"], res["fa2_bwd_tflops"] = round(t, 3), round(2.5 * flops_fwd / t / 1e9, 1)
    except Exception as exc:  # flash-attn missing or unsupported
        res["fa2"] = f"unavailable: {type(exc).__name__}: {exc}"[:200]
    print(json.dumps({"case": "packed_causal", "B": B, "S": S, "Hq": Hq, "Hkv": Hkv, "D": D, **res}), flush=True)


if __name__ == "__main__":
    main()
