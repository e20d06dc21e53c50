"""Rollout (decode) throughput of the sampler engine on Qwen3-4B shapes with synthetic prompts.

    python benchmarks/bench_decode.py [--layers 36] [--prompts 8] [--samples 16] [--prompt-len 2048]
                                      [--max-tokens 256] [--no-graph] [--no-cascade]

Tensor-parallel replica (one engine over all ranks of the job; every rank feeds the same prompts):

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 benchmarks/bench_decode.py \
        --model qwen3-8b
    APB_TP_DECODE=nccl python -m torch.distributed.run ... benchmarks/bench_decode.py --model qwen3-8b   # library twin

The twin runs the row-parallel projections as a local GEMM + NCCL all-reduce + residual/norm kernel on every rank;
the default is the fused pair (GEMM whose epilogue adds into the owner rank's accumulator, norm kernel that stores the
normalised rows into every rank's activation buffer).

Prints one JSON line (rank 0): decode ms/step (CUDA events over the whole generate call, max over ranks; prefill is
not separated, use a long --max-tokens so decode dominates), tokens/s, kernel launches.
"""
import argparse
import dataclasses
import json
import os
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from arctic_platform_b200.engine.sampler import SamplerEngine  # noqa: E402
from arctic_platform_b200.models.config import PRESETS  # noqa: E402
from arctic_platform_b200.models.decoder import DecoderLM  # noqa: E402
from arctic_platform_b200.ops import _lib  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-4b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--samples", type=int, default=16)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cascade", action="store_true")
    ap.add_argument("--repeat", type=int, default=2)
    args = ap.parse_args()
    cfg = PRESETS[args.model]
    if args.layers:
        cfg = dataclasses.replace(cfg, num_layers=args.layers)
    B = args.prompts * args.samples
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    group = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        group = dist.group.WORLD
    model = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=0)
    eng = SamplerEngine(cfg, "cuda", model=model, tp_group=group,
                        kv_cache_tokens=args.prompts * (args.prompt_len + 64) + B * (args.max_tokens + 64) + 4096,
                        max_batch=max(8, B), max_seq_len=args.prompt_len + args.max_tokens + 16,
                        cascade=not args.no_cascade, use_cuda_graph=not args.no_graph)
    g = torch.Generator().manual_seed(0)
    res = {}
    for it in range(args.repeat):
        prompts = [torch.randint(1, cfg.vocab_size, (args.prompt_len,), generator=g).tolist() for _ in range(args.prompts)]
        torch.cuda.synchronize()
        l0 = _lib.launch_count()
        st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.record()
        out = eng.generate(prompts, {"n": args.samples, "temperature": 1.0, "max_tokens": args.max_tokens, "ignore_eos": True})
        en.record()
        torch.cuda.synchronize()
        ms = st.elapsed_time(en)
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        toks = sum(len(o["token_ids"]) for o in out)
        res = {"ms_total": round(ms, 1), "ms_per_decode_step": round(ms / args.max_tokens, 3),
               "tokens_per_s": round(toks / ms * 1e3, 1), "launches": _lib.launch_count() - l0}
    _lib.check_status("bench_decode")
    if rank == 0:
        print(json.dumps({"model": args.model, "layers": cfg.num_layers, "batch": B, "prompt_len": args.prompt_len,
                          "max_tokens": args.max_tokens, "graph": not args.no_graph, "cascade": not args.no_cascade,
                          "tensor_parallel": world, "tp_step": os.environ.get("APB_TP_DECODE", "fused") if world > 1 else None,
                          **res}), flush=True)
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        if os.environ.get("APB_TP_DECODE", "fused") == "nccl":
            # NCCL collectives captured in CUDA graphs keep the communicator busy at teardown: leave without it
            sys.stdout.flush()
            os._exit(0)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
