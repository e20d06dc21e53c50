"""Fused compute + collective kernels against their NCCL (+ library GEMM) baselines, with roofline fractions.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_fused_collectives.py [--model qwen3-4b]

Every number is CUDA-event time on the launching stream, max over ranks, after warm-up; inputs rotate through a
pool larger than L2.  Roofline time of a case = max(FLOPs / measured GEMM peak, bytes that must cross NVLink per GPU
/ 770 GB/s measured peer-copy bandwidth); ``frac`` = roofline / achieved.  One JSON line per case on rank 0.

Cases: trainer step (reduce-scatter + clip + AdamW + all-gather), ZeRO-3 unit gather, trainer -> sampler weight
sync, tensor-parallel all-gather -> GEMM and GEMM -> reduce-scatter at decode shapes, expert-parallel MoE layer."""
import argparse
import dataclasses
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

NVLINK_GBS = 770.0


def timed(fn, iters=5, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for _ in range(iters):
        fn()
    en.record()
    torch.cuda.synchronize()
    t = torch.tensor([st.elapsed_time(en) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-4b")
    ap.add_argument("--layers", type=int, default=8, help="decoder blocks of the model used for the engine cases")
    ap.add_argument("--cases", default="step,tp,ep", help="comma list of case groups: step (trainer step, ZeRO-3 gather, "
                    "weight sync), tp (tensor-parallel GEMMs), ep (expert-parallel MoE layer)")
    ap.add_argument("--peak-tflops", type=float, default=1635.6,
                    help="bf16 GEMM peak of the machine (denominator of the compute side of the roofline)")
    args = ap.parse_args()
    cases = set(args.cases.split(","))
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.parallel import tensor_parallel as tp
    from arctic_platform_b200.parallel.weight_sync import flatten_like, sync_flat
    peak_tflops = args.peak_tflops
    cfg = dataclasses.replace(PRESETS[args.model], num_layers=args.layers)
    out = []

    def emit(case, ms, nvlink_bytes=0.0, flops=0.0, **extra):
        roof_ms = max(flops / (peak_tflops * 1e9), nvlink_bytes / (NVLINK_GBS * 1e6)) if (flops or nvlink_bytes) else 0.0
        rec = {"case": case, "world": world, "ms": round(ms, 4), "roofline_ms": round(roof_ms, 4),
               "frac_of_roofline": round(roof_ms / ms, 3) if ms > 0 and roof_ms > 0 else None,
               "nvlink_GBs_per_gpu": round(nvlink_bytes / ms / 1e6, 1) if nvlink_bytes else None, **extra}
        if rank == 0:
            print(json.dumps(rec), flush=True)
        out.append(rec)

    # ---- trainer step: fused vs collectives (stage 1: RS + AdamW + AG), and stage 3 (RS + local AdamW)
    step_cases = (("step_fused_zero1", 1, "fused"), ("step_nccl_zero1", 1, "collective"), ("step_fused_zero3", 3, "fused"))
    for name, stage, impl in (step_cases if "step" in cases else ()):
        model = DecoderLM(cfg, dev, torch.bfloat16).init_weights(seed=1)
        eng = TrainEngine(model, EngineConfig(lr=1e-6, max_grad_norm=1.0, impl=impl, zero_stage=stage))
        eng.grad_buf.tensor.normal_(0, 1e-3)
        n = eng.total
        # reduce-scatter reads (W-1)/W of the fp32 gradients of every peer shard; all-gather writes bf16 to W-1 peers
        rs = n * 4 * (world - 1) / world
        ag = n * 2 * (world - 1) / world if stage < 3 else 0.0
        ms = timed(lambda: (eng.grad_buf.tensor.add_(1e-6), eng.step()), iters=3, warmup=1)
        _lib.check_status(name)
        emit(name, ms, nvlink_bytes=rs + ag, params=n)
        if stage == 3 and world > 1:
            z = eng.zero3
            blocks = [ui for ui, b in enumerate(z.is_block) if b]
            bytes_unit = eng.units[blocks[0]].length * 2
            state = {"i": 0}

            def gather():
                ui = blocks[state["i"] % len(blocks)]
                state["i"] += 1
                z._gather(ui, z.slots[state["i"] % 2])
            emit("zero3_unit_gather", timed(gather, iters=8), nvlink_bytes=bytes_unit * (world - 1) / world,
                 unit_MB=round(bytes_unit / 1e6, 1), ctas=z.gather_ctas)
        # trainer -> sampler weight sync into a sampler-side flat buffer
        sampler_model = DecoderLM(cfg, dev, torch.bfloat16)
        dst = flatten_like(sampler_model, eng)
        ms = timed(lambda: sync_flat(eng, dst), iters=5)
        remote = n * 2 * (world - 1) / world if stage == 3 else 0.0
        emit(f"sync_weights_{name.split('_', 1)[1]}", ms, nvlink_bytes=remote, GBs_written=round(n * 2 / ms / 1e6, 1))
        del eng, model, sampler_model, dst
        torch.cuda.empty_cache()

    # ---- sampler tensor parallelism at decode shapes (128 sequences)
    if world > 1 and "tp" in cases:
        H, Q, I = PRESETS[args.model].hidden_size, PRESETS[args.model].q_size, PRESETS[args.model].intermediate_size
        ctx = tp.TPContext(dev, None, max_rows=128, max_cols=max(2 * I, Q))
        rows = 128 // world
        g = torch.Generator(device="cuda").manual_seed(3)
        for label, K, N in (("qkv", H, PRESETS[args.model].qkv_size // world), ("gate_up", H, 2 * I // world)):
            ws = [(torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16() for _ in range(max(2, int(300e6 // (N * K * 2)) + 1))]
            x = torch.randn(rows, K, device=dev, generator=g).bfloat16()
            it = {"i": 0}

            def fused():
                it["i"] += 1
                tp.ag_gemm(ctx, x, ws[it["i"] % len(ws)])

            def base():
                it["i"] += 1
                tp.ag_gemm_collective(x, ws[it["i"] % len(ws)])
            flops = 2.0 * 128 * N * K
            nv = (world - 1) * rows * K * 2
            emit(f"tp_ag_gemm_{label}_fused", timed(fused, iters=20), nvlink_bytes=nv, flops=flops, weight_MB=round(N * K * 2 / 1e6, 1))
            emit(f"tp_ag_gemm_{label}_nccl", timed(base, iters=20), nvlink_bytes=nv, flops=flops)
        for label, K, N in (("o_proj", Q // world, H), ("down", I // world, H)):
            ws = [(torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16() for _ in range(max(2, int(300e6 // (N * K * 2)) + 1))]
            x = torch.randn(128, K, device=dev, generator=g).bfloat16()
            it = {"i": 0}

            def fused():
                it["i"] += 1
                tp.gemm_rs(ctx, x, ws[it["i"] % len(ws)])

            def base():
                it["i"] += 1
                tp.gemm_rs_collective(x, ws[it["i"] % len(ws)])
            flops = 2.0 * 128 * N * K
            nv = (world - 1) / world * 128 * N * 4
            emit(f"tp_gemm_rs_{label}_fused", timed(fused, iters=20), nvlink_bytes=nv, flops=flops)
            emit(f"tp_gemm_rs_{label}_nccl", timed(base, iters=20), nvlink_bytes=nv, flops=flops)
        _lib.check_status("tp")

    if world > 1 and "ep" in cases:
        # ---- expert-parallel MoE layer (Qwen3-30B-A3B layer shape), 4096 tokens per rank
        from arctic_platform_b200.models.moe import MoEFeedForward
        from arctic_platform_b200.parallel.expert_parallel import ExpertParallel
        mcfg = PRESETS["qwen3-30b-a3b"]
        if mcfg.num_experts % world == 0:
            El = mcfg.num_experts // world
            T = 4096
            for impl in ("fused", "collective"):
                moe = MoEFeedForward(mcfg, dev, torch.bfloat16)
                with torch.no_grad():
                    moe.router.normal_(0, 0.02)
                    moe.wgu = torch.nn.Parameter(torch.randn(El, 2 * mcfg.moe_intermediate_size, mcfg.hidden_size, device=dev).mul_(0.02).bfloat16())
                    moe.wdown = torch.nn.Parameter(torch.randn(El, mcfg.hidden_size, mcfg.moe_intermediate_size, device=dev).mul_(0.02).bfloat16())
                moe.ep = ExpertParallel(mcfg.hidden_size, mcfg.num_experts, None, dev, max_recv_rows=T * mcfg.num_experts_per_tok * 2,
                                        max_pairs=T * mcfg.num_experts_per_tok, impl=impl)
                x = torch.randn(T, mcfg.hidden_size, device=dev).bfloat16()
                with torch.no_grad():
                    ms = timed(lambda: moe(x), iters=10)
                pairs = T * mcfg.num_experts_per_tok
                nv = 2 * pairs * mcfg.hidden_size * 2 * (world - 1) / world          # dispatch + combine
                flops = 2.0 * pairs * 3 * mcfg.hidden_size * mcfg.moe_intermediate_size
                emit(f"ep_moe_layer_infer_{impl}", ms, nvlink_bytes=nv, flops=flops, tokens=T)
                # training: forward + backward (data and weight gradients), dispatch and combine in both directions
                xg = x.clone().requires_grad_(True)
                gy = torch.randn_like(x)

                def train_pass():
                    moe.wgu.grad = moe.wdown.grad = moe.router.grad = None
                    moe(xg).backward(gy)
                ms = timed(train_pass, iters=5)
                emit(f"ep_moe_layer_train_{impl}", ms, nvlink_bytes=2 * nv, flops=3 * flops, tokens=T)
                del moe
                torch.cuda.empty_cache()
            _lib.check_status("ep")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
