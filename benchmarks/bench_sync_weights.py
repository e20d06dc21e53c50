"""sync_weights sweep: trainer ZeRO-3 bf16 shards -> sampler layout, one kernel against library twins.

For every model (Qwen3 dense 4B / 8B / 32B shapes), sampler tensor-parallel size and target dtype (bf16, or bf16 +
block-scaled fp8 matrices) the trainer side is a set of ZeRO-3 shard buffers in symmetric memory (random contents,
one per rank, every parameter cut into ``world`` pieces exactly as ``engine/zero3.py`` stores them) and the sampler
side is one tensor-parallel shard of the decoder on the same GPU (the colocated placement).  Timed, per
configuration, with CUDA events after warm-up, max over ranks:

  * ``fused``  -- ``sync_weights_table_kernel``: every 128 x 128 tile of the sampler's tensors is read once from the
    rank that owns it (plain loads over NVLink), written as bf16 and, for fp8, quantised in the same pass;
  * ``nccl``   -- the reference's shape of the job (arctic_platform/common/ray_server.py:1099-1165 gathers every
    ZeRO-3 parameter, then hands tensors over one by one): ``all_gather_into_tensor`` per parameter, a slice copy
    into the sampler's tensor, and a separate quantisation kernel for fp8;
  * ``peer_copy`` -- the CUDA-IPC shape (common/utils/weight_sync.py:47-142): one ``copy_`` per (parameter, owner rank)
    out of the peers' mapped buffers, then the slice copy / quantisation.

NVLink bytes = the part of the sampler's source bytes that lives on other ranks; GB/s and the fraction of the link
(``--link-gbs``, measured peer-copy bandwidth per direction) are reported for the fused kernel.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_sync_weights.py \\
        [--models 4b,8b,32b] [--tp 1,2,4,8] [--dtypes bf16,fp8] [--iters 3] [--layers 0] [--no-twins]
    python benchmarks/bench_sync_weights.py --models 4b            # one GPU: local copy + requantisation only

Prints one JSON line per configuration (rank 0).
"""
import argparse
import dataclasses
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from arctic_platform_b200.models.config import PRESETS, DecoderConfig  # noqa: E402
from arctic_platform_b200.models.decoder import DecoderLM  # noqa: E402
from arctic_platform_b200.ops import _lib  # noqa: E402
from arctic_platform_b200.parallel import weight_sync as ws  # noqa: E402
from arctic_platform_b200.parallel.symm import SymmetricBuffer  # noqa: E402
from arctic_platform_b200.parallel.tp_sampler import tp_config  # noqa: E402


def model_cfg(tag: str, layers: int) -> DecoderConfig:
    base = PRESETS["qwen3-4b"]
    shapes = {"4b": dict(num_layers=36, hidden_size=2560, num_heads=32, num_kv_heads=8, intermediate_size=9728),
              "8b": dict(num_layers=36, hidden_size=4096, num_heads=32, num_kv_heads=8, intermediate_size=12288,
                         tie_word_embeddings=False),
              "32b": dict(num_layers=64, hidden_size=5120, num_heads=64, num_kv_heads=8, intermediate_size=25600,
                          tie_word_embeddings=False)}[tag]
    shapes = {k: v for k, v in shapes.items() if hasattr(base, k)}
    cfg = dataclasses.replace(base, **shapes)
    return dataclasses.replace(cfg, num_layers=layers) if layers else cfg


def synthetic_layout(cfg: DecoderConfig, world: int):
    """Flat offsets and ZeRO-3 pieces of every parameter, laid out like the training engine does (embedding unit, one
    unit per block, final norm; parameters 8-element aligned, units padded to 8 x world), without building the model
    on the trainer side."""
    meta = DecoderLM(cfg, "meta", torch.bfloat16)
    units = [[("embed", meta.embed)] + ([("lm_head", meta.lm_head)] if meta.lm_head is not None else [])]
    for i, blk in enumerate(meta.blocks):
        units.append([(f"blocks.{i}.{n}", p) for n, p in blk.named_parameters()])
    units.append([("final_norm", meta.final_norm)])
    params, pieces = {}, {}
    off = shard = 0
    for unit in units:
        cur = off
        for name, p in unit:
            n = p.numel()
            if n % (8 * world):
                raise ValueError(f"{name}: {n} elements do not divide by 8 x {world}")
            params[name] = (cur, n, tuple(p.shape))
            pieces[name] = (n // world, shard)
            shard += n // world
            cur = (cur + n + 7) // 8 * 8
        off = (cur + 8 * world - 1) // (8 * world) * (8 * world)
    return {"total": off, "world": world, "dtype": "torch.bfloat16", "params": params, "zero3": pieces}, shard


def timed(fn, iters, world, dev):
    for _ in range(2):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for _ in range(iters):
        fn()
    en.record()
    torch.cuda.synchronize(dev)
    ms = st.elapsed_time(en) / iters
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--models", default="4b,8b,32b")
    ap.add_argument("--tp", default="1,2,4,8")
    ap.add_argument("--dtypes", default="bf16,fp8")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0, help="cut the models to this many layers (0 = full depth)")
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--no-twins", action="store_true")
    ap.add_argument("--max-gb", type=float, default=150.0, help="skip configurations that would hold more than this per GPU")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    for tag in args.models.split(","):
        cfg = model_cfg(tag, args.layers)
        layout, shard_len = synthetic_layout(cfg, world)
        need_gb = (shard_len * 2 + layout["total"] * 2 * 1.6) / 1e9
        if need_gb > args.max_gb:
            if rank == 0:
                print(json.dumps({"model": tag, "skipped": f"needs ~{need_gb:.0f} GB per GPU at {world} ranks"}), flush=True)
            continue
        shard = SymmetricBuffer(shard_len, torch.bfloat16, dev, None if world > 1 else False, zero=False)
        shard.tensor.normal_(0.0, 0.02)
        if world > 1:
            dist.barrier()
        src_ptrs = [int(p) for p in shard.peer_ptrs]
        for tp in [int(x) for x in args.tp.split(",")]:
            if tp > world and tp > 1:
                continue
            if cfg.num_kv_heads % tp or cfg.num_heads % tp:
                continue
            tp_rank = rank % tp
            local_cfg = tp_config(cfg, tp) if tp > 1 else cfg
            for dt in args.dtypes.split(","):
                fp8 = dt == "fp8"
                model = DecoderLM(local_cfg, dev, torch.bfloat16)
                plan = ws.build_sync_plan(layout, model, full_cfg=cfg, tp_rank=tp_rank, tp=tp, fp8=fp8)
                ms = timed(lambda: ws.run_sync_plan(plan, src_ptrs, rank), args.iters, world, dev)
                _lib.check_status("sync sweep")
                remote = plan.src_bytes * (world - 1) / world
                line = {"model": tag, "gpus": world, "sampler_tp": tp, "target": dt, "tensors": len(layout["params"]),
                        "table_records": plan.n_seg, "tiles": plan.total_tiles,
                        "src_gb_per_rank": round(plan.src_bytes / 1e9, 2), "dst_gb_per_rank": round(plan.dst_bytes / 1e9, 2),
                        "fused_ms": round(ms, 2), "fused_dst_gbs": round(plan.dst_bytes / ms / 1e6, 1),
                        "nvlink_gbs_per_gpu": round(remote / ms / 1e6, 1),
                        "frac_of_link": round(remote / ms / 1e6 / args.link_gbs, 3) if world > 1 else None}
                if not args.no_twins:
                    line.update(twins(layout, model, cfg, tp_rank, tp, fp8, shard, world, rank, dev, args.iters))
                if rank == 0:
                    print(json.dumps(line), flush=True)
                del plan, model
                torch.cuda.empty_cache()
        del shard
        torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()


def twins(layout, model, cfg, tp_rank, tp, fp8, shard, world, rank, dev, iters):
    """The same hand-over with library pieces: gather every parameter (NCCL all-gather, or one copy per owner out of
    the peers' mapped buffers), slice into the sampler's tensors, quantise separately."""
    params = ws._model_params(model)
    names = list(params)
    biggest = max(layout["params"][n][1] for n in names)
    full = torch.empty(biggest, dtype=torch.bfloat16, device=dev)

    def place(name, flat_full):
        _o, n, shape = layout["params"][name]
        src = flat_full[:n].view(shape)
        dst = params[name]
        for dst_row0, r0, c0, rows, cols in ws._tp_slices(name.split(".")[-1], shape, cfg, tp_rank, tp):
            if len(shape) == 1:
                dst.data.copy_(src)
            else:
                dst.data[dst_row0:dst_row0 + rows].copy_(src[r0:r0 + rows, c0:c0 + cols])
        if fp8 and name.split(".")[-1] in ws.FP8_MATRICES:
            ws.quantize_fp8_block128(dst.data)

    def nccl():
        for name in names:
            pl, so = layout["zero3"][name]
            mine = shard.tensor[so:so + pl]
            if world > 1:
                dist.all_gather_into_tensor(full[:pl * world], mine)
            else:
                full[:pl].copy_(mine)
            place(name, full)

    peers = None
    if world > 1 and shard._handle is not None:
        try:
            peers = [shard._handle.get_buffer(r, (shard.numel,), torch.bfloat16) for r in range(world)]
        except Exception:
            peers = None

    def peer_copy():
        for name in names:
            pl, so = layout["zero3"][name]
            for r in range(world):
                full[r * pl:(r + 1) * pl].copy_(peers[r][so:so + pl])
            place(name, full)

    out = {"nccl_twin_ms": round(timed(nccl, iters, world, dev), 2)}
    if peers is not None:
        out["peer_copy_twin_ms"] = round(timed(peer_copy, iters, world, dev), 2)
    return out


if __name__ == "__main__":
    main()
