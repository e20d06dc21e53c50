"""The table of the one-kernel weight sync (gather + tensor-parallel reshard + fp8 block scales), checked on the host:
an interpreter of the table records reproduces, for every tensor-parallel rank, the shard that the name-based
hand-over builds from full Hugging Face tensors -- from a replicated trainer buffer and from ZeRO-3 pieces."""
import ctypes
import dataclasses

import pytest
import torch

from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM
from arctic_platform_b200.models.hf_io import iter_hf_tensors, load_hf_tensor
from arctic_platform_b200.parallel import weight_sync as ws
from arctic_platform_b200.parallel.tp_sampler import tp_config, tp_slice


def _interpret(plan, sources, src_rank=0):
    """What ``sync_weights_table_kernel`` does, tile by tile in PyTorch: returns (bf16 flat, q bytes as float, scales)."""
    n = plan.n_seg
    raw = bytes(plan.segs.cpu().numpy().tobytes())
    segs = (ws._SyncSeg * n).from_buffer_copy(raw)
    flat = torch.zeros_like(plan.dst_flat)
    deq = {}
    tiles = 0
    for sg in segs:
        assert sg.tile_start == tiles
        tiles += ((sg.rows + 127) // 128) * sg.tiles_c
        rows = torch.arange(sg.rows)[:, None] + sg.row0
        cols = torch.arange(sg.cols)[None, :] + sg.col0
        e = rows * sg.src_ld + cols
        if sg.piece_len > 0:
            owner = e // sg.piece_len
            vals = torch.zeros(e.shape, dtype=sources[0].dtype)
            for r, buf in enumerate(sources):
                m = owner == r
                vals[m] = buf[(sg.shard_off + e - owner * sg.piece_len)[m]]
        else:
            vals = sources[src_rank][sg.src_elem + e]
        if sg.dst_elem >= 0:
            idx = sg.dst_elem + torch.arange(sg.rows)[:, None] * sg.dst_ld + torch.arange(sg.cols)[None, :]
            flat[idx] = vals.to(flat.dtype)
        if sg.fp8:
            deq[(sg.q_off, sg.scale_off)] = (vals.float(), sg.q_ld, sg.scale_ld)
    assert tiles == plan.total_tiles
    return flat, deq


def _full_model(seed=3):
    cfg = dataclasses.replace(PRESETS["qwen3-tiny"], num_layers=2)
    return cfg, DecoderLM(cfg, "cpu", torch.bfloat16).init_weights(seed=seed)


@pytest.mark.parametrize("tp", [1, 2])
def test_table_reproduces_the_tensor_parallel_shards(tp):
    cfg, full = _full_model()
    want_full = {n: t.clone() for n, t in iter_hf_tensors(full)}
    eng = TrainEngine(full, EngineConfig(zero_stage=1))
    layout = ws.trainer_layout(eng)
    assert layout["zero3"] is None and layout["params"]["embed"][2] == (cfg.vocab_size, cfg.hidden_size)
    for rank in range(tp):
        local = tp_config(cfg, tp) if tp > 1 else cfg
        shard = DecoderLM(local, "cpu", torch.bfloat16)
        plan = ws.build_sync_plan(layout, shard, full_cfg=cfg, tp_rank=rank, tp=tp)
        flat, _ = _interpret(plan, [eng.param_buf.tensor])
        plan.dst_flat.copy_(flat)
        ref = DecoderLM(local, "cpu", torch.bfloat16)
        for name, t in want_full.items():
            load_hf_tensor(ref, name, tp_slice(name, t, cfg, rank, tp))
        for (n1, a), (n2, b) in zip(shard.named_parameters(), ref.named_parameters()):
            assert n1 == n2 and torch.equal(a, b), n1
        assert plan.src_bytes == sum(p.numel() for p in shard.parameters()) * 2


def test_table_reads_zero3_pieces_from_their_owners():
    """Every parameter cut into ``world`` flat pieces (the stage-3 storage): the table names, per vector, the rank
    that owns it and the offset inside that rank's shard buffer."""
    cfg, full = _full_model(seed=5)
    eng = TrainEngine(full, EngineConfig(zero_stage=1))
    W = 2
    # lay the parameters out as stage 3 would on two ranks, without spawning them
    shard_bufs = [[], []]
    pieces, off = {}, 0
    for name, (o, n, shape) in eng.param_slices.items():
        assert n % (8 * W) == 0
        pl = n // W
        src = eng.param_buf.tensor[o:o + n]
        for r in range(W):
            shard_bufs[r].append(src[r * pl:(r + 1) * pl])
        pieces[name] = (pl, off)
        off += pl
    sources = [torch.cat(b) for b in shard_bufs]
    layout = ws.trainer_layout(eng)
    layout["zero3"], layout["world"] = pieces, W
    for rank in range(2):
        shard = DecoderLM(tp_config(cfg, 2), "cpu", torch.bfloat16)
        plan = ws.build_sync_plan(layout, shard, full_cfg=cfg, tp_rank=rank, tp=2)
        flat, _ = _interpret(plan, sources)
        plan.dst_flat.copy_(flat)
        for name, t in iter_hf_tensors(full):
            pass
        ref = DecoderLM(tp_config(cfg, 2), "cpu", torch.bfloat16)
        for name, t in iter_hf_tensors(full):
            load_hf_tensor(ref, name, tp_slice(name, t, cfg, rank, 2))
        for (n1, a), (_n2, b) in zip(shard.named_parameters(), ref.named_parameters()):
            assert torch.equal(a, b), n1


def test_fp8_segments_address_the_blocks_of_the_local_matrix():
    cfg = dataclasses.replace(PRESETS["qwen3-tiny-d128"], num_layers=1)
    full = DecoderLM(cfg, "cpu", torch.bfloat16).init_weights(seed=9)
    eng = TrainEngine(full, EngineConfig(zero_stage=1))
    layout = ws.trainer_layout(eng)
    shard = DecoderLM(tp_config(cfg, 2), "cpu", torch.bfloat16)
    plan = ws.build_sync_plan(layout, shard, full_cfg=cfg, tp_rank=1, tp=2, fp8=True)
    assert set(n for (_l, n) in plan.fp8) == set(ws.FP8_MATRICES)
    _flat, deq = _interpret(plan, [eng.param_buf.tensor])
    # every fp8 segment starts on a 128-row block of its local matrix, and the scale slots of one matrix do not collide
    seen = set()
    for (q_off, s_off), (vals, q_ld, s_ld) in deq.items():
        nb = ((vals.shape[0] + 127) // 128, (vals.shape[1] + 127) // 128)
        for rb in range(nb[0]):
            for cb in range(nb[1]):
                slot = s_off + rb * s_ld + cb
                assert slot not in seen
                seen.add(slot)
    assert len(seen) == plan.scale_buf.numel()
    q, sc = plan.fp8[(0, "wqkv")]
    assert q.shape == shard.blocks[0].wqkv.shape and sc.shape == ((q.shape[0] + 127) // 128, (q.shape[1] + 127) // 128)


def test_moe_models_use_the_name_based_path():
    cfg = PRESETS["qwen3-moe-tiny"] if "qwen3-moe-tiny" in PRESETS else None
    if cfg is None:
        pytest.skip("no MoE preset")
    m = DecoderLM(cfg, "cpu", torch.bfloat16)
    eng = TrainEngine(DecoderLM(cfg, "cpu", torch.bfloat16).init_weights(seed=1), EngineConfig(zero_stage=1))
    with pytest.raises(NotImplementedError):
        ws.build_sync_plan(ws.trainer_layout(eng), m)
