"""One-kernel weight hand-over on a GPU: tensor-parallel reshard and block-scaled fp8 requantisation in the same pass,
from a replicated trainer buffer and from ZeRO-3 pieces (two shard buffers on one GPU stand in for two ranks' memory:
the kernel only sees a table of source addresses)."""
import dataclasses

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(seed=3, layers=2):
    from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    cfg = dataclasses.replace(PRESETS["qwen3-tiny-d128"], num_layers=layers)
    full = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=seed)
    eng = TrainEngine(full, EngineConfig(zero_stage=1))
    return cfg, full, eng


@pytest.mark.parametrize("tp", [1, 2, 4])
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("pieces", [False, True])
def test_table_sync_matches_sliced_tensors(tp, fp8, pieces):
    from arctic_platform_b200.models.decoder import DecoderLM
    from arctic_platform_b200.models.hf_io import iter_hf_tensors, load_hf_tensor
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.parallel import weight_sync as ws
    from arctic_platform_b200.parallel.tp_sampler import tp_config, tp_slice
    cfg, full, eng = _setup()
    if cfg.num_kv_heads % tp:
        pytest.skip("head count does not divide")
    layout = ws.trainer_layout(eng)
    ptrs, src_rank = ws.engine_source(eng)
    if pieces:
        W = 2
        bufs, table, off = [[], []], {}, 0
        for name, (o, n, _shape) in eng.param_slices.items():
            pl = n // W
            for r in range(W):
                bufs[r].append(eng.param_buf.tensor[o + r * pl:o + (r + 1) * pl])
            table[name] = (pl, off)
            off += pl
        shard_bufs = [torch.cat(b).contiguous() for b in bufs]
        layout["zero3"], layout["world"] = table, W
        ptrs, src_rank = [b.data_ptr() for b in shard_bufs], 0
    hf = {n: t.clone() for n, t in iter_hf_tensors(full)}
    for rank in range(tp):
        local = tp_config(cfg, tp) if tp > 1 else cfg
        shard = DecoderLM(local, "cuda", torch.bfloat16)
        plan = ws.build_sync_plan(layout, shard, full_cfg=cfg, tp_rank=rank, tp=tp, fp8=fp8)
        ws.run_sync_plan(plan, ptrs, src_rank)
        _lib.check_status("sync table")
        ref = DecoderLM(local, "cuda", torch.bfloat16)
        for name, t in hf.items():
            load_hf_tensor(ref, name, tp_slice(name, t, cfg, rank, tp))
        for (n1, a), (_n2, b) in zip(shard.named_parameters(), ref.named_parameters()):
            assert torch.equal(a, b), n1                       # bf16 copies are exact
        if fp8:
            for li, blk in enumerate(ref.blocks):
                for name in ws.FP8_MATRICES:
                    q, sc = plan.fp8[(li, name)]
                    q_ref, sc_ref = ws.quantize_fp8_block128(getattr(blk, name).data)
                    assert torch.equal(sc, sc_ref), (li, name)
                    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8)), (li, name)


def test_fp8_sampler_takes_its_matrices_from_the_sync_pass():
    """A colocated fp8 sampler: after the worker-level hand-over the sampler serves from the block-scaled copies the
    sync kernel wrote (no separate quantisation pass), and generation runs."""
    from arctic_platform_b200.engine.worker import EngineWorker
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    from arctic_platform_b200.ops import _lib
    # every projection's inner dimension a multiple of 128 (the fp8 GEMM's scale blocks)
    cfg = dataclasses.replace(PRESETS["qwen3-tiny-d128"], hidden_size=256, intermediate_size=512, num_heads=4,
                              num_kv_heads=2, num_layers=2)
    job = {"model_name": "qwen3-tiny-d128", "seed": 5,
           "ds_config": {"zero_optimization": {"stage": 1}, "optimizer": {"params": {"lr": 1e-3}}}}
    tr, sm = EngineWorker(), EngineWorker()
    tr.initialize({**job, "job_type": "training"}, model=DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=5))
    sm.initialize({**job, "job_type": "sampling", "seed": 99,
                   "vllm_config": {"kv_cache_tokens": 1 << 13, "max_num_seqs": 8, "max_model_len": 256,
                                   "quantization": "fp8"}},
                  model=DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=99))
    assert sm.sampler.fp8 and sm.sampler._fp8_stale
    n = tr.sync_weights_to(sm)
    assert n > 0 and sm.sampler._sync_plan is not None and not sm.sampler._fp8_stale
    assert tr.engine.weight_norm()["norm"] == pytest.approx(sm.sampler.weight_norm()["norm"], rel=1e-3)
    out = sm.generate([[5, 6, 7, 8, 9, 10, 11, 12]], {"n": 2, "temperature": 0.0, "max_tokens": 6, "ignore_eos": True})
    _lib.check_status("fp8 sampler")
    assert len(out) == 2 and len(out[0]["token_ids"]) == 6 and out[0]["token_ids"] == out[1]["token_ids"]
