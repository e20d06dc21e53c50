"""Expert-parallel TRAINING through the engine on two gloo ranks: experts sharded over ranks (dispatch / combine by
all-to-all), dense parameters data-parallel.  After two optimizer steps the dense weights and each rank's experts
equal the single-process model trained on the whole batch -- for ZeRO stage 1 and stage 3."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.test_zorro_equivalence_cpu import make_grpo_batch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _data():
    from arctic_platform_b200.models.config import PRESETS
    cfg = PRESETS["qwen3-moe-tiny"]
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=2, seed=11)
    return cfg, ids % cfg.vocab_size, mask, R


def _train(eng, pb, weights, n_global, scale, steps=2):
    from arctic_platform_b200.models.decoder import token_logprobs
    norms = []
    for _ in range(steps):
        lp, _ = token_logprobs(eng.model, pb)
        eng.backward(-(lp * weights).sum() / n_global * scale)
        norms.append(float(eng.step()["grad_norm"]))
    return norms


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
        from arctic_platform_b200.models.decoder import DecoderLM
        from arctic_platform_b200.parallel.expert_parallel import attach_expert_parallel
        from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
        cfg, ids, mask, R = _data()
        B = ids.shape[0]
        sl = slice(rank * B // world, (rank + 1) * B // world)
        full_pb = build_packed_batch(ids, mask, R)
        n_global = full_pb.labels.numel()
        g = torch.Generator().manual_seed(3)
        w_all = torch.rand(B, R, generator=g) + 0.5
        pb = build_packed_batch(ids[sl], mask[sl], R)
        w_local = pb.gather_from_grid(w_all[sl])
        res = {}
        for stage in (1, 3):
            model = DecoderLM(cfg).init_weights(seed=5, std=0.05)
            attach_expert_parallel(model, world, impl="collective")
            eng = TrainEngine(model, EngineConfig(lr=5e-3, max_grad_norm=1.0, weight_decay=0.01, zero_stage=stage))
            assert any(u.local_only for u in eng.units)
            norms = _train(eng, pb, w_local, n_global, float(world))
            full = eng.full_flat_params().clone()
            named = {}
            for u in eng.units:
                for name, _p in u.params:
                    o, n, shape = eng.param_slices[name]
                    named[name] = full[o:o + n].view(shape).clone()
            res[stage] = {"norms": norms, "named": named, "wn": eng.weight_norm()["norm"]}
        torch.save(res, os.path.join(out_dir, f"e{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_expert_parallel_training_matches_single_process():
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank_main, args=(world, _free_port(), d), nprocs=world, join=True)
        res = [torch.load(os.path.join(d, f"e{r}.pt"), weights_only=False) for r in range(world)]
    # single-process reference on the whole batch
    from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
    from arctic_platform_b200.models.decoder import DecoderLM
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    cfg, ids, mask, R = _data()
    pb = build_packed_batch(ids, mask, R)
    g = torch.Generator().manual_seed(3)
    w_all = torch.rand(ids.shape[0], R, generator=g) + 0.5
    eng = TrainEngine(DecoderLM(cfg).init_weights(seed=5, std=0.05), EngineConfig(lr=5e-3, max_grad_norm=1.0, weight_decay=0.01))
    ref_norms = _train(eng, pb, pb.gather_from_grid(w_all), pb.labels.numel(), 1.0)
    ref = dict(eng.model.named_parameters())
    El = cfg.num_experts // world
    sq = 0.0
    for stage in (1, 3):
        for r in range(world):
            out = res[r][stage]
            assert out["norms"] == pytest.approx(ref_norms, rel=2e-4), (stage, out["norms"], ref_norms)
            for name, t in out["named"].items():
                want = ref[name].data
                if name.endswith("mlp.wgu") or name.endswith("mlp.wdown"):
                    want = want[r * El:(r + 1) * El]
                # Adam divides by sqrt(v): entries with a near-zero gradient may differ by a fraction of lr
                assert (t - want).abs().mean() < 2e-5, (stage, r, name, float((t - want).abs().mean()))
                assert ((t - want).abs() > 1e-3).float().mean() < 1e-3, (stage, r, name)
        # the weight norm counts every expert exactly once and every dense weight once
        sq = sum(float(p.data.double().pow(2).sum()) for p in eng.model.parameters()) ** 0.5
        assert res[0][stage]["wn"] == pytest.approx(sq, rel=1e-5)
    assert res[0][3]["wn"] == pytest.approx(sq, rel=1e-5)
