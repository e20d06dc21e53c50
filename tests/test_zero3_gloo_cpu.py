"""ZeRO stage 3 (parameters sharded, units gathered on demand) against stage 1 on two gloo ranks: identical losses,
gradient norms and parameters over two optimizer steps with gradient accumulation; full-buffer gather (weight sync),
checkpoint save / load and weight norm on the sharded engine."""
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


def _engine(stage, seed=7):
    from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    model = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32).init_weights(seed=seed)
    return TrainEngine(model, EngineConfig(lr=1e-2, max_grad_norm=1.0, weight_decay=0.01, zero_stage=stage))


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arctic_platform_b200.engine.checkpoint import load_checkpoint, save_checkpoint
        from arctic_platform_b200.models.decoder import token_logprobs
        from arctic_platform_b200.parallel.weight_sync import sync_flat
        from arctic_platform_b200.rl.processors.pipeline import run_pipeline
        from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
        ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=4, seed=3)
        B = ids.shape[0]
        adv = torch.randn(B, 1, generator=torch.Generator().manual_seed(5)).expand(B, R).contiguous()
        sl = slice(rank * B // world, (rank + 1) * B // world)
        res = {}
        for stage in (1, 3):
            eng = _engine(stage)
            assert (eng.zero3 is not None) == (stage == 3)
            losses, norms = [], []
            for step in range(2):
                pb = build_packed_batch(ids[sl], mask[sl], R, dedup=True)
                with torch.no_grad():
                    lp, _ = token_logprobs(eng.model, pb)
                half = (sl.stop - sl.start) // 2
                for mb in (slice(sl.start, sl.start + half), slice(sl.start + half, sl.stop)):     # two micro-batches
                    pbm = build_packed_batch(ids[mb], mask[mb], R, dedup=True)
                    with torch.no_grad():
                        old, _ = token_logprobs(eng.model, pbm)
                    batch = {"input_ids": ids[mb], "attention_mask": mask[mb], "response_mask": mask[mb, -R:],
                             "old_log_probs": pbm.scatter_to_grid(old) + 0.05, "advantages": adv[mb]}
                    meta = {"dp_size": world, "batch_num_tokens": float(mask[:, -R:].sum()), "global_batch_size": float(B)}
                    r = run_pipeline(eng, batch, meta, {"loss_fn": "verl_grpo"}, backward=True)
                    losses.append(r["avg_loss"])
                norms.append(float(eng.step()["grad_norm"]))
            full = eng.full_flat_params().clone()
            res[stage] = {"losses": losses, "norms": norms, "full": full, "wn": eng.weight_norm()["norm"]}
            if stage == 3:
                z = eng.zero3
                assert z.shard_buf.tensor.numel() * world == sum(sum(pl for _n, _f, pl, _s in rows) for rows in z.pieces) * world
                assert z.gathers > 0
                # weight sync target with the engine's flat layout
                dst = torch.zeros(eng.total, dtype=eng.param_dtype)
                sync_flat(eng, dst)
                assert torch.equal(dst, full)
                # checkpoint round trip restores shards, master weights and moments
                ck = os.path.join(out_dir, "ck")
                saved = save_checkpoint(eng, ck, "t1", export_hf=True)
                assert rank != 0 or any(f.endswith(".safetensors") for f in saved["files"])
                eng2 = _engine(3, seed=99)
                assert not torch.equal(eng2.full_flat_params(), full)
                assert load_checkpoint(eng2, ck, "t1") == 2
                assert torch.equal(eng2.full_flat_params(), full)
                assert torch.equal(eng2.exp_avg, eng.exp_avg) and torch.equal(eng2.master, eng.master)
                names = [n for n, _t in eng.iter_hf_tensors()]
                assert len(names) == len(set(names)) and any("q_proj" in n for n in names)
        torch.save(res, os.path.join(out_dir, f"z{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_zero3_matches_zero1_on_two_gloo_ranks():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank_main, args=(2, _free_port(), d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"z{r}.pt"), weights_only=False) for r in range(2)]
    for r in res:
        assert r[1]["losses"] == pytest.approx(r[3]["losses"], rel=1e-5, abs=1e-7)
        assert r[1]["norms"] == pytest.approx(r[3]["norms"], rel=1e-5)
        assert (r[1]["full"] - r[3]["full"]).abs().max() < 1e-5
        assert r[1]["wn"] == pytest.approx(r[3]["wn"], rel=1e-6)
    assert torch.equal(res[0][3]["full"], res[1][3]["full"])


def _live_rank_main(rank, world, port, out_dir):
    """Stage 3 with the gathered blocks kept live between uses (one slot per block) against two alternating slots."""
    import dataclasses
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
        from arctic_platform_b200.models.config import PRESETS
        from arctic_platform_b200.models.decoder import DecoderLM
        from arctic_platform_b200.rl.processors.pipeline import run_pipeline
        ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=4, seed=3)
        B = ids.shape[0]
        adv = torch.randn(B, 1, generator=torch.Generator().manual_seed(5)).expand(B, R).contiguous()
        sl = slice(rank * B // world, (rank + 1) * B // world)
        cfg4 = dataclasses.replace(PRESETS["qwen3-tiny"], num_layers=4)
        res = {}
        for live in (0, 10 ** 12):
            model = DecoderLM(cfg4, "cpu", torch.float32).init_weights(seed=7)
            eng = TrainEngine(model, EngineConfig.from_ds_config(
                {"zero_optimization": {"stage": 3, "stage3_max_live_parameters": live}, "gradient_clipping": 1.0,
                 "optimizer": {"params": {"lr": 1e-2, "weight_decay": 0.01}}}))
            assert eng.zero3.n_slots == (4 if live else 2)
            losses, norms, gathers = [], [], []
            for step in range(2):
                g0 = eng.zero3.gathers
                half = (sl.stop - sl.start) // 2
                for mb in (slice(sl.start, sl.start + half), slice(sl.start + half, sl.stop)):
                    batch = {"input_ids": ids[mb], "attention_mask": mask[mb], "response_mask": mask[mb, -R:],
                             "old_log_probs": torch.full((half, R), -2.0), "advantages": adv[mb]}
                    meta = {"dp_size": world, "batch_num_tokens": float(mask[:, -R:].sum()), "global_batch_size": float(B)}
                    losses.append(run_pipeline(eng, batch, meta, {"loss_fn": "verl_grpo"}, backward=True)["avg_loss"])
                gathers.append(eng.zero3.gathers - g0)
                norms.append(float(eng.step()["grad_norm"]))
            res[bool(live)] = {"losses": losses, "norms": norms, "full": eng.full_flat_params().clone(), "gathers": gathers}
        torch.save(res, os.path.join(out_dir, f"live{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_zero3_live_parameters_gather_once_per_step_and_change_nothing():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_live_rank_main, args=(2, _free_port(), d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"live{r}.pt"), weights_only=False) for r in range(2)]
    for r in res:
        assert r[True]["losses"] == r[False]["losses"] and r[True]["norms"] == r[False]["norms"]
        assert torch.equal(r[True]["full"], r[False]["full"])
        # two slots: every block is gathered in the forward and again in the backward of both micro-batches;
        # live: each of the 4 blocks once per step
        assert r[True]["gathers"] == [4, 4]
        assert all(g > 8 for g in r[False]["gathers"])
