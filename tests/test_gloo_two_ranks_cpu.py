"""Two gloo ranks on CPU: prompt-deduplicated forward/backward equals the ordinary computation, and the
data-parallel engine step (reduce-scatter + clip + AdamW + all-gather through torch.distributed) equals the
single-process step on the whole batch."""
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


def _build_engine(seed=7):
    from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    model = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32).init_weights(seed=seed)
    return TrainEngine(model, EngineConfig(lr=1e-2, max_grad_norm=1.0, weight_decay=0.01))


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arctic_platform_b200.models.decoder import token_logprobs
        from arctic_platform_b200.rl.processors.pipeline import run_pipeline
        from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
        torch.manual_seed(0)
        ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=4, seed=3)
        B = ids.shape[0]
        adv = torch.randn(B, 1, generator=torch.Generator().manual_seed(5)).expand(B, R).contiguous()
        sl = slice(rank * B // world, (rank + 1) * B // world)
        eng = _build_engine()
        # (1) dedup == full on this rank's shard
        pb = build_packed_batch(ids[sl], mask[sl], R, dedup=True)
        full = build_packed_batch(ids[sl], mask[sl], R, dedup=False)
        with torch.no_grad():
            lp_d, _ = token_logprobs(eng.model, pb)
            lp_f, _ = token_logprobs(eng.model, full)
        assert torch.allclose(lp_d, lp_f, atol=1e-5, rtol=1e-5)
        # (2) one GRPO step over two ranks
        old = pb.scatter_to_grid(lp_d)
        batch = {"input_ids": ids[sl], "attention_mask": mask[sl], "response_mask": mask[sl, -R:],
                 "old_log_probs": old + 0.05, "advantages": adv[sl]}
        meta = {"dp_size": world, "batch_num_tokens": float(mask[:, -R:].sum()), "global_batch_size": float(B)}
        r = run_pipeline(eng, batch, meta, {"loss_fn": "verl_grpo"}, backward=True)
        st = eng.step()
        torch.save({"params": eng.param_buf.tensor.clone(), "grad_norm": float(st["grad_norm"]), "loss": r["avg_loss"],
                    "metrics": r["metrics"]}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_match_single_process():
    world = 2
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank_main, args=(world, port, d), nprocs=world, join=True)
        outs = [torch.load(os.path.join(d, f"rank{r}.pt"), weights_only=False) for r in range(world)]
    assert torch.equal(outs[0]["params"], outs[1]["params"])            # replicas stay identical
    assert outs[0]["grad_norm"] == pytest.approx(outs[1]["grad_norm"], rel=1e-6)
    # single-process reference on the whole batch
    from arctic_platform_b200.models.decoder import token_logprobs
    from arctic_platform_b200.rl.processors.pipeline import run_pipeline
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=4, seed=3)
    B = ids.shape[0]
    adv = torch.randn(B, 1, generator=torch.Generator().manual_seed(5)).expand(B, R).contiguous()
    eng = _build_engine()
    pb = build_packed_batch(ids, mask, R)
    with torch.no_grad():
        lp, _ = token_logprobs(eng.model, pb)
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:],
             "old_log_probs": pb.scatter_to_grid(lp) + 0.05, "advantages": adv}
    r = run_pipeline(eng, batch, {}, {"loss_fn": "verl_grpo"}, backward=True)
    st = eng.step()
    assert float(st["grad_norm"]) == pytest.approx(outs[0]["grad_norm"], rel=1e-4)
    # first Adam step moves every weight by ~lr * sign(g): elements whose gradient is at rounding-noise level
    # may differ between summation orders, everything else must agree
    diff = (eng.param_buf.tensor - outs[0]["params"]).abs()
    assert diff.mean() < 1e-5 and (diff > 1e-3).float().mean() < 1e-3, (diff.mean(), (diff > 1e-3).float().mean())
    # global token-mean loss from the two shards equals the single-process loss
    from arctic_platform_b200.common.utils.metrics import finalize_fwd_bwd_metrics
    _, loss2 = finalize_fwd_bwd_metrics([{"metrics": o["metrics"]} for o in outs])
    assert loss2 == pytest.approx(r["metrics"]["loss.sum"] / r["metrics"]["loss.tokens"], rel=1e-5)
