"""Resume continuity: an engine restored from a checkpoint continues exactly as the one that wrote it -- same
losses, learning rates, gradient norms and bit-identical parameters -- with a warm-up + cosine schedule and
gradient accumulation in flight, for the replicated and the host-offloaded optimizer."""
import pytest
import torch

from arctic_platform_b200.engine.checkpoint import load_checkpoint, save_checkpoint
from arctic_platform_b200.engine.trainer import EngineConfig, SchedulerConfig, TrainEngine
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def _engine(seed, offload):
    model = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32).init_weights(seed=seed)
    cfg = EngineConfig(lr=3e-3, weight_decay=0.05, max_grad_norm=1.0, gradient_accumulation_steps=2,
                       offload_optimizer=offload,
                       scheduler=SchedulerConfig("cosine", warmup_steps=2, total_steps=8, min_lr_ratio=0.1))
    return TrainEngine(model, cfg)


def _run(eng, batches, steps):
    log = []
    for s in range(steps):
        losses = []
        for mb in range(2):
            ids, mask, R = batches[(eng.global_steps * 2 + mb) % len(batches)]
            lp, _ = token_logprobs(eng.model, build_packed_batch(ids, mask, R, dedup=True))
            loss = -(lp.sum() / lp.numel()) / 2
            eng.backward(loss)
            losses.append(float(loss.detach()))
        assert eng.is_gradient_accumulation_boundary()
        out = eng.step()
        log.append((losses, out["last_lr"], float(out["grad_norm"])))
    return log


@pytest.mark.parametrize("offload", [False, True])
def test_resumed_engine_continues_bit_for_bit(tmp_path, offload):
    batches = [make_grpo_batch(n_prompts=2, n_samples=2, seed=s) for s in range(4)]
    a = _engine(1, offload)
    _run(a, batches, 3)
    save_checkpoint(a, str(tmp_path), "mid")
    rest_a = _run(a, batches, 3)

    b = _engine(2, offload)                        # different initial weights: everything must come from the file
    assert load_checkpoint(b, str(tmp_path), "mid") == 3
    assert b.micro_steps == 6
    rest_b = _run(b, batches, 3)
    assert rest_b == rest_a
    assert [lr for _l, lr, _n in rest_b] == [pytest.approx(x) for x in [lr for _l, lr, _n in rest_a]]
    assert rest_b[0][1] < 3e-3                     # past the warm-up: the cosine part of the schedule was restored
    assert torch.equal(a.full_flat_params(), b.full_flat_params())
    assert torch.equal(a.master, b.master) and torch.equal(a.exp_avg, b.exp_avg) and torch.equal(a.exp_avg_sq, b.exp_avg_sq)


def test_latest_tag_and_missing_checkpoint(tmp_path):
    a = _engine(1, False)
    assert load_checkpoint(a, str(tmp_path / "nothing")) == 0      # nothing to resume from: a fresh start
    batches = [make_grpo_batch(n_prompts=2, n_samples=2, seed=0)]
    _run(a, batches, 1)
    save_checkpoint(a, str(tmp_path))                               # default tag global_step1 + "latest"
    _run(a, batches, 1)
    save_checkpoint(a, str(tmp_path))
    assert (tmp_path / "latest").read_text().strip() == "global_step2"
    b = _engine(3, False)
    assert load_checkpoint(b, str(tmp_path)) == 2
    assert torch.equal(a.full_flat_params(), b.full_flat_params())
    c = _engine(3, False)
    assert load_checkpoint(c, str(tmp_path), "global_step1") == 1
    assert not torch.equal(c.full_flat_params(), b.full_flat_params())
