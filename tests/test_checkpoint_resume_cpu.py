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


def test_sleep_is_idempotent_and_a_sleeping_engine_refuses_state_changes(tmp_path):
    """Sleep / wake state machine: sleeping twice keeps the real optimizer state, stepping or touching checkpoints
    while asleep raises (nothing reaches a kernel with empty tensors), waking twice is a no-op, and the engine
    continues exactly as one that never slept."""
    batches = [make_grpo_batch(n_prompts=2, n_samples=2, seed=s) for s in range(4)]
    a, b = _engine(1, False), _engine(1, False)
    _run(a, batches, 2)
    _run(b, batches, 2)
    master = a.master.clone()
    assert not a.asleep
    a.offload_states(("optimizer",))                     # "non_lp" ...
    assert a.asleep and a.master.numel() == 0
    a.offload_states(("optimizer", "grads", "params"))   # ... then "all": must not replace the host copy by an empty one
    assert torch.equal(a._offloaded["master"], master)
    ids, mask, R = batches[0]
    lp, _ = token_logprobs(a.model, build_packed_batch(ids, mask, R, dedup=True))
    with pytest.raises(RuntimeError, match="asleep"):
        a.backward(-lp.mean())
    with pytest.raises(RuntimeError, match="asleep"):
        a.step()
    with pytest.raises(RuntimeError, match="asleep"):
        save_checkpoint(a, str(tmp_path), "t")
    with pytest.raises(RuntimeError, match="asleep"):
        load_checkpoint(a, str(tmp_path), "t")
    assert not list(tmp_path.iterdir())                  # the refused save wrote nothing
    a.reload_states()
    a.reload_states()                                    # waking an engine that is awake changes nothing
    assert not a.asleep and torch.equal(a.master, master)
    for p in a.model.parameters():
        p.grad = None
    a.zero_grad()
    assert _run(a, batches, 2) == _run(b, batches, 2)
    assert torch.equal(a.master, b.master) and torch.equal(a.exp_avg_sq, b.exp_avg_sq)


def test_load_rejects_a_layout_mismatch_and_accepts_a_tag_directory(tmp_path):
    a = _engine(1, False)
    _run(a, [make_grpo_batch(n_prompts=2, n_samples=2, seed=0)], 1)
    saved = save_checkpoint(a, str(tmp_path))            # <dir>/latest -> global_step1
    b = _engine(2, False)
    assert load_checkpoint(b, saved["path"]) == 1        # the tag directory itself (holds the model-states file)
    assert torch.equal(a.master, b.master)
    with pytest.raises(FileNotFoundError):
        load_checkpoint(b, str(tmp_path / "void"), strict=True)
    # a checkpoint written for another parameter layout must not be poured into this engine's flat buffers
    import torch as _t
    f = tmp_path / "global_step1" / "mp_rank_00_model_states.pt"
    st = _t.load(f, weights_only=False)
    st["b200_layout"]["total"] += 8
    _t.save(st, f)
    with pytest.raises(ValueError, match="layout"):
        load_checkpoint(b, str(tmp_path))


class _CustomForPickleTest:
    pass


def test_checkpoint_files_are_read_as_data_only(tmp_path, monkeypatch):
    """A checkpoint file that needs arbitrary unpickling is refused unless the caller says it is trusted."""
    import torch

    from arctic_platform_b200.engine import checkpoint as ck

    Custom = _CustomForPickleTest                          # stands for "some class another framework pickled"
    good, bad = tmp_path / "good.pt", tmp_path / "bad.pt"
    torch.save({"w": torch.ones(2), "step": 3, "names": ["a"]}, good)
    torch.save({"w": torch.ones(2), "obj": Custom()}, bad)
    assert ck._load_pt(good)["step"] == 3
    monkeypatch.delenv("APB_TRUST_CHECKPOINT_PICKLES", raising=False)
    with pytest.raises(RuntimeError, match="APB_TRUST_CHECKPOINT_PICKLES"):
        ck._load_pt(bad)
    monkeypatch.setenv("APB_TRUST_CHECKPOINT_PICKLES", "1")
    assert isinstance(ck._load_pt(bad)["obj"], Custom)
