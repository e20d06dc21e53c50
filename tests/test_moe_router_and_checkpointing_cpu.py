"""Router variants (sigmoid scores, selection bias, group-limited routing, replayed decisions), routing replay
across activation-checkpoint recompute, and selective checkpointing of block parts."""
import pytest
import torch

from arctic_platform_b200.models import moe
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def test_route_topk_variants():
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0], [0.0, 0.0, 3.0, 1.0]])
    w, idx = moe.route_topk(logits, 2, renorm=True)
    assert idx.tolist() == [[0, 1], [2, 3]] and torch.allclose(w.sum(-1), torch.ones(2))
    ws, idxs = moe.route_topk(logits, 2, renorm=False, score_func="sigmoid", route_scale=2.5)
    assert idxs.tolist() == [[0, 1], [2, 3]]
    assert torch.allclose(ws, 2.5 * torch.sigmoid(torch.tensor([[2.0, 1.0], [3.0, 1.0]])))
    # a selection bias changes WHO is picked, not the weight they get
    bias = torch.tensor([-10.0, 0.0, 0.0, 0.0])
    wb, idxb = moe.route_topk(logits, 2, renorm=False, expert_bias=bias)
    probs = torch.softmax(logits, -1)
    assert idxb[0].tolist() == [1, 2] and torch.allclose(wb[0], probs[0, [1, 2]])
    # replay: decisions from outside, weights from the current scores
    forced = torch.tensor([[3, 0], [1, 0]])
    wr, idxr = moe.route_topk(logits, 2, renorm=False, routed_experts=forced)
    assert torch.equal(idxr, forced) and torch.allclose(wr, probs.gather(1, forced))
    with pytest.raises(ValueError):
        moe.route_topk(logits, 2, True, routed_experts=torch.tensor([[0], [1]]))
    with pytest.raises(NotImplementedError):
        moe.route_topk(logits, 2, True, score_func="tanh")
    # group-limited: two groups {0,1} {2,3}, one group allowed per token -> both picks from the better group
    lg = torch.tensor([[5.0, -5.0, 4.0, 3.9]])
    _w, free = moe.route_topk(lg, 2, True, score_func="sigmoid")
    _w, lim = moe.route_topk(lg, 2, True, score_func="sigmoid", n_group=2, topk_group=1)
    assert sorted(free[0].tolist()) == [0, 2] and sorted(lim[0].tolist()) == [2, 3]


def _moe_cfg(**kw):
    import dataclasses
    return dataclasses.replace(PRESETS["qwen3-moe-tiny"], **kw)


def test_expert_bias_moves_load_toward_balance():
    cfg = _moe_cfg(moe_expert_bias=True, moe_score_func="sigmoid")
    m = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=0)
    layer = m.blocks[0].mlp
    assert layer.expert_bias is not None and "blocks.0.mlp.expert_bias" in dict(m.named_buffers())
    with torch.no_grad():
        layer.router[0] += 0.5                               # expert 0 attracts everything
    x = torch.randn(256, cfg.hidden_size, generator=torch.Generator().manual_seed(0)) * 0.5 + 0.3
    m.train()
    loads = []
    for _ in range(60):
        layer(x)
        loads.append(layer.update_expert_bias(coeff=0.05, group=False))
    assert layer.tokens_per_expert.sum() == 0
    assert loads[-1].max() - loads[-1].min() < loads[0].max() - loads[0].min()
    assert layer.expert_bias[0] < 0 and abs(float(layer.expert_bias.mean())) < 1e-6
    m.eval()
    layer(x)
    assert layer.tokens_per_expert.sum() == 0                # counted in training passes only
    plain = DecoderLM(PRESETS["qwen3-moe-tiny"], "cpu", torch.float32).blocks[0].mlp
    assert plain.expert_bias is None and plain.update_expert_bias() is None


def _grads(model, pb):
    for p in model.parameters():
        p.grad = None
    lp, _ = token_logprobs(model, pb)
    lp.mean().backward()
    return lp.detach().clone(), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}


def test_routing_replay_keeps_recompute_consistent(monkeypatch):
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2, seed=4)
    pb = build_packed_batch(ids, mask, R, dedup=True)
    model = DecoderLM(PRESETS["qwen3-moe-tiny"], "cpu", torch.float32).init_weights(seed=1)
    want_lp, want = _grads(model, pb)
    # a router whose scores wobble from call to call, as last-bit noise upstream of the router would make them
    real = moe.route_topk
    calls = {"n": 0}

    def wobbly(logits, *a, **kw):
        calls["n"] += 1
        if kw.get("routed_experts") is None and len(a) < 6:
            with torch.no_grad():
                noise = torch.randn(logits.shape, generator=torch.Generator().manual_seed(calls["n"])) * 5.0
                _w, idx = real(logits + noise, *a, **kw)
            kw = {**kw, "routed_experts": idx}
        return real(logits, *a, **kw)

    model.gradient_checkpointing = True
    got_lp, got = _grads(model, pb)                           # deterministic router: replay changes nothing
    assert torch.equal(got_lp, want_lp)
    for n in want:
        assert torch.allclose(got[n], want[n], atol=1e-6), n
    monkeypatch.setattr(moe, "route_topk", wobbly)
    lp1, g1 = _grads(model, pb)                               # original pass and recompute would route differently ...
    assert all(torch.isfinite(v).all() for v in g1.values())  # ... but the recompute replays the captured decision
    assert all(m._captured == [] and m.replay_mode is None for m in model.modules() if isinstance(m, moe.MoEFeedForward))


@pytest.mark.parametrize("preset,targets", [("qwen3-tiny", ("mlp",)), ("qwen3-moe-tiny", ("routed_experts",)),
                                            ("qwen3.5-moe-tiny", ("linear_attn", "mlp")),
                                            ("qwen3-tiny", ("norm", "attn_proj")),
                                            ("qwen3.5-moe-tiny", ("norm", "attn_proj", "routed_experts"))])
def test_selective_checkpointing_matches_plain(preset, targets):
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2, seed=5)
    cfg = PRESETS[preset]
    pb = build_packed_batch(ids % cfg.vocab_size, mask, R, dedup=True)
    model = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=2)
    want_lp, want = _grads(model, pb)
    model.gradient_checkpointing = True
    model.checkpoint_targets = targets
    import torch.utils.checkpoint as ck
    seen = []
    real = ck.checkpoint

    def spy(fn, *a, **kw):
        seen.append(getattr(fn, "__name__", type(fn).__name__))
        return real(fn, *a, **kw)
    ck.checkpoint = spy
    try:
        got_lp, got = _grads(model, pb)
    finally:
        ck.checkpoint = real
    assert torch.equal(got_lp, want_lp) and seen and "DecoderBlock" not in seen
    for n in want:
        assert torch.allclose(got[n], want[n], atol=1e-6, rtol=1e-5), n


def test_checkpoint_frequency_and_target_validation():
    cfg = PRESETS["qwen3.5-moe-tiny"]
    model = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=2)
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2, seed=5)
    pb = build_packed_batch(ids % cfg.vocab_size, mask, R, dedup=True)
    want_lp, want = _grads(model, pb)
    import torch.utils.checkpoint as ck
    real, seen = ck.checkpoint, []

    def spy(fn, *a, **kw):
        seen.append(getattr(fn, "__name__", type(fn).__name__))
        return real(fn, *a, **kw)
    for mode, targets, freq, per_block in (("full", None, 2, 1), ("selective", None, 3, 2), ("selective", ["norm"], 1, 2)):
        model.set_activation_checkpointing(mode, targets, freq)
        assert model.checkpoint_targets == (() if mode == "full" else ("norm",))
        seen.clear()
        ck.checkpoint = spy
        try:
            got_lp, got = _grads(model, pb)
        finally:
            ck.checkpoint = real
        blocks = len(range(0, cfg.num_layers, freq))
        assert len(seen) == blocks * per_block, (mode, freq, seen)        # every freq-th block, 2 norms per block
        assert torch.equal(got_lp, want_lp)
        for n in want:
            assert torch.allclose(got[n], want[n], atol=1e-6, rtol=1e-5), n
    with pytest.raises(ValueError, match="Unsupported selective activation checkpoint targets: \\['mla_up'\\]"):
        model.set_activation_checkpointing("selective", ["norm", "mla_up"])
    with pytest.raises(ValueError, match="mode"):
        model.set_activation_checkpointing("partial")
    with pytest.raises(ValueError, match="freq"):
        model.set_activation_checkpointing("full", None, 0)
    dense = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32)
    assert dense.blocks[0].supported_ac_targets() == {"norm", "attn_proj", "mlp"}
    assert model.blocks[0].supported_ac_targets() == {"norm", "linear_attn", "routed_experts", "mlp"}
    with pytest.raises(ValueError, match="not supported by the selected model layers"):
        dense.set_activation_checkpointing("selective", ["linear_attn"])


def test_worker_config_selects_selective_mode():
    from arctic_platform_b200.engine.worker import EngineWorker
    w = EngineWorker("cpu")
    w.initialize({"model_name": "qwen3-moe-tiny", "job_type": "training", "ds_config": {"zero_optimization": {"stage": 1}},
                  "ds_worker_config": {"gradient_checkpointing": {"mode": "selective", "targets": ["routed_experts"]}}})
    assert w.engine.model.gradient_checkpointing and w.engine.model.checkpoint_targets == ("routed_experts",)


def test_worker_reads_the_nested_ac_config_of_the_training_config():
    from arctic_platform_b200.engine.worker import EngineWorker
    base = {"model_name": "qwen3-tiny", "job_type": "training", "ds_config": {"zero_optimization": {"stage": 1}}}
    w = EngineWorker("cpu")
    w.initialize({**base, "training_config": {"ac_config": {"mode": "full", "freq": 2, "offload_config": {
        "enabled": True, "keep_last_n": 1, "tensor_size_threshold": 4096}}}})
    m = w.engine.model
    assert m.gradient_checkpointing and m.checkpoint_targets == () and m.checkpoint_freq == 2
    assert w.activation_offload is not None and w.activation_offload.min_bytes == 4096
    w2 = EngineWorker("cpu")
    w2.initialize({**base, "training_config": {"ac_config": {"mode": "selective"}}})
    assert w2.engine.model.checkpoint_targets == ("norm",) and w2.activation_offload is None
    with pytest.raises(ValueError, match="requires ac_config.mode='full'"):
        EngineWorker("cpu").initialize({**base, "training_config": {"ac_config": {
            "mode": "selective", "offload_config": {"enabled": True}}}})


def test_engine_updates_and_checkpoints_the_load_balancing_bias(tmp_path):
    from arctic_platform_b200.engine.checkpoint import load_checkpoint, save_checkpoint
    from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
    cfg = _moe_cfg(moe_expert_bias=True)
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2, seed=3)
    pb = build_packed_batch(ids % cfg.vocab_size, mask, R, dedup=True)
    eng = TrainEngine(DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=1), EngineConfig(lr=1e-3, moe_bias_update_rate=0.01))
    for _ in range(2):
        lp, _ = token_logprobs(eng.model, pb)
        eng.backward(-lp.mean())
        eng.step()
    bias = eng.model.blocks[0].mlp.expert_bias.clone()
    assert bias.abs().max() > 0 and eng.model.blocks[0].mlp.tokens_per_expert.sum() == 0
    save_checkpoint(eng, str(tmp_path), "t")
    other = TrainEngine(DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=2), EngineConfig(lr=1e-3))
    assert other.model.blocks[0].mlp.expert_bias.abs().max() == 0
    load_checkpoint(other, str(tmp_path), "t")
    assert torch.equal(other.model.blocks[0].mlp.expert_bias, bias)
