"""Rollout routing replay: the sampler reports the experts it chose for every token it was fed, and the trainer's
forward uses exactly those choices (its own router only weighs them), through the packed, de-duplicated layout."""
import torch

from arctic_platform_b200.engine.hybrid_sampler import HybridSampler
from arctic_platform_b200.models import moe
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch


def test_partial_replay_routes_unrecorded_tokens_itself():
    logits = torch.randn(6, 8)
    _w, own = moe.route_topk(logits, 2, True)
    forced = own.flip(0).clone()
    forced[2] = -1
    w, idx = moe.route_topk(logits, 2, True, routed_experts=forced)
    assert torch.equal(idx[2], own[2]) and torch.equal(idx[[0, 1, 3, 4, 5]], forced[[0, 1, 3, 4, 5]])
    assert torch.allclose(w.sum(-1), torch.ones(6))


def _rollouts(cfg, model):
    sampler = HybridSampler(cfg, "cpu", model=model, max_seq_len=64)
    prompts = [[5, 9, 200, 31, 77], [7, 8, 9]]
    res = sampler.generate(prompts, {"n": 2, "temperature": 1.0, "max_tokens": 6, "seed": 3, "return_routed_experts": True})
    plain = sampler.generate(prompts, {"n": 2, "temperature": 1.0, "max_tokens": 6, "seed": 3})
    assert "routed_experts" not in plain[0] and [r["token_ids"] for r in plain] == [r["token_ids"] for r in res]
    assert all(m.routing_log is None for m in model.modules() if isinstance(m, moe.MoEFeedForward))
    return prompts, res


def test_sampler_reports_the_choices_of_a_teacher_forced_pass():
    cfg = PRESETS["qwen3-moe-tiny"]
    model = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=6)
    prompts, res = _rollouts(cfg, model)
    moes = [b.mlp for b in model.blocks]
    for r in res:
        seq = prompts[r["prompt_index"]] + r["token_ids"]
        fed = len(seq) - 1
        assert tuple(r["routed_experts"].shape) == (fed, cfg.num_layers, cfg.num_experts_per_tok)
        assert r["routed_experts"].dtype == torch.int32
        for m in moes:
            m.routing_log = []
        from arctic_platform_b200.ops.attention import AttnLayout
        import numpy as np
        with torch.no_grad():
            model.forward_hidden(torch.tensor(seq[:fed]), torch.arange(fed), AttnLayout.from_cu_seqlens(np.array([0, fed])))
        want = torch.stack([m.routing_log.pop() for m in moes], 1)
        for m in moes:
            m.routing_log = None
        assert torch.equal(r["routed_experts"].long().sort(-1).values, want.sort(-1).values)


def test_trainer_forward_uses_the_recorded_choices():
    cfg = PRESETS["qwen3-moe-tiny"]
    model = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=6)
    prompts, res = _rollouts(cfg, model)
    P, R, L, k = max(len(p) for p in prompts), 6, cfg.num_layers, cfg.num_experts_per_tok
    B = len(res)
    ids = torch.zeros(B, P + R, dtype=torch.int64)
    mask = torch.zeros_like(ids)
    routed = torch.full((B, P + R, L, k), -1, dtype=torch.int32)
    for b, r in enumerate(res):
        p, o = prompts[r["prompt_index"]], r["token_ids"]
        ids[b, P - len(p):P] = torch.tensor(p)
        ids[b, P:P + len(o)] = torch.tensor(o)
        mask[b, P - len(p):P + len(o)] = 1
        routed[b, P - len(p):P + len(o) - 1] = r["routed_experts"]              # the last drawn token was never fed
    pk = build_packed_batch(ids, mask, R, dedup=True)
    assert pk.total_tokens < pk.full_tokens and torch.equal(ids.reshape(-1)[pk.src_index], pk.input_ids)
    # the trainer's router has drifted: on its own it would route differently
    trainer = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=6)
    with torch.no_grad():
        for b in trainer.blocks:
            b.mlp.router.add_(torch.randn_like(b.mlp.router) * 0.5)
    moes = [b.mlp for b in trainer.blocks]

    def used(routed_experts):
        for m in moes:
            m.routing_log = []
        lp, _ = token_logprobs(trainer, pk, routed_experts=routed_experts)
        got = torch.stack([m.routing_log.pop() for m in moes], 1)
        for m in moes:
            m.routing_log = None
        return lp, got
    trainer.train()
    lp_own, own = used(None)
    lp_rep, rep = used(routed)
    want = pk.gather_inputs(routed).long()
    known = (want >= 0).all(-1).all(-1)
    assert known.sum() >= pk.total_tokens - B and not torch.equal(own[known], want[known])
    assert torch.equal(rep[known], want[known])                        # recorded tokens: the sampler's experts
    # unrecorded (last) tokens route themselves; in the first layer nothing upstream depends on the replay
    assert torch.equal(rep[~known][:, 0], own[~known][:, 0])
    assert not torch.allclose(lp_own, lp_rep)
    # gradients flow through the replayed weights, with activation checkpointing as well
    trainer.gradient_checkpointing = True
    lp_ck, _ = used(routed)
    assert torch.allclose(lp_ck, lp_rep, atol=1e-6)
    (-lp_ck.mean()).backward()
    assert all(b.mlp.router.grad is not None and torch.isfinite(b.mlp.router.grad).all() for b in trainer.blocks)
    assert all(m.routed_experts is None for m in moes)


def test_workers_carry_the_choices_from_generate_to_forward_backward():
    from arctic_platform_b200.engine.worker import EngineWorker
    s = EngineWorker("cpu")
    s.initialize({"model_name": "qwen3-moe-tiny", "job_type": "sampling", "seed": 2,
                  "vllm_config": {"max_model_len": 64, "enable_return_routed_experts": True}})
    assert type(s.sampler).__name__ == "HybridSampler"
    prompts = [[5, 9, 200, 31], [7, 8, 9, 11]]
    res = s.generate(prompts, {"n": 2, "temperature": 1.0, "max_tokens": 4})
    cfg = PRESETS["qwen3-moe-tiny"]
    P, R, B = 4, 4, len(res)
    ids = torch.zeros(B, P + R, dtype=torch.int64)
    mask = torch.zeros_like(ids)
    routed = torch.full((B, P + R, cfg.num_layers, cfg.num_experts_per_tok), -1, dtype=torch.int32)
    for b, r in enumerate(res):
        o = r["token_ids"]
        ids[b, :P] = torch.tensor(prompts[r["prompt_index"]])
        ids[b, P:P + len(o)] = torch.tensor(o)
        mask[b, :P + len(o)] = 1
        routed[b, :P + len(o) - 1] = torch.as_tensor(r["routed_experts"])
    t = EngineWorker("cpu")
    t.initialize({"model_name": "qwen3-moe-tiny", "job_type": "training", "seed": 9,
                  "ds_config": {"zero_optimization": {"stage": 1}, "optimizer": {"params": {"lr": 1e-3}}}})
    g = torch.Generator().manual_seed(0)
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, P:].contiguous(),
             "old_log_probs": torch.randn(B, R, generator=g) * 0.01 - 2.0,
             "advantages": torch.randn(B, 1, generator=g).expand(B, R).contiguous(), "routed_experts": routed}
    seen = []
    real = moe.route_topk

    def spy(*a, **kw):
        forced = kw.get("routed_experts", a[6] if len(a) > 6 else None)
        seen.append(forced is not None)
        return real(*a, **kw)
    moe.route_topk = spy
    try:
        out = t.forward_backward(batch, {"response_length": R, "zorro_train_enable": True, "num_micro_batches": 2},
                                 {"loss_fn": "verl_grpo"})
    finally:
        moe.route_topk = real
    # every layer pass of both micro-batches replayed a decision (each asks the router itself once more, for the
    # last token of every row, which no sampler pass ever saw)
    assert sum(seen) == cfg.num_layers * 2 and seen[0::2] == [True] * (cfg.num_layers * 2)
    assert torch.isfinite(torch.as_tensor(out["avg_loss"]))
    assert t.step()["metrics"]["grad_norm"] > 0
