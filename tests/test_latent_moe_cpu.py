"""Latent mixture of experts with non-gated relu^2 experts: the layer against a per-token restatement, its place in
the decoder (training step, activation checkpointing with routing replay, sampling) and checkpoint names."""
import tempfile

import pytest
import torch

from arctic_platform_b200.models.config import PRESETS, DecoderConfig
from arctic_platform_b200.models.decoder import DecoderLM
from arctic_platform_b200.models.latent_moe import LatentMoEFeedForward, nongated_grouped_ffn, relu2


def _layer(latent=True, seed=0, **over):
    base = PRESETS["latent-moe-tiny"]
    cfg = DecoderConfig(**{**base.to_dict(), "moe_latent_dim": 64 if latent else 0, **over})
    torch.manual_seed(seed)
    m = LatentMoEFeedForward(cfg, "cpu", torch.float32)
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.2)
        m.e_score_correction_bias.normal_(0, 0.05)
    return cfg, m


def _per_token(cfg, m, x):
    """The layer written token by token from its definition."""
    scores = torch.sigmoid(x @ m.router.t())
    pick = scores + m.e_score_correction_bias + (m.expert_bias if m.expert_bias is not None else 0)
    out = torch.zeros_like(x)
    E, G = cfg.num_experts, cfg.moe_n_group
    for t in range(x.shape[0]):
        groups = pick[t].view(G, E // G)
        best = groups.topk(2, -1).values.sum(-1).topk(cfg.moe_topk_group).indices.tolist()
        cand = [e for e in range(E) if e // (E // G) in best]
        chosen = sorted(cand, key=lambda e: -float(pick[t, e]))[:cfg.num_experts_per_tok]
        w = scores[t, chosen]
        if cfg.norm_topk_prob:
            w = w / w.sum()
        for e, we in zip(chosen, w):
            z = x[t] if m.fc1 is None else m.fc1 @ x[t]
            y = m.wdown[e] @ relu2(m.wup[e] @ z) * we * cfg.moe_route_scale
            out[t] += y if m.fc2 is None else m.fc2 @ y
        out[t] += m.shared_wdown @ relu2(m.shared_wup @ x[t])
    return out


@pytest.mark.parametrize("latent", [True, False])
def test_layer_matches_its_per_token_definition(latent):
    cfg, m = _layer(latent)
    x = torch.randn(23, cfg.hidden_size)
    with torch.no_grad():
        assert torch.allclose(m(x), _per_token(cfg, m, x), atol=1e-4, rtol=1e-4)
    assert int(m.last_tokens_per_expert.sum()) == 23 * cfg.num_experts_per_tok
    assert (m.wup.shape[-1] == 64) == latent and (m.fc1 is not None) == latent


def test_gradients_reach_every_part_and_replay_keeps_the_decision():
    cfg, m = _layer()
    m.train()
    x = torch.randn(40, cfg.hidden_size, requires_grad=True)
    m(x).square().sum().backward()
    for name, p in m.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().sum() > 0, name
    assert x.grad.abs().sum() > 0 and float(m.tokens_per_expert.sum()) == 40 * cfg.num_experts_per_tok
    # a forced decision is used as given, with weights from the current scores
    forced = torch.randint(0, cfg.num_experts, (40, cfg.num_experts_per_tok))
    m.routed_experts = forced
    m(x.detach())
    assert torch.equal(m.last_tokens_per_expert, torch.bincount(forced.reshape(-1), minlength=cfg.num_experts))
    m.routed_experts = None
    before = m.expert_bias.clone()
    load = m.update_expert_bias(1e-2, group=False)
    assert load is not None and not torch.equal(m.expert_bias, before) and float(m.tokens_per_expert.sum()) == 0


def test_empty_experts_and_empty_input():
    w1, w2 = torch.randn(3, 5, 4), torch.randn(3, 4, 5)
    x = torch.randn(6, 4)
    y = nongated_grouped_ffn(x, w1, w2, torch.tensor([0, 6, 0]))
    assert torch.allclose(y, relu2(x @ w1[1].t()) @ w2[1].t(), atol=1e-6)
    assert nongated_grouped_ffn(x[:0], w1, w2, torch.tensor([0, 0, 0])).shape == (0, 4)


def _batch(cfg, seed=0):
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    from tests.test_zorro_equivalence_cpu import make_grpo_batch
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2, seed=seed)
    return build_packed_batch(ids, mask, R, dedup=True)


def test_decoder_trains_checkpoints_and_samples_with_the_layer():
    from arctic_platform_b200.engine.hybrid_sampler import HybridSampler
    from arctic_platform_b200.engine.reference_sampler import ReferenceSampler
    from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
    from arctic_platform_b200.models.decoder import token_logprobs
    cfg = PRESETS["latent-moe-tiny"]
    assert cfg.num_parameters() == sum(p.numel() for p in DecoderLM(cfg, "meta", torch.float32).parameters())
    model = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=1)
    plain = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=1)
    model.gradient_checkpointing, model.checkpoint_targets = True, ("routed_experts",)
    pb = _batch(cfg)
    grads = []
    for mdl in (plain, model):
        mdl.train()
        lp, _ = token_logprobs(mdl, pb)
        (-lp.mean()).backward()
        grads.append(torch.cat([p.grad.reshape(-1) for p in mdl.parameters()]))
    assert torch.allclose(grads[0], grads[1], atol=1e-6)              # recompute with replayed routing == no recompute
    eng = TrainEngine(DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=1),
                      EngineConfig.from_ds_config({"optimizer": {"params": {"lr": 1e-3}}, "zero_optimization": {"stage": 1}}))
    losses = []
    for _ in range(3):
        lp, _ = token_logprobs(eng.model, pb)
        loss = -lp.mean()
        eng.backward(loss)
        eng.step()
        losses.append(float(loss.detach()))
    assert losses[2] < losses[0]
    bias = [m.expert_bias.clone() for m in eng.model.modules() if isinstance(m, LatentMoEFeedForward)]
    assert len(bias) == cfg.num_layers and any(float(b.abs().sum()) > 0 for b in bias)   # nudged at every step
    hyb = HybridSampler(cfg, "cpu", model=eng.model, max_seq_len=64)
    ref = ReferenceSampler(cfg, "cpu", model=eng.model, max_seq_len=64)
    sp = {"n": 1, "temperature": 0.0, "max_tokens": 6}
    prompts = [[5, 9, 200, 31], [7, 8, 9]]
    assert [r["token_ids"] for r in hyb.generate(prompts, sp)] == [r["token_ids"] for r in ref.generate(prompts, sp)]


def test_expert_parallelism_refuses_the_layout():
    from arctic_platform_b200.parallel import expert_parallel
    model = DecoderLM(PRESETS["latent-moe-tiny"], "cpu", torch.float32)
    with pytest.raises(NotImplementedError, match="SwiGLU"):
        expert_parallel.attach_expert_parallel(model, 1, None)


def test_checkpoint_names_and_config_round_trip():
    from arctic_platform_b200.models.hf_io import iter_hf_tensors, load_hf_checkpoint, save_hf_checkpoint
    cfg = PRESETS["latent-moe-tiny"]
    a = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=2)
    with torch.no_grad():
        for m in a.modules():
            if isinstance(m, LatentMoEFeedForward):
                m.e_score_correction_bias.uniform_(-0.1, 0.1)
    names = [n for n, _ in iter_hf_tensors(a)]
    for want in ("model.layers.0.mlp.gate.e_score_correction_bias", "model.layers.1.mlp.fc1_latent_proj.weight",
                 "model.layers.0.mlp.shared_experts.up_proj.weight", "model.layers.1.mlp.experts.7.down_proj.weight"):
        assert want in names
    assert not any("gate_proj" in n for n in names if ".mlp." in n)
    with tempfile.TemporaryDirectory() as d:
        save_hf_checkpoint(a, d)
        import json, os
        back = DecoderConfig.from_hf_dict(json.load(open(os.path.join(d, "config.json"))))
        for f in ("moe_activation", "moe_latent_dim", "moe_score_func", "moe_route_scale", "moe_n_group",
                  "moe_topk_group", "moe_expert_bias", "shared_expert_intermediate_size", "num_experts"):
            assert getattr(back, f) == getattr(cfg, f), f
        b = DecoderLM(back, "cpu", torch.float32).init_weights(seed=9)
        load_hf_checkpoint(b, d)
    for (n1, p1), (_n2, p2) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.equal(p1, p2), n1
    for m1, m2 in zip(a.modules(), b.modules()):
        if isinstance(m1, LatentMoEFeedForward):
            assert torch.equal(m1.e_score_correction_bias, m2.e_score_correction_bias)
