"""Qwen3.5-style hybrid (gated delta-net linear attention + gated full attention with partial rotary + (1+w) norms +
routed experts with a shared expert): the chunked rule against the token recurrence, prompt reuse under the
deduplicated layout, Hugging Face name round trip, one engine step."""
import pytest
import torch

from arctic_platform_b200.models.config import PRESETS, DecoderConfig
from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
from arctic_platform_b200.models.linear_attention import (causal_conv1d, gated_delta_rule_chunked,
                                                          gated_delta_rule_recurrent)
from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
from tests.test_zorro_equivalence_cpu import make_grpo_batch


@pytest.mark.parametrize("T,chunk", [(150, 64), (64, 64), (7, 16), (130, 16)])
def test_chunked_rule_equals_recurrence_and_carries_state(T, chunk):
    torch.manual_seed(T)
    H, Dk, Dv = 3, 16, 24
    q, k, v = torch.randn(T, H, Dk), torch.randn(T, H, Dk), torch.randn(T, H, Dv)
    g, beta = -torch.rand(T, H) * 0.5, torch.sigmoid(torch.randn(T, H))
    S0 = torch.randn(H, Dk, Dv) * 0.1
    o1, S1 = gated_delta_rule_recurrent(q, k, v, g, beta, S0)
    o2, S2 = gated_delta_rule_chunked(q, k, v, g, beta, S0, chunk=chunk)
    assert (o1 - o2).abs().max() < 1e-5 and (S1 - S2).abs().max() < 1e-5
    cut = T // 3 + 1
    oa, Sa = gated_delta_rule_chunked(q[:cut], k[:cut], v[:cut], g[:cut], beta[:cut], S0, chunk=chunk)
    ob, Sb = gated_delta_rule_chunked(q[cut:], k[cut:], v[cut:], g[cut:], beta[cut:], Sa, chunk=chunk)
    assert (torch.cat([oa, ob]) - o1).abs().max() < 1e-5 and (Sb - S1).abs().max() < 1e-5


def test_causal_conv_state_carry():
    torch.manual_seed(0)
    x, w = torch.randn(20, 5), torch.randn(5, 4)
    y, _ = causal_conv1d(x, w)
    ya, st = causal_conv1d(x[:9], w)
    yb, _ = causal_conv1d(x[9:], w, st)
    assert torch.allclose(torch.cat([ya, yb]), y, atol=1e-6)
    assert torch.allclose(y[0], x[0] * w[:, -1], atol=1e-6)          # the first output sees only the first input


def test_hybrid_model_dedup_equivalence_and_hf_round_trip(tmp_path):
    cfg = PRESETS["qwen3.5-moe-tiny"]
    m = DecoderLM(cfg).init_weights(seed=2, std=0.05)
    assert [b.kind for b in m.blocks] == ["linear_attention"] * 3 + ["full_attention"]
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=3, seed=1)
    ids = ids % cfg.vocab_size
    pd, pf = build_packed_batch(ids, mask, R, dedup=True), build_packed_batch(ids, mask, R, dedup=False)
    lp_d, e_d = token_logprobs(m, pd)
    lp_f, e_f = token_logprobs(m, pf)
    assert pd.total_tokens < pf.total_tokens
    assert (lp_d - lp_f).abs().max() < 1e-4 and (e_d - e_f).abs().max() < 1e-4
    lp_d.sum().backward()
    g1 = [p.grad.clone() for p in m.parameters()]
    for p in m.parameters():
        p.grad = None
    token_logprobs(m, pf)[0].sum().backward()
    assert all(p.grad is not None for p in m.parameters())
    assert max(float((a - p.grad).abs().max()) for a, p in zip(g1, m.parameters())) < 2e-3
    # Hugging Face names: save, reload into a differently initialised model, same outputs
    from arctic_platform_b200.models.hf_io import hf_param_names, iter_hf_tensors, load_hf_checkpoint, save_hf_checkpoint
    names = [n for n, _ in iter_hf_tensors(m)]
    assert names == hf_param_names(cfg) and any("linear_attn.conv1d.weight" in n for n in names)
    assert any("shared_expert_gate" in n for n in names)
    save_hf_checkpoint(m, tmp_path)
    cfg2 = DecoderConfig.from_hf_dict(__import__("json").loads((tmp_path / "config.json").read_text()))
    assert cfg2.layer_types == cfg.layer_types and cfg2.partial_rotary_factor == 0.25 and cfg2.attn_output_gate
    m2 = DecoderLM(cfg2).init_weights(seed=9, std=0.05)
    load_hf_checkpoint(m2, tmp_path)
    with torch.no_grad():
        assert (token_logprobs(m2, pd)[0] - lp_d).abs().max() < 1e-5


def test_hybrid_model_trains_through_the_engine():
    from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
    cfg = PRESETS["qwen3.5-moe-tiny"]
    eng = TrainEngine(DecoderLM(cfg).init_weights(seed=3, std=0.05), EngineConfig(lr=1e-2, max_grad_norm=1.0))
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2, seed=4)
    pb = build_packed_batch(ids % cfg.vocab_size, mask, R)
    before = float(-token_logprobs(eng.model, pb)[0].mean())
    for _ in range(3):
        eng.backward(-token_logprobs(eng.model, pb)[0].mean())
        assert float(eng.step()["grad_norm"]) > 0
    assert float(-token_logprobs(eng.model, pb)[0].mean()) < before
