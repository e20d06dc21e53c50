"""Speculative decoding on the tensor-op engine: greedy output equals plain greedy decoding for any draft, a draft
equal to the target is always accepted, the sampled distribution is the target's, and the worker builds the engine
from ``speculative_decoding.model``."""
import dataclasses

import pytest
import torch

from arctic_platform_b200.engine.reference_sampler import ReferenceSampler
from arctic_platform_b200.engine.speculative import SpeculativeSampler
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM


def _models(vocab=64, seed_t=1, seed_d=2):
    cfg = dataclasses.replace(PRESETS["qwen3-tiny"], vocab_size=vocab, num_layers=2)
    dcfg = dataclasses.replace(cfg, num_layers=1)
    target = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=seed_t, std=0.2)
    draft = DecoderLM(dcfg, "cpu", torch.float32).init_weights(seed=seed_d, std=0.2)
    return cfg, target, draft


def test_greedy_output_equals_plain_greedy_whatever_the_draft():
    cfg, target, draft = _models()
    plain = ReferenceSampler(cfg, "cpu", model=target, max_seq_len=64)
    prompts = [[3, 9, 27, 5], [11, 2]]
    want = plain.generate(prompts, {"temperature": 0.0, "max_tokens": 13})
    for k in (1, 3, 6):
        spec = SpeculativeSampler(cfg, "cpu", model=target, draft_model=draft, num_speculative_tokens=k, max_seq_len=64)
        got = spec.generate(prompts, {"temperature": 0.0, "max_tokens": 13})
        assert [g["token_ids"] for g in got] == [w["token_ids"] for w in want]
        for g, w in zip(got, want):
            assert g["logprobs"] == pytest.approx(w["logprobs"], abs=1e-4)
        assert spec.stats["target_passes"] <= 2 * 13                     # never more target passes than tokens
    # stop tokens end a sequence inside a round
    stop = want[0]["token_ids"][4]
    spec = SpeculativeSampler(cfg, "cpu", model=target, draft_model=draft, num_speculative_tokens=4, max_seq_len=64)
    out = spec.generate(prompts[:1], {"temperature": 0.0, "max_tokens": 13, "stop_token_ids": [stop]})[0]
    first = want[0]["token_ids"].index(stop)
    assert out["token_ids"] == want[0]["token_ids"][:first + 1] and out["finish_reason"] == "stop"


def test_draft_equal_to_target_is_always_accepted():
    cfg, target, _ = _models()
    spec = SpeculativeSampler(cfg, "cpu", model=target, draft_model=target, num_speculative_tokens=4, max_seq_len=64)
    spec.generate([[1, 2, 3]], {"temperature": 0.0, "max_tokens": 10})
    assert spec.acceptance_rate() == 1.0 and spec.stats["target_passes"] == 2     # 5 tokens per round
    spec.stats.update(proposed=0, accepted=0)
    spec.generate([[1, 2, 3]], {"temperature": 1.0, "max_tokens": 10, "seed": 3})
    assert spec.acceptance_rate() == 1.0                                            # p / q = 1 at every position


def test_sampled_tokens_follow_the_target_distribution():
    """First two generated tokens over many seeded runs against the target's exact joint distribution."""
    cfg, target, draft = _models(vocab=16)
    spec = SpeculativeSampler(cfg, "cpu", model=target, draft_model=draft, num_speculative_tokens=3, max_seq_len=32)
    prompt = [5, 1, 7]
    n = 3000
    out = spec.generate([prompt], {"temperature": 1.0, "max_tokens": 2, "n": n, "seed": 11})
    counts = torch.zeros(16, 16)
    for o in out:
        counts[o["token_ids"][0], o["token_ids"][1]] += 1
    plain = ReferenceSampler(cfg, "cpu", model=target, max_seq_len=32)
    p1 = torch.softmax(spec._logits(target, prompt, 1)[0], -1)
    joint = torch.zeros(16, 16)
    for a in range(16):
        joint[a] = p1[a] * torch.softmax(spec._logits(target, prompt + [a], 1)[0], -1)
    emp = counts / n
    assert float((emp.sum(1) - p1).abs().max()) < 0.035                  # first-token marginal
    assert float((emp - joint).abs().max()) < 0.03                       # joint of the first two tokens
    assert 0.0 < spec.acceptance_rate() < 1.0 and plain is not None


def test_worker_builds_the_speculative_engine_from_the_job_config():
    from arctic_platform_b200.engine.worker import EngineWorker
    w = EngineWorker()
    ok = w.initialize({"job_type": "sampling", "model_name": "qwen3-tiny", "device": "cpu", "dtype": "float32",
                       "vllm_config": {"max_model_len": 64},
                       "arctic_inference_config": {"speculative_decoding": {"model": "qwen3-tiny",
                                                                            "num_speculative_tokens": 3}}})
    assert ok and isinstance(w.sampler, SpeculativeSampler) and w.sampler.k == 3
    out = w.generate([[4, 5, 6]], {"temperature": 0.0, "max_tokens": 6})
    assert len(out[0]["token_ids"]) == 6 and w.sampler.stats["proposed"] > 0
    # a request with history-dependent shaping takes the plain path
    before = dict(w.sampler.stats)
    w.generate([[4, 5, 6]], {"temperature": 0.0, "max_tokens": 4, "repetition_penalty": 1.3})
    assert w.sampler.stats == before
    with pytest.raises(ValueError, match="needs a draft model"):
        SpeculativeSampler(PRESETS["qwen3-tiny"], "cpu", model=w.sampler.model, draft_model=None)


def test_sequences_of_a_request_advance_in_packed_passes():
    """Model passes per round do not grow with the number of sequences, and a batch of ragged prompts (one of which
    stops early) gives each sequence exactly what it gets alone."""
    cfg, target, draft = _models()
    prompts = [[3, 9, 27, 5], [11, 2], [7, 7, 7, 7, 7, 7, 1]]
    plain = ReferenceSampler(cfg, "cpu", model=target, max_seq_len=64)
    want = plain.generate(prompts, {"temperature": 0.0, "max_tokens": 9, "n": 2})
    stop = want[2]["token_ids"][3]                                       # ends prompt 1 (or another one) early
    want = plain.generate(prompts, {"temperature": 0.0, "max_tokens": 9, "n": 2, "stop_token_ids": [stop]})
    spec = SpeculativeSampler(cfg, "cpu", model=target, draft_model=draft, num_speculative_tokens=3, max_seq_len=64)
    got = spec.generate(prompts, {"temperature": 0.0, "max_tokens": 9, "n": 2, "stop_token_ids": [stop]})
    assert [(g["prompt_index"], g["token_ids"], g["finish_reason"]) for g in got] == \
        [(w["prompt_index"], w["token_ids"], w["finish_reason"]) for w in want]
    assert any(g["finish_reason"] == "stop" for g in got) and any(g["finish_reason"] == "length" for g in got)
    passes_six = spec.stats["target_passes"]
    alone = SpeculativeSampler(cfg, "cpu", model=target, draft_model=draft, num_speculative_tokens=3, max_seq_len=64)
    alone.generate(prompts[:1], {"temperature": 0.0, "max_tokens": 9})
    assert passes_six <= 9 and passes_six < 6 * alone.stats["target_passes"]      # six sequences share the passes
    assert spec.stats["rounds"] >= passes_six                                     # rounds are counted per sequence
    # the packed helper returns exactly the rows asked for
    lg = spec._logits_packed(target, [[1, 2, 3], [4, 5]], [2, 1])
    assert [t.shape[0] for t in lg] == [2, 1]
    torch.testing.assert_close(lg[1][0], spec._logits(target, [4, 5], 1)[0], rtol=1e-5, atol=1e-5)
