"""Stateful sampler for the hybrid family against the recompute-everything oracle: identical greedy tokens and
log-probs for hybrid, MoE and dense tiny models; prompt work shared between samples; stops, seeds, waves."""
import pytest
import torch

from arctic_platform_b200.engine.hybrid_sampler import HybridSampler
from arctic_platform_b200.engine.reference_sampler import ReferenceSampler
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM


def _pair(preset, seed=3):
    cfg = PRESETS[preset]
    model = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=seed)
    return cfg, HybridSampler(cfg, "cpu", model=model, max_seq_len=256), ReferenceSampler(cfg, "cpu", model=model,
                                                                                          max_seq_len=256)


def _prompts(cfg, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]


@pytest.mark.parametrize("preset", ["qwen3.5-moe-tiny", "qwen3-tiny", "qwen3-moe-tiny"])
def test_greedy_matches_the_recompute_oracle(preset):
    cfg, hyb, ref = _pair(preset)
    prompts = _prompts(cfg, [5, 17, 9])
    sp = {"n": 1, "temperature": 0.0, "max_tokens": 12}
    a, b = hyb.generate(prompts, sp), ref.generate(prompts, sp)
    assert [r["token_ids"] for r in a] == [r["token_ids"] for r in b]
    for ra, rb in zip(a, b):
        assert ra["logprobs"] == pytest.approx(rb["logprobs"], abs=2e-4)
        assert ra["prompt_index"] == rb["prompt_index"] and ra["prompt_len"] == rb["prompt_len"]
    assert hyb.prefill_tokens == 31 and hyb.decode_steps == 11 and hyb.kv_bytes() > 0


def test_prompt_state_is_shared_and_samples_differ():
    cfg, hyb, _ref = _pair("qwen3.5-moe-tiny")
    p = _prompts(cfg, [11])[0]
    res = hyb.generate([p, p, _prompts(cfg, [6], seed=2)[0]], {"n": 4, "temperature": 1.0, "max_tokens": 8, "seed": 5})
    assert len(res) == 12 and [r["prompt_index"] for r in res] == [0] * 4 + [1] * 4 + [2] * 4
    assert hyb.prefill_tokens == 11 + 6                       # the repeated prompt is computed once
    assert len({tuple(r["token_ids"]) for r in res[:8]}) > 1
    again = hyb.generate([p, p, _prompts(cfg, [6], seed=2)[0]], {"n": 4, "temperature": 1.0, "max_tokens": 8, "seed": 5})
    assert [r["token_ids"] for r in again] == [r["token_ids"] for r in res]
    assert all(lp <= 0 for r in res for lp in r["logprobs"])


def test_top_k_one_is_greedy_and_stop_tokens_end_a_sequence():
    cfg, hyb, _ref = _pair("qwen3.5-moe-tiny")
    prompts = _prompts(cfg, [7, 13])
    greedy = hyb.generate(prompts, {"n": 1, "temperature": 0.0, "max_tokens": 10})
    k1 = hyb.generate(prompts, {"n": 2, "temperature": 0.8, "top_k": 1, "max_tokens": 10})
    assert [r["token_ids"] for r in k1] == [greedy[0]["token_ids"]] * 2 + [greedy[1]["token_ids"]] * 2
    stop = greedy[0]["token_ids"][3]
    cut = hyb.generate(prompts, {"n": 1, "temperature": 0.0, "max_tokens": 10, "stop_token_ids": [stop]})
    first = greedy[0]["token_ids"].index(stop)
    assert cut[0]["token_ids"] == greedy[0]["token_ids"][:first + 1] and cut[0]["finish_reason"] == "stop"
    if stop not in greedy[1]["token_ids"]:
        assert cut[1]["token_ids"] == greedy[1]["token_ids"] and cut[1]["finish_reason"] == "length"


def test_waves_and_limits():
    cfg, hyb, _ref = _pair("qwen3.5-moe-tiny")
    prompts = _prompts(cfg, [4, 8, 5, 9, 6])
    sp = {"n": 2, "temperature": 0.0, "max_tokens": 5}
    whole = hyb.generate(prompts, sp)
    hyb.max_batch = 4                                         # two prompts per wave
    waves = hyb.generate(prompts, sp)
    assert [r["token_ids"] for r in waves] == [r["token_ids"] for r in whole]
    with pytest.raises(ValueError):
        hyb.generate([[]], sp)
    with pytest.raises(ValueError):
        hyb.generate([[1] * 255], sp)
    hyb.sleep()
    with pytest.raises(RuntimeError):
        hyb.generate(prompts, sp)
    hyb.wake()
    assert len(hyb.generate(prompts[:1], {"n": 1, "max_tokens": 0, "temperature": 0.0})[0]["token_ids"]) == 0


def test_worker_serves_the_hybrid_family_with_the_stateful_engine():
    from arctic_platform_b200.engine.worker import EngineWorker
    w = EngineWorker("cpu")
    w.initialize({"model_name": "qwen3.5-moe-tiny", "job_type": "sampling", "vllm_config": {"max_model_len": 128}})
    assert isinstance(w.sampler, HybridSampler)
    out = w.generate([[5, 6, 7, 8]], {"n": 2, "temperature": 1.0, "max_tokens": 4})
    assert len(out) == 2 and all(len(r["token_ids"]) == 4 for r in out)
    t = EngineWorker("cpu")
    t.initialize({"model_name": "qwen3.5-moe-tiny", "job_type": "training", "seed": 9,
                  "ds_config": {"zero_optimization": {"stage": 1}}})
    before = w.weight_norm()["norm"]
    t.sync_weights_to(w)
    assert w.weight_norm()["norm"] == pytest.approx(t.weight_norm()["norm"], rel=1e-6) != before


def test_logits_processor_arithmetic():
    from arctic_platform_b200.engine.reference_sampler import LogitsProcessor
    logits = torch.tensor([2.0, -1.0, 0.5, 3.0, -2.0])
    lp = LogitsProcessor({"repetition_penalty": 2.0, "presence_penalty": 0.5, "frequency_penalty": 0.25,
                          "logit_bias": {"4": 1.0, "99": 5.0}, "min_tokens": 3}, stop_ids=[3])
    got = lp.before_temperature(logits, prompt=[0], output=[1, 1])
    # token 0 (prompt): 2 / 2; token 1 (output twice): -1 * 2 - 0.5 - 2 * 0.25; token 4: bias; token 3: held back
    assert got.tolist() == [1.0, -3.0, 0.5, float("-inf"), -1.0]
    assert torch.equal(logits, torch.tensor([2.0, -1.0, 0.5, 3.0, -2.0]))          # the input is not modified
    assert lp.before_temperature(logits, [0], [1, 1, 2])[3] == 3.0                 # min_tokens reached
    assert not LogitsProcessor({"repetition_penalty": 1.0, "min_p": 0.0}).active
    mp_ = LogitsProcessor({"min_p": 0.5})
    kept = mp_.after_temperature(torch.tensor([[0.0, -0.1, -5.0]]))
    assert kept[0, :2].tolist() == pytest.approx([0.0, -0.1]) and kept[0, 2] == float("-inf")


def test_penalties_and_min_tokens_agree_between_the_two_samplers():
    import warnings
    cfg, hyb, ref = _pair("qwen3.5-moe-tiny")
    prompts = _prompts(cfg, [6, 10])
    plain = ref.generate(prompts, {"n": 1, "temperature": 0.0, "max_tokens": 12})
    stop = plain[0]["token_ids"][1]
    sp = {"n": 1, "temperature": 0.0, "max_tokens": 12, "repetition_penalty": 1.3, "frequency_penalty": 0.4,
          "presence_penalty": 0.2, "min_tokens": 6, "stop_token_ids": [stop]}
    with warnings.catch_warnings():
        warnings.simplefilter("error")                     # keys that these engines implement are not reported
        a, b = hyb.generate(prompts, sp), ref.generate(prompts, sp)
    assert [r["token_ids"] for r in a] == [r["token_ids"] for r in b]
    for r in a:
        assert stop not in r["token_ids"][:6]
        assert len(r["token_ids"]) >= 6
    # a strong repetition penalty leaves no token repeated in a short greedy continuation
    strong = hyb.generate(prompts, {"n": 1, "temperature": 0.0, "max_tokens": 10, "repetition_penalty": 50.0,
                                    "presence_penalty": 50.0})
    for r in strong:
        assert len(set(r["token_ids"])) == len(r["token_ids"])
    # min_p = 1 keeps only the most likely token: sampling becomes greedy
    greedy = hyb.generate(prompts, {"n": 1, "temperature": 0.0, "max_tokens": 8})
    mp1 = hyb.generate(prompts, {"n": 2, "temperature": 1.0, "min_p": 1.0, "max_tokens": 8, "seed": 1})
    assert [r["token_ids"] for r in mp1] == [greedy[0]["token_ids"]] * 2 + [greedy[1]["token_ids"]] * 2
