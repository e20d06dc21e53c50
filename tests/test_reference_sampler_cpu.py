"""CPU sampler (recompute oracle): filtering, determinism, stop tokens, full RL loop through the local client."""
import subprocess
import sys

import torch

from arctic_platform_b200.engine.reference_sampler import ReferenceSampler, filter_logits
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM


def test_filter_logits_top_k_top_p():
    z = torch.log(torch.tensor([0.5, 0.3, 0.15, 0.05]))
    assert torch.isfinite(filter_logits(z, 2, 1.0)).tolist() == [True, True, False, False]
    assert torch.isfinite(filter_logits(z, -1, 0.6)).tolist() == [True, True, False, False]   # 0.5 < 0.6 -> need the second
    assert torch.isfinite(filter_logits(z, -1, 0.45)).tolist() == [True, False, False, False]
    assert torch.isfinite(filter_logits(z, 3, 0.9)).tolist() == [True, True, True, False]
    assert torch.equal(filter_logits(z, -1, 1.0), z)


def test_reference_sampler_greedy_seed_and_stop():
    cfg = PRESETS["qwen3-tiny"]
    model = DecoderLM(cfg).init_weights(seed=3)
    s = ReferenceSampler(cfg, "cpu", model=model, max_seq_len=64, seed=1)
    a = s.generate([[5, 6, 7]], {"n": 2, "temperature": 0.0, "max_tokens": 4})
    assert a[0]["token_ids"] == a[1]["token_ids"] and len(a[0]["token_ids"]) == 4 and a[0]["finish_reason"] == "length"
    assert all(lp <= 0 for lp in a[0]["logprobs"])
    b1 = s.generate([[5, 6, 7]], {"n": 3, "temperature": 1.0, "max_tokens": 3, "seed": 11, "top_k": 50, "top_p": 0.9})
    b2 = s.generate([[5, 6, 7]], {"n": 3, "temperature": 1.0, "max_tokens": 3, "seed": 11, "top_k": 50, "top_p": 0.9})
    assert [r["token_ids"] for r in b1] == [r["token_ids"] for r in b2]
    first = a[0]["token_ids"][0]
    c = s.generate([[5, 6, 7]], {"temperature": 0.0, "max_tokens": 4, "stop_token_ids": [first]})
    assert c[0]["token_ids"] == [first] and c[0]["finish_reason"] == "stop"
    s.sleep()
    try:
        s.generate([[1]], None)
        raise AssertionError("generate on a sleeping sampler must raise")
    except RuntimeError:
        pass
    s.wake()
    assert s.weight_norm()["norm"] > 0


def test_simple_grpo_recipe_runs_on_cpu():
    out = subprocess.run([sys.executable, "-m", "recipes.rl.simple_grpo.run_grpo", "--steps", "1", "--prompts", "2",
                          "--samples", "2", "--max-tokens", "4"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert '"step": 0' in out.stdout and "grad_norm" in out.stdout
