"""Rollout record / replay around the clients' ``generate`` and the opt-in per-phase timing of training calls."""
import asyncio
import json

import pytest
import torch

from arctic_platform_b200.utils import record_replay, sft_profile
from arctic_platform_b200.utils.record_replay import ReplayMiss, record_replay_generation


def test_decorator_records_then_replays(tmp_path, monkeypatch):
    calls = []

    @record_replay_generation
    def gen(prompts, n=1):
        calls.append(prompts)
        return [{"token_ids": [len(calls)] * n, "prompt_index": i} for i, _ in enumerate(prompts)]

    @record_replay_generation
    async def agen(prompts):
        calls.append(("async", prompts))
        return [{"token_ids": [7]}]

    for k in ("REPLAY_GENERATION_DIR", "REPLAY_GENERATION_MODE", "REPLAY_START_RECORD", "REPLAY_GENERATION"):
        monkeypatch.delenv(k, raising=False)
    assert gen([[1]])[0]["token_ids"] == [1] and not list(tmp_path.iterdir())        # switched off: a plain call
    monkeypatch.setenv("REPLAY_GENERATION_DIR", str(tmp_path))
    monkeypatch.setenv("REPLAY_GENERATION_MODE", "record")
    monkeypatch.setenv("REPLAY_START_RECORD", "2")
    gen._replay_counter["i"] = 0
    outs = [gen([[1, 2]], n=2) for _ in range(4)]
    assert sorted(p.name for p in tmp_path.iterdir()) == ["generate-2.json", "generate-3.json"]     # tape starts at call 2
    assert json.loads((tmp_path / "generate-3.json").read_text())["result"] == outs[3]
    monkeypatch.setenv("REPLAY_GENERATION_MODE", "replay")
    gen._replay_counter["i"] = 2
    n_before = len(calls)
    assert gen([["anything"]]) == outs[2] and gen([[0]]) == outs[3] and len(calls) == n_before      # the sampler is not asked
    with pytest.raises(ReplayMiss):
        gen([[0]])
    # the async flavour shares the protocol
    monkeypatch.setenv("REPLAY_GENERATION_MODE", "record")
    monkeypatch.setenv("REPLAY_START_RECORD", "0")
    rec = tmp_path / "a"
    monkeypatch.setenv("REPLAY_GENERATION_DIR", str(rec))
    assert asyncio.run(agen([[3]])) == [{"token_ids": [7]}]
    monkeypatch.delenv("REPLAY_GENERATION_MODE")
    monkeypatch.setenv("REPLAY_GENERATION", "1")                                       # the short switch means replay
    agen._replay_counter["i"] = 0
    n_before = len(calls)
    assert asyncio.run(agen([[9]])) == [{"token_ids": [7]}] and len(calls) == n_before


def test_client_generate_goes_through_the_tape(tmp_path, monkeypatch):
    from arctic_platform_b200.rl import ArcticRLClientConfig, create_arctic_rl_client
    from arctic_platform_b200.rl.local_client import ArcticRLLocalClient
    monkeypatch.setenv("REPLAY_GENERATION_DIR", str(tmp_path))
    monkeypatch.setenv("REPLAY_GENERATION_MODE", "record")
    ArcticRLLocalClient.generate._replay_counter["i"] = 0
    c = create_arctic_rl_client(ArcticRLClientConfig(comm_protocol="local", model_name="qwen3-tiny", training_gpus=0,
                                                     sampling_gpus=1, log_prob_gpus=0, vllm_config={"max_model_len": 32}))
    first = c.call("generate", [[4, 5, 6]], {"n": 2, "max_tokens": 3, "temperature": 1.0})
    assert (tmp_path / "generate-0.json").exists()
    monkeypatch.setenv("REPLAY_GENERATION_MODE", "replay")
    ArcticRLLocalClient.generate._replay_counter["i"] = 0
    again = c.call("generate", [[1]], {"n": 1, "max_tokens": 1})
    assert [o["token_ids"] for o in again] == [o["token_ids"] for o in first]
    c.call("shutdown")


def test_phase_buckets_reach_the_metrics(monkeypatch):
    from arctic_platform_b200.engine.worker import EngineWorker
    w = EngineWorker("cpu")
    w.initialize({"model_name": "qwen3-tiny", "job_type": "training", "ds_config": {"zero_optimization": {"stage": 1}}})
    ids = torch.randint(3, 100, (2, 10))
    batch = {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids}
    monkeypatch.delenv("ARL_SFT_PROFILE", raising=False)
    sft_profile.snapshot()
    out = w.forward_backward(batch, {}, {"loss_fn": "sft_ce"})
    assert set(out["metrics"]["_profile_ms"]) == {"fwd_bwd"}
    monkeypatch.setenv("ARL_SFT_PROFILE", "1")
    out = w.forward_backward(batch, {}, {"loss_fn": "sft_ce"})
    prof = out["metrics"]["_profile_ms"]
    assert {"h2d", "fwd", "loss", "bwd", "fwd_bwd"} <= set(prof) and all(v >= 0 for v in prof.values())
    assert prof["fwd"] + prof["bwd"] <= prof["fwd_bwd"] * 1.5
    st = w.step()
    assert st["_profile_ms"]["step"] > 0 and st["metrics"]["grad_norm"] > 0
    assert sft_profile.snapshot() == {}                                    # merged and cleared
    line = sft_profile.format_line(prof)
    assert "fwd=" in line and "%" in line
