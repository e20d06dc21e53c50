"""The hosted-service recipes (SFT and GRPO loops) against the in-memory service."""
import json

import torch

from cortex_client.dss_client import NeutrinoClient
from cortex_client.recipes import rl_loop, sft_loop
from tests.fake_service import FakeServiceSession


def _client(s):
    return NeutrinoClient("http://svc", session=s, sleep=lambda x: None, poll_interval=0.0)


def test_sft_loop_creates_trains_saves_and_cancels(tmp_path):
    data = tmp_path / "d.jsonl"
    data.write_text("\n".join(json.dumps(r) for r in [{"input_ids": [1, 2, 3, 4]}, {"input_ids": [5, 6], "labels": [-100, 6]},
                                                        {"input_ids": [7, 8, 9]}]))
    b = sft_loop.collate(sft_loop.read_rows(str(data))[:2])
    assert b["input_ids"].tolist() == [[1, 2, 3, 4], [5, 6, 0, 0]] and b["attention_mask"].tolist() == [[1, 1, 1, 1], [1, 1, 0, 0]]
    assert b["labels"].tolist() == [[1, 2, 3, 4], [-100, 6, -100, -100]]
    s = FakeServiceSession()
    logs = []
    assert sft_loop.main(["--model", "qwen3-4b", "--data", str(data), "--steps", "3", "--batch-size", "2", "--gpus", "2",
                          "--save-every", "2"], client=_client(s)) == 0
    hist = sft_loop.run(_client(s), "qwen3-4b", str(data), steps=2, batch_size=2, log=logs.append)
    assert len(hist) == 2 and hist[0]["loss"] == 0.25 and hist[0]["grad_norm"] == 1.5 and len(logs) == 2
    ops = [c[1].rsplit("/", 1)[-1] for c in s.calls if c[0] == "POST" and c[1].count("/") == 3]
    assert ops.count("forward_backward") == 5 and ops.count("step") == 5 and ops.count("save") == 1
    assert all(j["status"] == "CANCELLED" for j in s.jobs.values()) and len(s.jobs) == 2
    first = next(iter(s.jobs.values()))["body"]
    assert first["sub_jobs"][0]["num_devices"] == 2 and first["sub_jobs"][0]["sub_job_type"] == "training"


def test_rl_loop_samples_scores_updates_and_syncs(tmp_path):
    rows = [{"prompt_ids": [3, 4, 5], "answer_ids": [1, 2]}, {"prompt_ids": [6, 7], "answer_ids": [9]}]
    assert rl_loop.contains_answer([5, 1, 2, 8], rows[0]) == 1.0 and rl_loop.contains_answer([1, 3, 2], rows[0]) == 0.0
    assert rl_loop.contains_answer([1], {}) == 0.0
    outs = [{"token_ids": [1, 2], "prompt_index": 0}, {"token_ids": [8], "prompt_index": 0},
            {"token_ids": [9, 9, 9, 9, 9], "prompt_index": 1}, {"token_ids": [], "prompt_index": 1}]
    batch = rl_loop.build_batch([[3, 4, 5], [6, 7]], outs, 4, torch.tensor([1.0, 0.0, 1.0, 0.0]), n=2)
    assert batch["input_ids"].shape == (4, 7) and batch["input_ids"][2].tolist() == [0, 6, 7, 9, 9, 9, 9]
    assert batch["response_mask"].sum(1).tolist() == [2, 1, 4, 0] and batch["advantages"][0, 0] > 0 > batch["advantages"][1, 0]
    s = FakeServiceSession()
    pf = tmp_path / "p.jsonl"
    pf.write_text("\n".join(json.dumps(r) for r in rows))
    assert rl_loop.main(["--model", "qwen3-4b", "--prompts", str(pf), "--steps", "2", "--prompts-per-step", "2", "--n", "2",
                         "--max-tokens", "4"], client=_client(s)) == 0
    ops = [c[1].rsplit("/", 1)[-1] for c in s.calls if c[0] == "POST" and c[1].count("/") == 3]
    assert ops == ["weight_sync"] + ["generate", "forward", "forward_backward", "step", "weight_sync"] * 2
    body = next(iter(s.jobs.values()))["body"]
    assert [x["sub_job_type"] for x in body["sub_jobs"]] == ["training", "sampling"]
    assert next(iter(s.jobs.values()))["status"] == "CANCELLED"
