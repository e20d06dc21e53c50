"""The packaged examples run end to end on CPU with the tiny preset."""
import json

import pytest


def _records(lines):
    return [json.loads(x) for x in lines]


def test_rl_weight_sync_example():
    from arctic_platform_b200.rl.examples import weight_sync_example as ex
    lines = []
    res = ex.run(steps=2, log=lines.append)
    recs = _records(lines)
    assert [r["step"] for r in recs[:2]] == [0, 1] and all(r["grad_norm"] > 0 for r in recs[:2])
    assert res["training_norm_after"] != res["training_norm_before"]                # the weights moved
    assert res["sampling_norm_after"] == pytest.approx(res["training_norm_after"], rel=1e-3)    # and the sampler has them
    assert ex.main(["--steps", "1"]) == 0


def test_rl_async_example_trains_on_stale_rollouts():
    from arctic_platform_b200.rl.examples import local_server_example as ex
    hist = ex.run(updates=3, sync_every=2, log=lambda _x: None)
    assert [h["update"] for h in hist] == [0, 1, 2]
    assert all(h["staleness"] >= 0 and h["grad_norm"] > 0 for h in hist)
    assert hist[0]["sampled_at_version"] == 0


def test_rl_inference_example():
    from arctic_platform_b200.rl.examples import inference_example as ex
    lines = []
    res = ex.run(log=lines.append)
    assert len(res["greedy"]) == 2 and len(res["sampled"]) == 6 and res["reattached_equal"]
    assert res["stopped"][0]["finish_reason"] == "stop" and len(res["stopped"][0]["token_ids"]) <= 3
    assert {"token_ids", "logprobs", "finish_reason", "prompt_index"} <= set(_records(lines)[0]["fields"])


def test_sft_examples(tmp_path):
    from arctic_platform_b200.sft.examples import run_sft_ckpt_resume_demo, run_sft_generate_demo, sft_example
    lines = []
    a = sft_example.parser().parse_args(["--steps", "12", "--accumulate", "2", "--save-every", "6",
                                         "--checkpoint-path", str(tmp_path / "ck")])
    hist = sft_example.run(a, log=lines.append)
    assert len(hist) == 12 and hist[-1]["loss"] < hist[0]["loss"]
    assert sum("saved" in json.loads(x) for x in lines) == 2 and len(list((tmp_path / "ck").glob("arctic_rl_job_*/checkpoint-12"))) == 1
    lines = []
    assert run_sft_ckpt_resume_demo.main(["--steps", "3", "--checkpoint-path", str(tmp_path / "resume")], log=lines.append) == 0
    recs = _records(lines)
    assert recs[1]["resumed_at"] == 3 and recs[2]["max_abs_difference"] < 1e-4
    lines = []
    assert run_sft_generate_demo.main(["--steps", "10", "--checkpoint-path", str(tmp_path / "gen")], log=lines.append) == 0
    last = _records(lines)[-1]
    assert 0.0 <= last["rule_accuracy_before"] <= 1.0 and 0.0 <= last["rule_accuracy_after"] <= 1.0


def test_sft_http_demo_with_a_server_child(tmp_path):
    from arctic_platform_b200.sft.examples import run_sft_http_demo
    lines = []
    rc = run_sft_http_demo.main(["--launch-local-server", "--steps", "8", "--checkpoint-path", str(tmp_path / "ck")],
                                log=lines.append)
    last = json.loads(lines[-1])
    assert rc == 0 and last["improved"] and last["last_loss"] < last["first_loss"]
