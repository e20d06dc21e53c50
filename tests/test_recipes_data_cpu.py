"""Dataset preparation of the recipes (recipes/rl/data/prepare_data.py) with injected loaders -- no network -- and the
Ray start / stop helpers the multi-node script uses."""
import os

import pandas as pd
import pytest

from arctic_platform_b200.common import ray_cluster as rc
from recipes.rl.data import prepare_data as pd_mod


def test_gsm8k_answer_extraction():
    assert pd_mod.gsm8k_final_answer("a\nb\n#### 1,234") == "1234"
    assert pd_mod.gsm8k_final_answer("so #### -7.5") == "-7.5"
    with pytest.raises(ValueError):
        pd_mod.gsm8k_final_answer("no marker")


def test_gsm8k_rows_and_files(tmp_path):
    data = {"train": [{"question": f"q{i}?", "answer": f"work\n#### {i * 3}"} for i in range(5)],
            "test": [{"question": "t?", "answer": "#### 9"}]}
    calls = []

    def load(repo, name, split):
        calls.append((repo, name, split))
        return data[split]

    out = pd_mod.prepare_gsm8k(str(tmp_path / "g"), load=load)
    assert out == {"train": 5, "test": 1}
    assert calls == [("openai/gsm8k", "main", "train"), ("openai/gsm8k", "main", "test")]
    df = pd.read_parquet(tmp_path / "g" / "train.parquet")
    assert list(df.columns) == list(pd_mod.ROW_KEYS)
    row = df.iloc[2]
    assert row["reward_model"]["ground_truth"] == "6" and row["reward_model"]["style"] == "rule"
    assert row["prompt"][0]["role"] == "user" and row["prompt"][0]["content"].startswith("q2? Let's think")
    assert row["extra_info"]["index"] == 2 and row["extra_info"]["split"] == "train"
    # the reward function of the recipes scores the ground truth as written
    from recipes.rl.rewards.gsm8k_reward import gsm8k_reward
    assert gsm8k_reward("thinking... #### 6", row["reward_model"]["ground_truth"]) == 1.0


def test_long_context_rows_split_and_merge(tmp_path):
    def load(repo, name, split):
        assert repo == pd_mod.LOONGRL_REPO and split == "train"
        return [{"data_source": name, "prompt": [{"role": "user", "content": f"{name}-{i}"}], "ability": "qa",
                 "reward_model": {"style": "rule", "ground_truth": str(i)}, "extra_info": {"i": i}, "junk": 1}
                for i in range(10)]

    out = pd_mod.prepare_long_context_qa(str(tmp_path / "l"), test_ratio=0.2, seed=1, load=load)
    assert out["hotpotqa"] == {"train": 16, "test": 4}
    assert out["merged"] == {"train": 48, "test": 12}
    df = pd.read_parquet(tmp_path / "l" / "musique" / "train.parquet")
    assert "junk" not in df.columns
    msgs = df.iloc[0]["prompt"]
    assert msgs[0]["role"] == "system" and "\\boxed{" in msgs[0]["content"] and msgs[1]["role"] == "user"
    # the split is a partition and is reproducible
    a = pd_mod.split_rows(list(range(20)), 0.25, 7)
    b = pd_mod.split_rows(list(range(20)), 0.25, 7)
    assert a == b and sorted(a[0] + a[1]) == list(range(20)) and len(a[1]) == 5
    # an existing system prompt is kept
    kept = pd_mod.long_context_row({"prompt": [{"role": "system", "content": "mine"}, {"role": "user", "content": "x"}]})
    assert [m["content"] for m in kept["prompt"]] == ["mine", "x"]


def test_ray_start_commands(monkeypatch):
    monkeypatch.delenv("ARL_RAY_MIN_WORKER_PORT", raising=False)
    monkeypatch.delenv("ARL_RAY_MAX_WORKER_PORT", raising=False)
    assert rc.head_start_command(6379, 8265, "/tmp/x", 8) == \
        ["ray", "start", "--head", "--port=6379", "--dashboard-port=8265", "--temp-dir=/tmp/x", "--num-gpus=8"]
    monkeypatch.setenv("ARL_RAY_MIN_WORKER_PORT", "20000")
    monkeypatch.setenv("ARL_RAY_MAX_WORKER_PORT", "20100")
    assert rc.worker_start_command("h:6379", num_gpus=4) == \
        ["ray", "start", "--address=h:6379", "--num-gpus=4", "--min-worker-port=20000", "--max-worker-port=20100"]


def test_ray_cluster_cli(capsys, monkeypatch, tmp_path):
    monkeypatch.delenv("ARL_RAY_TEMP_DIR", raising=False)
    assert rc.main(["head", "--port", "7000", "--temp-dir", "/tmp/a b"]) == 0
    assert capsys.readouterr().out.strip() == "ray start --head --port=7000 '--temp-dir=/tmp/a b'"
    assert rc.main(["worker"]) == 2                       # no head address
    assert rc.main(["stop"]) == 2                         # no temp dir: nothing is ours to stop
    capsys.readouterr()
    # nothing on this machine runs with this temp dir, so nothing is stopped
    assert rc.main(["stop", "--temp-dir", str(tmp_path / "never-used")]) == 0
    assert capsys.readouterr().out.strip() == "0"


def test_launchers_are_valid_shell():
    import subprocess
    root = os.path.join(os.path.dirname(__file__), "..", "recipes", "rl")
    for rel in ("multi_node/restart_ray.sh", "verl/simple/run_qwen3_1p7b_gsm8k_grpo_baseline.sh",
                "verl/txt2sql/run_qwen3_32b_bird_grpo_baseline.sh",
                "verl/long_context_qa/run_qwen3_32b_loongrl_grpo_baseline.sh"):
        subprocess.run(["bash", "-n", os.path.join(root, rel)], check=True)


def test_skyrl_launcher_flags_become_platform_config():
    from recipes.rl.skyrl.arctic_backend import SkyRLArcticBackend
    from recipes.rl.skyrl.run_loop import build_parser
    a = build_parser().parse_args(["--data", "d", "--env", "e", "--sampler-tp", "4", "--sequence-parallel", "4", "--offload-optimizer"])
    assert (a.sampler_tp, a.sequence_parallel, a.offload_optimizer) == (4, 4, True)
    cfg = SkyRLArcticBackend.client_config("qwen3-32b", 32, 32, 32, sampler_tp=4, sequence_parallel=4, offload_optimizer=True,
                                           max_model_len=36864)
    assert cfg.ds_config["zero_optimization"] == {"stage": 3, "offload_optimizer": {"device": "cpu", "pin_memory": True}}
    assert cfg.ds_worker_config == {"zorro_train": {"enable": True}, "sequence_parallel": 4}
    assert cfg.vllm_config == {"max_model_len": 36864, "tensor_parallel_size": 4}
    plain = SkyRLArcticBackend.client_config("qwen3-tiny")
    assert "sequence_parallel" not in plain.ds_worker_config and "tensor_parallel_size" not in plain.vllm_config
    import subprocess
    root = os.path.join(os.path.dirname(__file__), "..", "recipes", "rl", "skyrl")
    for rel in ("txt2sql/run_qwen3_32b_bird_grpo_4node.sh", "long_context_qa/run_qwen3_32b_loongrl_grpo_4node.sh"):
        subprocess.run(["bash", "-n", os.path.join(root, rel)], check=True)
