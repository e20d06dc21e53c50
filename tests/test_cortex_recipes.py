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


# ------------------------------------------------------------------------------------------------- shared pieces
import dataclasses
from typing import Optional

import pytest

from cortex_client.recipes import common


class ChatTokenizer:
    """A chat template in miniature: ``<role>`` marker (1000 + role index), one token per character, end-of-turn 999;
    the generation prompt is the assistant marker."""
    ROLES = {"system": 1000, "user": 1001, "assistant": 1002}

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=False):
        ids = []
        for m in messages:
            ids += [self.ROLES[m["role"]]] + [ord(c) for c in m["content"]] + [999]
        return ids + ([1002] if add_generation_prompt else [])

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(i) for i in ids if i < 999)


def test_overrides_are_typed_and_checked():
    @dataclasses.dataclass
    class S:
        lr: float = 1e-5
        steps: int = 10
        name: str = "x"
        flag: bool = False
        path: Optional[str] = None
        tags: list = dataclasses.field(default_factory=list)

    s = common.apply_overrides(S(), ["lr=3e-4", "steps=7", "name=Qwen/Qwen3-8B", "flag=yes", "path=/tmp/a=b", "tags=[1, 2]"])
    assert (s.lr, s.steps, s.name, s.flag, s.path, s.tags) == (3e-4, 7, "Qwen/Qwen3-8B", True, "/tmp/a=b", [1, 2])
    assert common.apply_overrides(s, ["path=none"]).path is None
    for bad, needle in (["stepz=1"], "unknown setting"), (["steps=1.5"], "steps"), (["flag=maybe"], "flag"), (["steps"], "key=value"):
        with pytest.raises(ValueError, match=needle):
            common.apply_overrides(S(), bad)


def test_chat_rendering_puts_the_loss_on_assistant_turns():
    tok = ChatTokenizer()
    msgs = [{"role": "system", "content": "s"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"},
            {"role": "user", "content": "q"}, {"role": "assistant", "content": "a"}]
    ids, mask = common.render_chat(msgs, tok)
    assert ids == tok.apply_chat_template(msgs)
    on = [t for t, m in zip(ids, mask) if m]
    assert on == [ord("y"), ord("o"), 999, ord("a"), 999]               # contents and end-of-turn, not the role markers
    ids2, mask2 = common.render_chat(msgs, tok, max_length=9)
    assert len(ids2) == 9 and ids2 == ids[:9] and mask2 == mask[:9]
    with pytest.raises(ValueError):
        common.render_chat([], tok)


def test_boxed_answers_and_the_math_reward():
    assert common.boxed_answer(r"so \boxed{1} then \boxed{\frac{3}{4}}.") == r"\frac{3}{4}"
    assert common.boxed_answer("no box") is None and common.boxed_answer(r"\boxed{unclosed") is None
    assert common.math_reward(r"... \boxed{ 1,234 }", "1234") == 1.0
    assert common.math_reward(r"\boxed{\dfrac{6}{8}}", r"\boxed{\frac{3}{4}}") == 1.0
    assert common.math_reward(r"\boxed{0.50}", "1/2") == 0.0 and common.math_reward(r"\boxed{2.0}", "2") == 1.0
    assert common.math_reward(r"\boxed{\text{yes}}", "yes") == 1.0
    assert common.math_reward("I think 4", "4", format_penalty=0.1) == -0.1


def test_metrics_logger_writes_config_and_lines(tmp_path):
    seen = []
    lg = common.MetricsLogger(str(tmp_path / "run"), {"lr": 1e-5}, wandb_project=None, echo=seen.append)
    lg.log(0, {"loss": 1.5})
    lg.log(1, {"loss": torch.tensor(1.25)})
    lg.close()
    assert json.loads((tmp_path / "run" / "config.json").read_text()) == {"lr": 1e-5}
    lines = [json.loads(x) for x in (tmp_path / "run" / "metrics.jsonl").read_text().splitlines()]
    assert [x["step"] for x in lines] == [0, 1] and lines[1]["loss"] == 1.25 and len(seen) == 2


def test_sft_settings_form_with_chat_rows_and_accumulation(tmp_path):
    data = tmp_path / "chat.jsonl"
    conv = lambda a: {"messages": [{"role": "user", "content": "hello"}, {"role": "assistant", "content": a}]}
    data.write_text("\n".join(json.dumps(conv(a)) for a in ("abc", "de", "f", "ghij")))
    st = common.apply_overrides(sft_loop.SFTSettings(), [f"data={data}", "url=http://svc", "steps=2", "batch_size=4",
                                                         "micro_batch_size=1", "n_gpus=2", "lora_rank=16", "max_length=64",
                                                         f"log_path={tmp_path / 'log'}", "model_name=qwen3-4b"])
    rows = sft_loop.tokenize_rows(sft_loop.read_rows(str(data)), ChatTokenizer(), 64)
    assert [t for t in rows[0]["labels"] if t != -100] == [ord("a"), ord("b"), ord("c"), 999]
    s = FakeServiceSession()
    hist = sft_loop.run(_client(s), st.model_name, st.data, st.steps, st.batch_size, st.n_gpus, st.learning_rate,
                        micro_batch_size=st.micro_batch_size, max_length=st.max_length, tokenizer=ChatTokenizer(),
                        extra=st.training_extra(), max_seq_len=st.max_length,
                        logger=common.MetricsLogger(st.log_path, dataclasses.asdict(st), echo=None))
    ops = [c[1].rsplit("/", 1)[-1] for c in s.calls if c[0] == "POST" and c[1].count("/") == 3]
    assert ops == ["forward_backward", "forward_backward", "step"] * 2               # 4 rows in slices of 1 x 2 GPUs
    body = next(iter(s.jobs.values()))["body"]["sub_jobs"][0]
    assert body["lora_rank"] == 16 and body["max_seq_len"] == 64 and body["num_devices"] == 2
    assert hist[0]["loss_tokens"] == 4 + 3 + 2 + 5 and hist[0]["train_mean_nll"] == 0.25
    assert len((tmp_path / "log" / "metrics.jsonl").read_text().splitlines()) == 2
    with pytest.raises(ValueError, match="multiple"):
        common.apply_overrides(st, ["batch_size=5"]).validate()
    with pytest.raises(ValueError, match="ep_size"):
        common.apply_overrides(st, ["ep_size=4", "n_gpus=6", "micro_batch_size=0"]).validate()


def test_rl_settings_form_with_text_rows_and_held_out_eval(tmp_path):
    tok = ChatTokenizer()
    pf, ef = tmp_path / "p.jsonl", tmp_path / "e.jsonl"
    pf.write_text("\n".join(json.dumps({"prompt": f"what is {i}+{i}?", "answer": str(2 * i)}) for i in range(4)))
    ef.write_text(json.dumps({"messages": [{"role": "user", "content": "1+1?"}], "answer": "2"}))
    rows = rl_loop.prepare_rows(rl_loop.read_rows(str(pf)), tok)
    assert rows[0]["prompt_ids"][0] == 1001 and rows[0]["prompt_ids"][-1] == 1002           # ends with the generation prompt
    reward = rl_loop.make_reward(tok)
    boxed = [ord(c) for c in r"so \boxed{0}"]
    assert reward(boxed, rows[0]) == 1.0 and reward(boxed, rows[1]) == 0.0
    assert reward([1, 2], {"answer_ids": [1, 2]}) == 1.0
    s = FakeServiceSession()
    st = common.apply_overrides(rl_loop.RLSettings(), [f"prompts={pf}", f"eval_prompts={ef}", "steps=2", "prompts_per_step=2",
                                                      "group_size=2", "max_tokens=4", "max_seq_len=64", "eval_every=2",
                                                      "training_gpus=2", "sampling_gpus=1", "lora_rank=8",
                                                      f"log_path={tmp_path / 'log'}", "model_name=qwen3-4b"])
    hist = rl_loop.run_settings(st, client=_client(s), tokenizer=tok, echo=None)
    assert "eval/reward_mean" not in hist[0] and hist[1]["eval/prompts"] == 1 and "prompts_solved" in hist[0]
    body = next(iter(s.jobs.values()))["body"]["sub_jobs"]
    assert body[0]["lora_rank"] == 8 and body[0]["num_devices"] == 2 and body[1]["num_devices"] == 1
    assert body[1]["vllm_config"]["max_model_len"] == 64
    ops = [c[1].rsplit("/", 1)[-1] for c in s.calls if c[0] == "POST" and c[1].count("/") == 3]
    assert ops.count("generate") == 3                                                   # two training steps + one eval
    with pytest.raises(ValueError, match="do not fit"):
        rl_loop.run_settings(common.apply_overrides(st, ["max_seq_len=10"]), client=_client(s), tokenizer=tok, echo=None)
    with pytest.raises(ValueError, match="tokenizer"):
        rl_loop.prepare_rows([{"prompt": "x"}], None)
