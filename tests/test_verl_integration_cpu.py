"""verl plugin on CPU: config mapping, padding helpers, the adapter's call sequence against a recording fake,
and one real update through the in-process client with the tiny model."""
import asyncio

import pytest
import torch

from arctic_platform_b200.integrations.verl import (ArcticRLClientWrapper, cfg_get, no_padding_to_padded_prompt_response,
                                                    prepare_padded_batch)
from arctic_platform_b200.integrations.verl import register
from arctic_platform_b200.integrations.verl.rollout import ArcticLLMServer, ArcticReplica, RolloutMode
from arctic_platform_b200.integrations.verl.worker import ArcticRLActorRolloutRefWorker, estimate_flops_per_token
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def _config(**over):
    cfg = {
        "data": {"train_batch_size": 4, "max_prompt_length": 16, "max_response_length": 8},
        "trainer": {"seed": 7},
        "actor_rollout_ref": {
            "model": {"path": "qwen3-tiny", "enable_gradient_checkpointing": False},
            "rollout": {"n": 2, "temperature": 1.0},
            "actor": {"ppo_mini_batch_size": 2, "ppo_micro_batch_size_per_gpu": 2, "ppo_epochs": 2,
                      "optim": {"lr": 1e-3}, "grad_clip": 1.0, "fsdp_config": {"ulysses_sequence_parallel_size": 1}},
        },
        "remote_backend": {"colocate": True, "training_gpus": 1, "sampling_gpus": 0, "log_prob_gpus": 1,
                           "comm_protocol": "local", "weight_sync": {"cuda_ipc": False},
                           "train": {"zorro_train": {"enable": True, "max_rollouts": 2},
                                     "deepspeed": {"zero_optimization": {"stage": 2}, "data_types": {"grad_accum_dtype": "fp32"}}}},
    }
    for k, v in over.items():
        node = cfg
        *path, last = k.split(".")
        for p in path:
            node = node[p]
        node[last] = v
    return cfg


class _Obj:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def test_cfg_get_reads_dicts_and_objects():
    cfg = {"a": _Obj(b={"c": 3}, n=None)}
    assert cfg_get(cfg, "a.b.c") == 3 and cfg_get(cfg, "a.x.y", 5) == 5 and cfg_get(cfg, "a.n", 9) == 9
    with pytest.raises(KeyError):
        cfg_get(cfg, "a.b.missing")


def test_jagged_to_padded():
    vals = torch.arange(1, 12)
    pl, rl = torch.tensor([2, 3, 1]), torch.tensor([1, 2, 2])
    dense, P, R = no_padding_to_padded_prompt_response(vals, pl, rl, pad_value=0)
    assert (P, R) == (3, 2)
    assert dense.tolist() == [[0, 1, 2, 3, 0], [4, 5, 6, 7, 8], [0, 0, 9, 10, 11]]
    b, P2, R2 = prepare_padded_batch({"input_ids": vals, "prompt_lens": pl, "response_lens": rl, "max_prompt_len": 4}, 99)
    assert (P2, R2) == (4, 2) and b["input_ids"][0].tolist() == [99, 99, 1, 2, 3, 99] and b["attention_mask"][0].tolist() == [0, 0, 1, 1, 1, 0]
    with pytest.raises(ValueError):
        no_padding_to_padded_prompt_response(vals[:-1], pl, rl)


class _FakeClient:
    def __init__(self):
        self.calls = []
        self.job_ids = {"training": 1, "sampling": 2, "log_prob": 3}

    def call(self, name, *a, **kw):
        self.calls.append((name, a, kw))
        if name in ("fwd_no_grad",):
            B, S = a[0]["batch"]["input_ids"].shape
            R = a[0]["meta"]["response_length"]
            return {"batch": {"log_probs": torch.zeros(B, R), "entropy": torch.ones(B, R)}}
        if name == "fwd_bwd":
            return {"metrics": {"actor/pg_loss": 0.5}, "avg_loss": 0.5}
        if name == "step":
            return {"metrics": {"grad_norm": 2.0, "last_lr": 1e-3}}
        if name == "generate":
            return [{"outputs": [{"token_ids": [7, 8, 9], "finish_reason": "length"}]} for _ in a[0]]
        return {"status": "ok"}


def test_adapter_call_sequence_and_ds_config():
    fake = _FakeClient()
    w = ArcticRLClientWrapper(_config(), client=fake)
    ds = w.client_config.ds_config
    assert ds["train_batch_size"] == 4 and ds["gradient_accumulation_steps"] == 2 and ds["train_micro_batch_size_per_gpu"] == 2
    assert ds["optimizer"]["params"]["lr"] == 1e-3 and ds["gradient_clipping"] == 1.0 and ds["zero_optimization"]["stage"] == 2
    assert "data_types" not in w.client_config.log_prob_ds_config and "data_types" in ds
    assert w.client_config.ds_worker_config["zorro_train"] == {"enable": True, "max_rollouts": 2}
    assert w.requires_single_forwarder
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=2)
    data = {"input_ids": ids, "attention_mask": mask, "responses": ids[:, -R:], "advantages": torch.randn(8, R)}
    lp = w.compute_log_prob(data, calculate_entropy=True)
    assert lp["old_log_probs"].shape == (8, R) and lp["entropys"].shape == (8, R)
    assert w.compute_ref_log_prob(data)["ref_log_prob"].shape == (8, R) and fake.calls[-1][2] == {"reference_model": True}
    data["old_log_probs"] = lp["old_log_probs"]
    fake.calls.clear()
    m = w.update_actor(data)
    names = [c[0] for c in fake.calls]
    assert names == ["fwd_bwd", "step"] * 4                        # 2 epochs x 2 mini-batches of (2 prompts x 2 rollouts)
    assert fake.calls[0][1][0]["batch"]["input_ids"].shape[0] == 4 and fake.calls[0][1][0]["meta"]["zorro_train_enable"]
    assert m["actor/pg_loss"] == 0.5 and m["grad_norm"] == 2.0 and w.global_steps == 1
    out = w.generate([[1, 2], [3]], {"max_tokens": 3})
    assert len(out) == 2 and fake.calls[-1][1][1]["max_tokens"] == 3 and fake.calls[-1][1][1]["temperature"] == 1.0
    w.update_weights()
    w.sleep_inference(2)
    w.wake_up_inference(["weights"])
    assert [c[0] for c in fake.calls[-3:]] == ["sync_weights", "sleep_inference", "wake_inference"]
    with pytest.raises(ValueError):
        ArcticRLClientWrapper(_config(**{"data.train_batch_size": 3}), client=fake)


def test_rollout_server_and_registry():
    fake = _FakeClient()
    w = ArcticRLClientWrapper(_config(**{"remote_backend.sampling_gpus": 2}), client=fake)
    rep = asyncio.run(ArcticReplica(0, w, RolloutMode.HYBRID).init())
    srv: ArcticLLMServer = rep.server_handle
    out = asyncio.run(srv.generate([1, 2, 3], {"max_new_tokens": 5}, request_id="r1"))
    assert out.token_ids == [7, 8, 9] and out.stop_reason == "length" and fake.calls[-1][1][1]["max_tokens"] == 5
    assert out.routed_experts is None and "return_routed_experts" not in fake.calls[-1][1][1]
    replay = asyncio.run(ArcticReplica(1, w, RolloutMode.HYBRID, enable_rollout_routing_replay=True).init()).server_handle
    asyncio.run(replay.generate([1, 2, 3], {"max_new_tokens": 5}))
    assert fake.calls[-1][1][1]["return_routed_experts"] is True      # the sampler is asked for its expert choices
    asyncio.run(srv.sleep())
    asyncio.run(srv.sleep())                                        # idempotent
    asyncio.run(srv.wake_up())
    assert [c[0] for c in fake.calls[-2:]] == ["sleep_inference", "wake_inference"] and rep.world_size == 2
    assert register.STATUS["local"] and register.resolve("backend") is ArcticRLClientWrapper
    assert register.resolve("worker") is ArcticRLActorRolloutRefWorker and register.config_search_path().endswith("config")
    with pytest.raises(KeyError):
        register.resolve("backend", "other")


def test_real_update_through_local_client(tmp_path):
    cfg = _config(**{"actor_rollout_ref.actor.ppo_epochs": 1, "data.train_batch_size": 2})
    cfg["trainer"]["default_local_dir"] = str(tmp_path)
    worker = ArcticRLActorRolloutRefWorker(cfg, peak_tflops=1.0)
    worker.init_model()
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2)
    data = {"input_ids": ids, "attention_mask": mask, "responses": ids[:, -R:],
            "advantages": torch.randn(4, 1).expand(4, R).contiguous()}
    lp = worker.compute_log_prob(data)
    assert lp["old_log_probs"].shape == (4, R) and lp["metrics"]["perf/tokens_per_s"] > 0
    data["old_log_probs"] = lp["old_log_probs"]
    out = worker.update_actor(data)["metrics"]
    assert out["grad_norm"] > 0 and "actor/pg_loss" in out and out["perf/tflops"] > 0 and "perf/mfu" in out
    # the same batch in verl's padding-free layout: nested rows in, nested rows out, each value on its predicting token
    lens = mask.sum(1)
    P = ids.shape[1] - R
    rows = [ids[b][mask[b].bool()] for b in range(4)]
    pl = mask[:, :P].sum(1)
    nested = {"input_ids": torch.nested.nested_tensor(rows, layout=torch.jagged),
              "prompts": torch.nested.nested_tensor([r[:int(p)] for r, p in zip(rows, pl)], layout=torch.jagged),
              "responses": torch.nested.nested_tensor([r[int(p):] for r, p in zip(rows, pl)], layout=torch.jagged),
              "max_prompt_len": P, "max_response_len": R}
    dense_ref = worker.compute_ref_log_prob(data)["ref_log_prob"]
    got = worker.compute_ref_log_prob(nested)["ref_log_prob"]
    assert got.is_nested and torch.equal(got.offsets().diff(), lens)
    for b, row in enumerate(got.unbind()):
        p, r = int(pl[b]), int(lens[b] - pl[b])
        torch.testing.assert_close(row[p - 1:p - 1 + r], dense_ref[b, :r], rtol=1e-4, atol=1e-5)
        assert float(row[:p - 1].abs().sum()) == 0.0
    assert worker.compute_log_prob(nested)["metrics"]["perf/tokens_per_s"] > 0
    assert worker.to("cpu") is None and worker.set_loss_fn(None) is None and worker.reset() is None
    handle = worker.reconnect_handle()
    again = ArcticRLClientWrapper.from_config(cfg, handle={**handle})   # attaches: no new jobs
    assert again.client_config.training_job_id == handle["job_ids"]["training"]
    from arctic_platform_b200.models.config import PRESETS
    assert estimate_flops_per_token(PRESETS["qwen3-4b"], 4096) > 6 * 3.5e9
    worker.destroy()
    assert worker.wrapper is None


def test_rollout_endpoint_protocol_details():
    """Token budget resolution, log-prob flag, verl's stop vocabulary, per-mode sleep / wake and the hybrid weight
    hand-over order."""
    from arctic_platform_b200.integrations.verl.rollout import (RolloutServerConfig, resolve_max_tokens,
                                                                verl_stop_reason)
    cfg = RolloutServerConfig(max_model_len=16, prompt_length=8, response_length=6)
    assert resolve_max_tokens({"max_tokens": 100}, 4, cfg) == 12          # clamped to the context space
    assert resolve_max_tokens({"max_new_tokens": 3}, 4, cfg) == 3
    assert resolve_max_tokens({}, 4, cfg) == 10                           # response + prompt budget - prompt
    with pytest.raises(ValueError, match="exceeds the model's maximum context length"):
        resolve_max_tokens({}, 17, cfg)
    assert resolve_max_tokens({}, 4, RolloutServerConfig()) == -1         # nothing configured: engine default
    assert [verl_stop_reason(r) for r in ("abort", "stop", "length", "other", None)] == \
        ["aborted", "completed", "completed", "other", None]
    assert RolloutServerConfig.from_verl({"response_length": 5, "free_cache_engine": False}).free_cache_engine is False

    fake = _FakeClient()
    w = ArcticRLClientWrapper(_config(), client=fake)
    rep = asyncio.run(ArcticReplica(0, w, RolloutMode.COLOCATED, config=cfg, nnodes=2).init())
    assert len(rep.servers) == 2 and not rep.rollout_worker_use_gpu()
    srv = rep.server_handle.use_verl_stop_reasons()
    out = asyncio.run(srv.generate([1, 2, 3], {"logprobs": True}, request_id="a"))
    sent = fake.calls[-1][1][1]
    assert sent["max_tokens"] == 11 and sent["logprobs"] == 0 and out.stop_reason == "completed"
    assert out.finish_reason == "length" and out.extra["global_steps"] == 0
    # colocated: sleep, then wake restores weights + cache and resets cached prefixes; node 1 never touches the engine
    n0 = len(fake.calls)
    asyncio.run(rep.servers[1].sleep())
    asyncio.run(rep.servers[1].wake_up())
    assert len(fake.calls) == n0
    asyncio.run(srv.sleep())
    asyncio.run(srv.wake_up())
    assert [c[0] for c in fake.calls[n0:]] == ["sleep_inference", "wake_inference", "reset_prefix_cache"]
    assert fake.calls[n0 + 1][1][0] == ["kv_cache", "weights"]
    # hybrid hand-over: weights while asleep, then the cache, then the prefix reset
    hyb = asyncio.run(ArcticReplica(1, w, RolloutMode.HYBRID).init()).server_handle
    asyncio.run(hyb.sleep())
    n1 = len(fake.calls)
    asyncio.run(hyb.update_weights(global_steps=7))
    assert [c[0] for c in fake.calls[n1:]] == ["sync_weights", "wake_inference", "reset_prefix_cache"]
    assert fake.calls[n1 + 1][1][0] == ["kv_cache"] and hyb.global_steps == 7
    # standalone and free_cache_engine=False: sleep / wake are no-ops
    n2 = len(fake.calls)
    alone = ArcticLLMServer(w, RolloutMode.STANDALONE)
    keep = ArcticLLMServer(w, RolloutMode.HYBRID, config=RolloutServerConfig(free_cache_engine=False))
    for s_ in (alone, keep):
        asyncio.run(s_.sleep())
        asyncio.run(s_.wake_up())
    assert len(fake.calls) == n2
    assert asyncio.run(rep.abort_request("a"))["aborted"] is False


def test_update_actor_detailed_meta_and_reductions():
    fake = _FakeClient()
    w = ArcticRLClientWrapper(_config(), client=fake)
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=2)
    data = {"input_ids": ids, "attention_mask": mask, "responses": ids[:, -R:], "advantages": torch.randn(8, R),
            "old_log_probs": torch.zeros(8, R), "rollout_is_weights": torch.arange(8.0)[:, None].expand(8, R)}
    out = w.update_actor_detailed(data)
    assert set(out) == {"loss", "metrics", "global_token_num"} and len(out["global_token_num"]) == 8
    assert out["global_token_num"] == mask.sum(-1).tolist()
    first = fake.calls[0][1][0]["meta"]
    assert first["global_batch_size"] == 4 and first["batch_num_tokens"] == int(first_mask_tokens(fake))
    assert first["rollout_is_weights"].shape[0] == 4 and float(first["rollout_is_weights"][3, 0]) == 3.0
    second = [c for c in fake.calls if c[0] == "fwd_bwd"][1][1][0]["meta"]
    assert float(second["rollout_is_weights"][0, 0]) == 4.0          # the chunk's own slice
    assert isinstance(first["actor_config"], dict) and first["actor_config"].get("ppo_epochs") == 2
    assert out["metrics"]["actor/pg_loss"] == 0.5 and "lr" not in out["metrics"] or isinstance(out["metrics"]["lr"], float)


def first_mask_tokens(fake):
    return fake.calls[0][1][0]["batch"]["response_mask"].sum()
