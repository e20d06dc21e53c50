"""Tensor-parallel sampling replica on two gloo ranks against the single-rank engine: same greedy tokens, same
log-probs, half the K/V bytes per rank, whole-model weight norm, weights replaced through the sliced load."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.parallel.tp_sampler import shard_axis, tp_config, tp_slice


def test_shard_axes_and_shapes():
    assert shard_axis("model.layers.0.self_attn.q_proj.weight") == 0
    assert shard_axis("model.layers.0.self_attn.o_proj.weight") == 1
    assert shard_axis("model.layers.3.mlp.experts.5.down_proj.weight") == 1
    assert shard_axis("model.layers.3.mlp.shared_expert.up_proj.weight") == 0
    for replicated in ("model.layers.3.mlp.gate.weight", "model.layers.3.mlp.shared_expert_gate.weight",
                       "model.embed_tokens.weight", "model.layers.0.self_attn.q_norm.weight", "lm_head.weight",
                       "model.layers.0.input_layernorm.weight"):
        assert shard_axis(replicated) is None
    cfg = PRESETS["qwen3-moe-tiny"]
    local = tp_config(cfg, 2)
    assert (local.num_heads, local.num_kv_heads, local.moe_intermediate_size) == (2, 1, 64) and local.hidden_size == cfg.hidden_size
    t = torch.arange(24.0).view(6, 4)
    assert torch.equal(tp_slice("model.layers.0.mlp.down_proj.weight", t, cfg, 1, 2), t[:, 2:])
    assert torch.equal(tp_slice("model.layers.0.self_attn.k_proj.weight", t, cfg, 0, 3), t[:2])
    assert tp_slice("model.norm.weight", t, cfg, 1, 2) is t
    with pytest.raises(ValueError, match="does not divide"):
        tp_config(cfg, 3)
    with pytest.raises(NotImplementedError):
        tp_config(PRESETS["qwen3.5-moe-tiny"], 2)


def _rank_main(rank, world, port, out_dir, preset):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arctic_platform_b200.engine.hybrid_sampler import HybridSampler
        from arctic_platform_b200.models.decoder import DecoderLM
        from arctic_platform_b200.models.hf_io import iter_hf_tensors
        from arctic_platform_b200.parallel.tp_sampler import TensorParallelSampler
        cfg = PRESETS[preset]
        full = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=4)
        other = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=8)
        one = HybridSampler(cfg, "cpu", model=full, max_seq_len=128)
        tp = TensorParallelSampler(cfg, "cpu", model=full, max_seq_len=128)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 12, 8)]
        greedy = {"n": 1, "temperature": 0.0, "max_tokens": 10}
        res = {"one": one.generate(prompts, greedy), "tp": tp.generate(prompts, greedy),
               "norm_one": one.weight_norm(), "norm_tp": tp.weight_norm(), "kv_one": one.kv_bytes(), "kv_tp": tp.kv_bytes()}
        # every rank seeds its generator differently: the drawn tokens still agree (rank 0 of the group decides)
        res["sampled"] = tp.generate(prompts, {"n": 2, "temperature": 1.0, "max_tokens": 6, "seed": 100 + rank})
        tp.load_weights(iter_hf_tensors(other))
        res["tp_other"] = tp.generate(prompts, greedy)
        res["one_other"] = HybridSampler(cfg, "cpu", model=other, max_seq_len=128).generate(prompts, greedy)
        torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("preset", ["qwen3-tiny", "qwen3-moe-tiny"])
def test_two_rank_replica_equals_one_rank(preset):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank_main, args=(2, port, d, preset), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"r{r}.pt"), weights_only=False) for r in range(2)]
    for r in res:
        assert [x["token_ids"] for x in r["tp"]] == [x["token_ids"] for x in r["one"]]
        for a, b in zip(r["tp"], r["one"]):
            assert a["logprobs"] == pytest.approx(b["logprobs"], abs=2e-4)
        assert r["norm_tp"]["num_params"] == r["norm_one"]["num_params"]
        assert r["norm_tp"]["norm"] == pytest.approx(r["norm_one"]["norm"], rel=1e-9)
        assert r["kv_tp"] * 2 == r["kv_one"]
        assert [x["token_ids"] for x in r["tp_other"]] == [x["token_ids"] for x in r["one_other"]]
    assert [x["token_ids"] for x in res[0]["sampled"]] == [x["token_ids"] for x in res[1]["sampled"]]
    assert res[0]["sampled"][0]["logprobs"] == res[1]["sampled"][0]["logprobs"]


@pytest.mark.timeout(600)
def test_tensor_parallel_replica_behind_the_server():
    """Two rank processes host a two-rank trainer and ONE two-rank sampling replica: the server calls both ranks of
    the replica together, the trainer's weights reach the shards, and the rollouts are those of a one-rank sampler
    with the same weights."""
    from arctic_platform_b200.common.server import ArcticRLServerCore, JobError
    from arctic_platform_b200.engine.worker import EngineWorker
    from tests.test_server_multirank_spawn_cpu import _job, _train
    core = ArcticRLServerCore(training_gpus=2, sampling_gpus=2, colocate=True)
    try:
        tj = core.initialize(_job(1))["job_id"]
        with pytest.raises(JobError, match="does not divide"):
            core.initialize({"model_name": "qwen3-tiny", "job_type": "sampling", "num_devices": 3,
                             "vllm_config": {"tensor_parallel_size": 2}})
        sj = core.initialize({"model_name": "qwen3-tiny", "job_type": "sampling", "seed": 5,
                              "vllm_config": {"max_model_len": 64, "tensor_parallel_size": 2}})["job_id"]
        assert len(core._replicas(core._job(sj))) == 1
        _train(core, tj, steps=1)
        core.weight_sync(tj, [sj])
        tn = core.weight_norm(training_job_id=tj)
        sn = core.weight_norm(sampling_job_id=sj)
        assert sn["sampling_norm"] == pytest.approx(tn["training_norm"], rel=1e-6)
        assert sn["sampling_num_params"] == tn["training_num_params"]
        prompts = [[3, 4, 5, 9], [6, 7]]
        greedy = {"n": 1, "max_tokens": 5, "temperature": 0.0}
        out = core.generate(sj, prompts, greedy)["results"]
        scores = core.log_probs(sj, prompts, [r["token_ids"] for r in out])["log_probs"]
        for r, s in zip(out, scores):
            assert s == pytest.approx(r["logprobs"], abs=2e-4)          # scoring == what sampling reported
        # a plain one-rank sampler given the trainer's weights draws the same tokens
        weights = call_all_first(core, tj)
        solo = EngineWorker("cpu")
        solo.initialize({"model_name": "qwen3-tiny", "job_type": "sampling", "seed": 5, "vllm_config": {"max_model_len": 64}})
        solo.load_weights(weights)
        want = solo.generate(prompts, greedy)
        assert [r["token_ids"] for r in out] == [r["token_ids"] for r in want]
    finally:
        core.destroy()


def call_all_first(core, job_id):
    from arctic_platform_b200.common.server import call_all
    return call_all(core._job(job_id).workers, "get_weights", None, 0)[0]
