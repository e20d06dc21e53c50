"""Two data-parallel ranks as spawned worker processes behind the job server (gloo): the server dispatches to all
ranks at once (the ranks meet in collectives inside initialize / forward / step), the ranks form their process
group from the launcher's environment, and the result equals one process training on the whole batch.  Stage 3
adds gathers inside the forward pass and a weight hand-over that needs every source rank."""
import socket

import pytest
import torch

from arctic_platform_b200.common.local_actors import spawned_worker_factory
from arctic_platform_b200.common.server import ArcticRLServerCore, call_all
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _job(stage):
    return {"model_name": "qwen3-tiny", "job_type": "training", "seed": 11,
            "ds_config": {"zero_optimization": {"stage": stage}, "gradient_clipping": 1.0,
                          "optimizer": {"type": "AdamW", "params": {"lr": 1e-3, "weight_decay": 0.01}}}}


def _payload():
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=2, seed=3)
    B = ids.shape[0]
    g = torch.Generator().manual_seed(1)
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:],
             "old_log_probs": torch.randn(B, R, generator=g) * 0.01 - 2.0,
             "advantages": torch.randn(B, 1, generator=g).expand(B, R).contiguous()}
    meta = {"response_length": R, "zorro_train_enable": True, "batch_num_tokens": float(mask[:, -R:].sum()),
            "global_batch_size": float(B)}
    return {"batch": batch, "meta": meta, "processing": {"loss_fn": "verl_grpo"}}


def _train(core, job_id, steps=2):
    out = []
    for _ in range(steps):
        r = core.forward_backward(job_id, _payload())
        s = core.step(job_id)
        out.append((r["avg_loss"], s["metrics"]["grad_norm"]))
    return out


@pytest.mark.timeout(600)
@pytest.mark.parametrize("stage", [1, 3])
def test_two_spawned_ranks_match_one_process(stage):
    single = ArcticRLServerCore()
    j1 = single.initialize(_job(stage))["job_id"]
    want = _train(single, j1)
    want_norm = single.weight_norm(training_job_id=j1)["training_norm"]

    core = ArcticRLServerCore(worker_factory=spawned_worker_factory(_free_port()), training_gpus=2)
    try:
        info = core.initialize(_job(stage))
        assert info["num_devices"] == 2
        job = core.jobs[info["job_id"]]
        ranks = call_all(job.workers, "rank_info")
        assert [r["rank"] for r in ranks] == [0, 1] and all(r["world"] == 2 and r["process_group"] for r in ranks)
        assert all(r["zero3"] == (stage == 3) for r in ranks)
        got = _train(core, info["job_id"])
        for (la, na), (lb, nb) in zip(got, want):
            assert la == pytest.approx(lb, rel=1e-4, abs=1e-6) and na == pytest.approx(nb, rel=1e-4)
        norms = [r["norm"] for r in call_all(job.workers, "weight_norm")]      # stage 3: a collective
        assert core.weight_norm(training_job_id=info["job_id"])["training_norm"] == pytest.approx(norms[0], rel=1e-7)
        assert norms[0] == pytest.approx(norms[1], rel=1e-7) and norms[0] == pytest.approx(want_norm, rel=1e-5)
        # hand the trained weights to a sampler job (its own process, no process group)
        sj = core.initialize({"model_name": "qwen3-tiny", "job_type": "sampling", "num_devices": 1, "seed": 5,
                              "vllm_config": {"max_model_len": 64}})
        before = core.weight_norm(sampling_job_id=sj["job_id"])["sampling_norm"]
        res = core.weight_sync(info["job_id"], [sj["job_id"]])
        assert res["strategies"] == (["gather_bulk"] if stage == 3 else ["bulk"])
        after = core.weight_norm(sampling_job_id=sj["job_id"])["sampling_norm"]
        assert after == pytest.approx(norms[0], rel=1e-6) and after != pytest.approx(before, rel=1e-6)
        out = core.generate(sj["job_id"], [[3, 4, 5]], {"n": 2, "max_tokens": 3, "temperature": 1.0})
        assert len(out["results"]) == 2
    finally:
        core.destroy()
        single.destroy()


def test_call_all_runs_workers_concurrently_and_reports_the_first_failure():
    import threading
    import time
    barrier = threading.Barrier(3, timeout=5)

    class W:
        def __init__(self, i):
            self.i = i

        def call(self, method, *args):
            if method == "meet":
                barrier.wait()                       # passes only if all three calls are in flight together
                return (self.i,) + args
            if method == "boom" and self.i == 1:
                raise ValueError("rank 1 failed")
            time.sleep(0.05)
            return self.i

    ws = [W(i) for i in range(3)]
    assert call_all(ws, "meet", None, "x") == [(0, "x"), (1, "x"), (2, "x")]
    barrier.reset()
    assert call_all(ws, "meet", [(10,), (11,), (12,)]) == [(0, 10), (1, 11), (2, 12)]
    with pytest.raises(ValueError, match="rank 1"):
        call_all(ws, "boom")
    assert call_all(ws[:1], "other") == [0]


@pytest.mark.timeout(600)
def test_rank_process_pool_hosts_trainer_and_sampler_of_a_rank_together():
    """The server's default for more than one rank per job: one process per rank hosting that rank's engines of
    every job.  Stage-3 trainer + log-prob engine + sampler replicas share the processes; the weight hand-over runs
    inside each rank process on all ranks at once."""
    core = ArcticRLServerCore(training_gpus=2, sampling_gpus=2, log_prob_gpus=2, colocate=True)
    assert core.pool is not None and core.pool.world == 2
    try:
        tj = core.initialize(_job(3))["job_id"]
        lj = core.initialize({**_job(3), "job_type": "log_prob"})["job_id"]
        sj = core.initialize({"model_name": "qwen3-tiny", "job_type": "sampling", "seed": 5,
                              "vllm_config": {"max_model_len": 64}})["job_id"]
        assert len(core.pool.actors) == 2                       # three jobs, still two processes
        assert sorted(k.split("-")[0] for k in core.pool.actors[0].call("keys")) == ["log_prob", "sampling", "training"]
        got = _train(core, tj, steps=1)
        assert got[0][1] > 0
        res = core.weight_sync(tj, [sj, lj])
        assert res["strategies"] == ["in_process"]
        tn = core.weight_norm(training_job_id=tj)["training_norm"]
        assert core.weight_norm(sampling_job_id=sj)["sampling_norm"] == pytest.approx(tn, rel=1e-6)
        # the log-prob engine scores with the synced weights: same log-probs as the trainer's own forward
        p = _payload()
        a = core.forward(tj, {"batch": p["batch"], "meta": p["meta"]})["batch"]["log_probs"]
        b = core.forward(lj, {"batch": p["batch"], "meta": p["meta"]})["batch"]["log_probs"]
        assert torch.allclose(a, b, atol=1e-5)
        out = core.generate(sj, [[3, 4, 5], [6, 7]], {"n": 2, "max_tokens": 3, "temperature": 1.0})
        assert len(out["results"]) == 4
        # destroying one job leaves the processes (and the other jobs) alive
        core.destroy(lj)
        assert len(core.pool.actors[0].call("keys")) == 2
        assert _train(core, tj, steps=1)[0][1] > 0
    finally:
        core.destroy()
    assert core.pool.actors == {}


@pytest.mark.timeout(600)
@pytest.mark.parametrize("stage", [3])
def test_sequence_parallel_group_of_two_equals_one_process(stage):
    """Two ranks as ONE Ulysses group behind the server: both receive the whole batch, each runs half of the packed
    token axis; scores, loss, gradient norm and updated weights equal the single-process run."""
    single = ArcticRLServerCore()
    j1 = single.initialize(_job(stage))["job_id"]
    p = _payload()
    want_lp = single.forward(j1, {"batch": p["batch"], "meta": p["meta"]})["batch"]["log_probs"]
    want = _train(single, j1, steps=2)
    want_norm = single.weight_norm(training_job_id=j1)["training_norm"]
    core = ArcticRLServerCore(worker_factory=spawned_worker_factory(_free_port()), training_gpus=2)
    try:
        job = {**_job(stage), "ds_worker_config": {"sequence_parallel": 2}}
        jid = core.initialize(job)["job_id"]
        got_lp = core.forward(jid, {"batch": p["batch"], "meta": p["meta"]})["batch"]["log_probs"]
        assert got_lp.shape == want_lp.shape and torch.allclose(got_lp, want_lp, atol=1e-5)
        got = _train(core, jid, steps=2)
        for (la, na), (lb, nb) in zip(got, want):
            assert la == pytest.approx(lb, rel=1e-4, abs=1e-6) and na == pytest.approx(nb, rel=1e-4)
        assert core.weight_norm(training_job_id=jid)["training_norm"] == pytest.approx(want_norm, rel=1e-5)
        with pytest.raises(Exception):
            core.initialize({**_job(1), "job_type": "log_prob", "num_devices": 2,
                             "ds_worker_config": {"sequence_parallel": 3}})
    finally:
        core.destroy()
        single.destroy()


@pytest.mark.timeout(600)
def test_expert_parallel_job_behind_the_server(tmp_path):
    """``ds_worker_config.expert_parallel = 2``: each rank keeps half of every layer's experts; training equals the
    single-process run, and checkpoint export and the weight hand-over gather the expert shards."""
    def moe_job(**extra):
        return {"model_name": "qwen3-moe-tiny", "job_type": "training", "seed": 11, **extra,
                "ds_config": {"zero_optimization": {"stage": 1}, "gradient_clipping": 1.0,
                              "optimizer": {"type": "AdamW", "params": {"lr": 1e-3}}}}
    single = ArcticRLServerCore()
    j1 = single.initialize(moe_job())["job_id"]
    want = _train(single, j1, steps=2)
    want_norm = single.weight_norm(training_job_id=j1)["training_norm"]
    core = ArcticRLServerCore(training_gpus=2, sampling_gpus=2, colocate=True)       # rank process pool
    try:
        jid = core.initialize(moe_job(ds_worker_config={"expert_parallel": 2}, checkpoint_path=str(tmp_path)))["job_id"]
        got = _train(core, jid, steps=2)
        for (la, na), (lb, nb) in zip(got, want):
            assert la == pytest.approx(lb, rel=2e-3, abs=1e-5) and na == pytest.approx(nb, rel=2e-3)
        assert core.weight_norm(training_job_id=jid)["training_norm"] == pytest.approx(want_norm, rel=1e-4)
        saved = core.save(jid, step=2, export_hf=True)
        hf = [f for f in saved["files"] if f.endswith(".safetensors")]
        assert hf
        from arctic_platform_b200.models.hf_io import read_safetensors
        names = {n for f in hf for n, _t in read_safetensors(f)}
        assert {f"model.layers.0.mlp.experts.{e}.down_proj.weight" for e in range(4)} <= names      # all experts, once
        sj = core.initialize({"model_name": "qwen3-moe-tiny", "job_type": "sampling", "seed": 5,
                              "vllm_config": {"max_model_len": 64}})["job_id"]
        res = core.weight_sync(jid, [sj])
        assert res["strategies"] == ["in_process"]
        assert core.weight_norm(sampling_job_id=sj)["sampling_norm"] == pytest.approx(want_norm, rel=1e-4)
    finally:
        core.destroy()
        single.destroy()


@pytest.mark.timeout(300)
def test_a_rank_that_dies_between_steps_fails_the_job_and_frees_its_peer():
    """Host-side fault: one rank's process is ended between two calls (nothing in flight).  The next call must not
    leave the surviving rank waiting in a collective: the server stops it, marks the job FAILED and says why."""
    import time
    from arctic_platform_b200.common.server import JobError
    core = ArcticRLServerCore(worker_factory=spawned_worker_factory(_free_port()), training_gpus=2)
    try:
        jid = core.initialize(_job(3))["job_id"]
        _train(core, jid, steps=1)
        job = core.jobs[jid]
        assert core.check_workers(jid)["alive"] == [True, True]
        victim = job.workers[1]
        victim._proc.terminate()                        # the exact child this test started
        victim._proc.join(10)
        t0 = time.time()
        with pytest.raises(JobError, match="FAILED"):
            core.forward_backward(jid, _payload())      # rank 0 would wait for rank 1 in the first gather
        assert time.time() - t0 < 60
        assert job.status == "FAILED" and "failure" in job.info
        assert not job.workers[0]._proc.is_alive() and not job.workers[1]._proc.is_alive()
        with pytest.raises(JobError, match="FAILED"):
            core.step(jid)                              # a failed job answers with its state, it does not hang
        # the server itself is fine: a fresh job runs
        core.destroy(jid)
        j2 = core.initialize(_job(1))["job_id"]
        assert _train(core, j2, steps=1)[0][1] > 0
    finally:
        core.destroy()


@pytest.mark.timeout(300)
def test_a_rank_that_raises_does_not_leave_its_peer_waiting(monkeypatch):
    """One rank gets a shard it rejects (host-side error before any collective); the other enters the forward pass
    and would wait for it in the first ZeRO-3 gather.  After the grace period the waiting rank is stopped."""
    from arctic_platform_b200.common import server as srv
    from arctic_platform_b200.common.server import JobError, RanksLost, call_all
    core = ArcticRLServerCore(worker_factory=spawned_worker_factory(_free_port()), training_gpus=2)
    try:
        jid = core.initialize(_job(3))["job_id"]
        job = core.jobs[jid]
        p = _payload()
        good = (p["batch"], p["meta"], p["processing"])
        bad = ({"input_ids": "not a tensor"}, p["meta"], p["processing"])
        with pytest.raises(RanksLost, match="waiting peer"):
            call_all(job.workers, "forward_backward", [good, bad], peer_grace_s=3.0)
        assert not job.workers[0]._proc.is_alive()
    finally:
        core.destroy()


@pytest.mark.timeout(600)
def test_recovery_is_checkpoint_plus_restart(tmp_path):
    """Train, checkpoint, lose a rank (host-side: its process is ended between calls), recover: a new job on fresh
    rank processes continues from the checkpoint exactly as the uninterrupted run does."""
    from arctic_platform_b200.common.server import JobError
    steady = ArcticRLServerCore()
    js = steady.initialize(_job(3))["job_id"]
    want = _train(steady, js, steps=3)
    core = ArcticRLServerCore(training_gpus=2)                                  # rank process pool
    try:
        job_cfg = {**_job(3), "checkpoint_path": str(tmp_path)}
        jid = core.initialize(job_cfg)["job_id"]
        got = _train(core, jid, steps=2)
        saved = core.save(jid, step=2)
        assert saved["path"].endswith("checkpoint-2") and saved["global_step"] == 2
        lost = core.pool.actors[1]
        lost._proc.terminate()                                                  # the exact child of this pool
        lost._proc.join(10)
        with pytest.raises(JobError, match="FAILED"):
            core.forward_backward(jid, _payload())
        assert core.get_job_status(jid)["status"] == "FAILED"
        info = core.recover(jid)
        assert info["recovered_from"] == jid and info["global_steps"] == 2 and info["job_id"] != jid
        assert all(a.alive() for a in core.pool.actors.values()) and len(core.pool.actors) == 2
        got += _train(core, info["job_id"], steps=1)
        for (la, na), (lb, nb) in zip(got, want):
            assert la == pytest.approx(lb, rel=1e-4, abs=1e-6) and na == pytest.approx(nb, rel=1e-4)
        with pytest.raises(JobError):
            core.recover(12345)
    finally:
        core.destroy()
        steady.destroy()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("agg_mode", ["token-mean", "seq-mean-token-mean"])
def test_token_budget_micro_batches_stay_in_step_across_ranks(agg_mode):
    """Two ZeRO-3 ranks whose shards need different numbers of token-budget micro-batches: the rank with fewer pads
    with loss-free passes, so the per-pass gathers line up; results equal one process on the whole batch.  The
    sequence-mean aggregation divides by the number of REAL rows: the filler passes must not count as sequences."""
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=2, seed=21, p_rng=(4, 8), r_rng=(2, 6))
    # rank 0's half: long sequences; rank 1's half: short ones -> different micro-batch counts under one budget
    ids2, mask2, _ = make_grpo_batch(n_prompts=4, n_samples=2, seed=22, p_rng=(30, 40), r_rng=(2, 6))
    P = ids2.shape[1] - R
    big_ids = torch.zeros(8, P + R, dtype=torch.int64)
    big_mask = torch.zeros_like(big_ids)
    big_ids[:, P - (ids.shape[1] - R):] = ids
    big_mask[:, P - (mask.shape[1] - R):] = mask
    all_ids, all_mask = torch.cat([ids2[:4], big_ids[:4]]), torch.cat([mask2[:4], big_mask[:4]])
    B = all_ids.shape[0]
    g = torch.Generator().manual_seed(2)
    batch = {"input_ids": all_ids, "attention_mask": all_mask, "response_mask": all_mask[:, -R:].contiguous(),
             "old_log_probs": torch.randn(B, R, generator=g) * 0.01 - 2.0,
             "advantages": torch.randn(B, 1, generator=g).expand(B, R).contiguous()}
    budget = int(all_mask.sum(1).max()) + 4
    meta = {"response_length": R, "zorro_train_enable": False, "max_tokens_per_mb": budget,
            "actor_config": {"loss_agg_mode": agg_mode}}
    single = ArcticRLServerCore()
    j1 = single.initialize(_job(3))["job_id"]
    want_lp = single.forward(j1, {"batch": batch, "meta": dict(meta)})["batch"]["log_probs"]
    want = single.forward_backward(j1, {"batch": batch, "meta": dict(meta), "processing": {"loss_fn": "verl_grpo"}})
    want_norm = single.step(j1)["metrics"]["grad_norm"]
    core = ArcticRLServerCore(worker_factory=spawned_worker_factory(_free_port()), training_gpus=2)
    try:
        jid = core.initialize(_job(3))["job_id"]
        got_lp = core.forward(jid, {"batch": batch, "meta": dict(meta)})["batch"]["log_probs"]
        assert torch.allclose(got_lp, want_lp, atol=1e-5)
        got = core.forward_backward(jid, {"batch": batch, "meta": dict(meta), "processing": {"loss_fn": "verl_grpo"}})
        assert got["avg_loss"] == pytest.approx(want["avg_loss"], rel=1e-4, abs=1e-6)
        assert core.step(jid)["metrics"]["grad_norm"] == pytest.approx(want_norm, rel=1e-4)
    finally:
        core.destroy()
        single.destroy()


@pytest.mark.timeout(600)
def test_sequence_parallel_hybrid_model_equals_one_process():
    """The hybrid family under sequence parallelism: softmax-attention layers exchange heads for sequence, the
    recurrent layers run on the gathered rows and keep their slice; two ranks equal one process."""
    def job(**extra):
        return {"model_name": "qwen3.5-moe-tiny", "job_type": "training", "seed": 11, **extra,
                "ds_config": {"zero_optimization": {"stage": 1}, "gradient_clipping": 1.0,
                              "optimizer": {"type": "AdamW", "params": {"lr": 1e-3}}}}
    p = _payload()
    p["batch"] = {k: v[:4].contiguous() for k, v in p["batch"].items()}          # two prompt groups are enough here
    p["meta"] = {**p["meta"], "batch_num_tokens": float(p["batch"]["response_mask"].sum()), "global_batch_size": 4.0}
    single = ArcticRLServerCore()
    j1 = single.initialize(job())["job_id"]
    want_lp = single.forward(j1, {"batch": p["batch"], "meta": p["meta"]})["batch"]["log_probs"]
    want = single.forward_backward(j1, p)
    want_norm = single.step(j1)["metrics"]["grad_norm"]
    core = ArcticRLServerCore(worker_factory=spawned_worker_factory(_free_port()), training_gpus=2)
    try:
        jid = core.initialize(job(ds_worker_config={"sequence_parallel": 2}))["job_id"]
        got_lp = core.forward(jid, {"batch": p["batch"], "meta": p["meta"]})["batch"]["log_probs"]
        assert torch.allclose(got_lp, want_lp, atol=2e-5)
        got = core.forward_backward(jid, p)
        assert got["avg_loss"] == pytest.approx(want["avg_loss"], rel=1e-4, abs=1e-6)
        assert core.step(jid)["metrics"]["grad_norm"] == pytest.approx(want_norm, rel=2e-4)
    finally:
        core.destroy()
        single.destroy()
