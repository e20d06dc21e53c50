"""The Ray-protocol server objects (state + async facade) with the state hosted in process (no Ray needed)."""
import asyncio

import pytest
import torch

from arctic_platform_b200.common.ray_server import (ArcticRLRayServer, ArcticRLRayServerState,
                                                    create_arctic_rl_ray_server_state)
from arctic_platform_b200.common.server import JobError
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def test_state_accessors_and_facade_calls(tmp_path):
    state = create_arctic_rl_ray_server_state(colocate=True)
    assert isinstance(state, ArcticRLRayServerState) and state.get_colocate() and state.get_next_job_id() == 1
    srv = ArcticRLRayServer(state)

    async def scenario():
        assert (await srv.health()) == {"status": "ok"}
        t = await srv.initialize({"model_name": "qwen3-tiny", "job_type": "training", "num_devices": 1,
                                  "checkpoint_path": str(tmp_path),
                                  "ds_config": {"optimizer": {"params": {"lr": 1e-3}}, "gradient_clipping": 1.0}})
        s = await srv.initialize({"model_name": "qwen3-tiny", "job_type": "sampling", "num_devices": 1,
                                  "vllm_config": {"max_model_len": 64}})
        tj, sj = t["job_id"], s["job_id"]
        assert set(state.get_jobs()) == {tj, sj} and state.get_next_job_id() == max(tj, sj) + 1
        assert len(state.get_training_workers()) == 1 and len(state.get_sampling_pool()) == 1 and state.get_weight_sync_ready()
        assert state.get_log_prob_workers() == []
        # wrong kind, unknown id, malformed bodies
        with pytest.raises(JobError) as e:
            await srv.step(sj)
        assert e.value.status == 400
        with pytest.raises(JobError) as e:
            await srv.generate(999, {"prompts": [[1]]})
        assert e.value.status == 404
        with pytest.raises(JobError):
            await srv.generate(sj, {"prompts": "text"})
        with pytest.raises(JobError):
            await srv.weight_sync(tj, {})
        with pytest.raises(JobError):
            await srv.operation(tj, {})
        # one RL step through the facade, a trainer call and a sampler call in flight together
        sync = await srv.weight_sync(tj, {"target_sub_job_ids": [sj]})
        assert sync["status"] == "ok"
        ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2)
        B = ids.shape[0]
        batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:],
                 "advantages": torch.randn(B, 1).expand(B, R).contiguous()}
        old, gen = await asyncio.gather(srv.forward(tj, {"batch": batch, "meta": {}}),
                                        srv.generate(sj, {"prompts": [[1, 2, 3]], "sampling_params": {"n": 2, "max_tokens": 3}}))
        assert old["batch"]["log_probs"].shape == (B, R) and len(gen["results"]) == 2
        batch["old_log_probs"] = old["batch"]["log_probs"]
        out = await srv.forward_backward(tj, {"batch": batch, "meta": {"zorro_train_enable": True}})
        assert "avg_loss" in out
        st = await srv.step(tj, {"learning_rate": 5e-4})
        assert st["metrics"]["last_lr"] == pytest.approx(5e-4)
        assert (await srv.step(tj, 2e-4))["metrics"]["last_lr"] == pytest.approx(2e-4)        # bare value form
        saved = await srv.save(tj, {"step": 2, "export_hf": False})
        assert saved["path"].endswith("checkpoint-2")
        assert (await srv.load_checkpoint(tj, {"step": 2}))["global_steps"] == 2
        assert (await srv.sleep_inference(sj, 1))["status"] == "sleeping"
        assert (await srv.wake_inference(sj, ["weights", "kv_cache"]))["status"] == "awake"
        assert (await srv.reset_prefix_cache(sj))["status"] == "ok"
        assert (await srv.sleep_training(tj, "all"))["status"] == "sleeping"
        assert (await srv.wake_training(tj))["status"] == "awake"
        norms = await srv.weight_norm(tj, sj)
        assert norms["training_norm"] > 0
        op = await srv.operation(tj, {"operation_type": "reset-prefix-cache", "sub_job_id": sj})
        assert op["status"] == "ok"
        lp = await srv.log_probs(sj, {"prompts": [[1, 2, 3]], "completions": [[4, 5]]})
        assert len(lp["log_probs"][0]) == 2
        assert {j["job_id"] for j in (await srv.status())["jobs"]} == {tj, sj}
        assert (await srv.get_job_status(tj))["status"] == "RUNNING"
        with pytest.raises(JobError):
            await srv.destroy(tj, "sampling")
        await srv.destroy(tj, "training")
        assert set(state.get_jobs()) == {sj} and not state.get_weight_sync_ready()
        await srv.destroy()
        assert state.get_jobs() == {}

    asyncio.run(scenario())
