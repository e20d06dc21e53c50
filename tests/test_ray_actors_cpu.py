"""Ray-actor workers against a fake ``ray`` that runs actors in-process: placement options, launcher environment,
one actor per rank shared by the jobs, error translation, and a real two-job run through the server core."""
import os
import sys
import types

import pytest


class _Ref:
    def __init__(self, fn):
        self.fn = fn


class _Method:
    def __init__(self, actor, name):
        self.actor, self.name = actor, name

    def remote(self, *a, **k):
        return _Ref(lambda: self.actor._call(self.name, a, k))


class _Actor:
    def __init__(self, cls, opts, log):
        self.obj, self.opts, self.dead, self.env = cls(), opts, False, {}
        log.append(self)

    def _call(self, name, a, k):
        if self.dead:
            raise FakeRay.exceptions.RayActorError("actor died")
        saved = dict(os.environ)
        os.environ.update(self.env)                       # every actor has its own process environment
        try:
            out = getattr(self.obj, name)(*a, **k)
            if name == "setup":
                self.env.update(a[0])
            return out
        except Exception as exc:
            raise FakeRay.exceptions.RayTaskError(f"{type(exc).__name__}: {exc}") from exc
        finally:
            os.environ.clear()
            os.environ.update(saved)

    def __getattr__(self, name):
        return _Method(self, name)


class FakeRay(types.ModuleType):
    class exceptions:
        class RayActorError(Exception):
            pass

        class RayTaskError(Exception):
            pass

        class GetTimeoutError(Exception):
            pass

    def __init__(self):
        super().__init__("ray")
        self.actors = []

    def is_initialized(self):
        return True

    def remote(self, cls):
        ray = self

        class Remote:
            def options(self_inner, **opts):
                self_inner.opts = opts
                return self_inner

            def remote(self_inner):
                return _Actor(cls, getattr(self_inner, "opts", {}), ray.actors)
        return Remote()

    def get(self, ref, timeout=None):
        return ref.fn()

    def kill(self, actor, no_restart=True):
        actor.dead = True

    def nodes(self):
        return []


@pytest.fixture
def fake_ray(monkeypatch):
    ray = FakeRay()
    monkeypatch.setitem(sys.modules, "ray", ray)
    util = types.ModuleType("ray.util")
    monkeypatch.setitem(sys.modules, "ray.util", util)
    pg = types.ModuleType("ray.util.placement_group")
    pg.placement_group = lambda bundles, strategy: types.SimpleNamespace(bundles=bundles, strategy=strategy,
                                                                          ready=lambda: _Ref(lambda: True))
    monkeypatch.setitem(sys.modules, "ray.util.placement_group", pg)
    ss = types.ModuleType("ray.util.scheduling_strategies")
    ss.PlacementGroupSchedulingStrategy = lambda placement_group, placement_group_bundle_index: \
        ("pg", placement_group.strategy, placement_group_bundle_index)
    monkeypatch.setitem(sys.modules, "ray.util.scheduling_strategies", ss)
    return ray


def test_pool_places_one_actor_per_rank_and_translates_errors(fake_ray, monkeypatch):
    from arctic_platform_b200.common import ray_actors
    from arctic_platform_b200.common.local_actors import ActorDied, ActorError
    from arctic_platform_b200.common.utils import ray_pg
    monkeypatch.setattr(ray_pg, "detect_gpus_per_node", lambda default=8: 2)
    monkeypatch.setattr("arctic_platform_b200.rl.config.primary_ip", lambda: "10.1.2.3")
    pool = ray_actors.RayRankPool(2, master_port=31000)
    h1 = pool.factory({"job_type": "training"}, 1, 2)          # asking for rank 1 first still creates rank 0 before it
    h0 = pool.factory({"job_type": "training"}, 0, 2)
    hs = pool.factory({"job_type": "sampling"}, 0, 1)
    assert len(fake_ray.actors) == 2 and h0.actor is hs.actor and h0.key != hs.key
    a0, a1 = pool.actors[0], pool.actors[1]
    assert a0.opts["num_gpus"] == 1.0 and a0.opts["scheduling_strategy"] == ("pg", "STRICT_PACK", 0)
    assert a1.opts["scheduling_strategy"] == ("pg", "STRICT_PACK", 1)
    assert a1.env == {"RANK": "1", "LOCAL_RANK": "0", "WORLD_SIZE": "2", "MASTER_PORT": "31000", "MASTER_ADDR": "10.1.2.3"}
    assert a0.env["MASTER_ADDR"] == "10.1.2.3" and a0.env["RANK"] == "0"
    assert sorted(a0.obj.keys()) == sorted([h0.key, hs.key])
    assert h0.alive() and h0.heartbeat()
    with pytest.raises(ActorError, match="AttributeError"):
        h0.call("no_such_method")
    hs.kill()
    assert a0.obj.keys() == [h0.key]                            # the sampler's engines are gone, the actor is not
    h1.terminate()
    assert not h1.alive()
    with pytest.raises(ActorDied):
        h1.call("rank_info")
    with pytest.raises(ValueError):
        pool.factory({"job_type": "training"}, 0, 1)            # a training job must span the pool
    with pytest.raises(ValueError):
        pool.factory({"job_type": "sampling"}, 5, 8)
    pool.shutdown()
    assert pool.actors == {} and all(a.dead for a in fake_ray.actors)


def test_server_core_runs_jobs_on_ray_actors(fake_ray, monkeypatch):
    """With a Ray cluster attached the server picks the Ray pool; a one-rank-per-job deployment keeps using in-process
    workers, so the pool is driven directly here: trainer and sampler of rank 0 share an actor and sync in process."""
    import torch
    from arctic_platform_b200.common import ray_actors
    from arctic_platform_b200.common.server import ArcticRLServerCore
    from arctic_platform_b200.common.utils import ray_pg
    monkeypatch.setattr(ray_pg, "detect_gpus_per_node", lambda default=8: 1)
    monkeypatch.setattr("arctic_platform_b200.rl.config.primary_ip", lambda: "127.0.0.1")
    assert isinstance(ArcticRLServerCore(training_gpus=2).pool, ray_actors.RayRankPool)
    pool = ray_actors.RayRankPool(1)
    core = ArcticRLServerCore(worker_factory=pool.factory, colocate=True)
    tj = core.initialize({"model_name": "qwen3-tiny", "job_type": "training", "seed": 2,
                          "ds_config": {"optimizer": {"params": {"lr": 1e-2}}}})["job_id"]
    sj = core.initialize({"model_name": "qwen3-tiny", "job_type": "sampling", "seed": 9,
                          "vllm_config": {"max_model_len": 32}})["job_id"]
    assert len(fake_ray.actors) == 1
    ids = torch.randint(3, 100, (2, 10))
    batch = {"input_ids": ids, "attention_mask": torch.ones_like(ids), "response_mask": torch.ones(2, 4, dtype=torch.long),
             "advantages": torch.ones(2, 4), "old_log_probs": torch.full((2, 4), -4.0)}
    core.forward_backward(tj, {"batch": batch, "meta": {"response_length": 4}, "processing": {"loss_fn": "verl_grpo"}})
    core.step(tj)
    assert core.weight_sync(tj, [sj])["strategies"] == ["in_process"]
    wn = core.weight_norm(training_job_id=tj, sampling_job_id=sj)
    assert wn["training_norm"] == pytest.approx(wn["sampling_norm"], rel=1e-6)
    assert len(core.generate(sj, [[4, 5]], {"n": 2, "max_tokens": 2})["results"]) == 2
    core.destroy()
