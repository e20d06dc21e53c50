"""Ray actors as the job server's workers: one actor per GPU, placed by the colocation plan, hosting that GPU's
engines of every job (the same ``_RankHost`` the spawned-process pool uses, so trainer and sampler of a GPU share an
actor and hand weights over in process).

``RayRankPool(world).factory`` is a ``worker_factory`` for ``ArcticRLServerCore``.  Ray places the actor (fractional
GPU claims are not needed: one actor owns the GPU for all three job types), sets ``CUDA_VISIBLE_DEVICES`` to the
granted device, and the actor exports ``RANK / LOCAL_RANK = 0 / WORLD_SIZE / MASTER_ADDR / MASTER_PORT`` before it
builds its first engine; rank 0's node is the rendezvous host.  The reference spawns its DeepSpeed workers the same
way (arctic_platform/common/deepspeed_worker.py:89-104, arctic_platform/common/ray_server.py:300-522)."""
from __future__ import annotations

import threading
from typing import Any, Dict, Optional

from .local_actors import ActorDied, ActorError, _RankHost
from .utils.ray_pg import ColocatePlacement, create_colocate_placement, pg_scheduling_options


class _RayRankHost(_RankHost):
    """``_RankHost`` plus what an actor has to do for itself: export the launcher variables, report its address."""

    def setup(self, env: Dict[str, str]) -> str:
        import os
        os.environ.update(env)
        from ..rl.config import primary_ip
        return primary_ip()

    def ping(self) -> bool:
        return True


class RayWorkerHandle:
    """The actor interface of one (Ray actor, job) pair."""

    def __init__(self, actor, key: str, rank: int):
        self.actor, self.key, self.rank = actor, key, rank

    def call(self, method: str, *args, timeout: Optional[float] = None, **kwargs):
        import ray
        try:
            return ray.get(self.actor.invoke.remote(self.key, method, *args, **kwargs), timeout=timeout)
        except ray.exceptions.RayActorError as exc:                    # the actor's process is gone
            raise ActorDied(f"ray actor of rank {self.rank} died: {exc}") from exc
        except ray.exceptions.GetTimeoutError as exc:
            raise ActorDied(f"no answer from the ray actor of rank {self.rank} within {timeout}s") from exc
        except ray.exceptions.RayTaskError as exc:                     # the method raised
            raise ActorError(str(exc)) from exc

    def alive(self) -> bool:
        import ray
        try:
            ray.get(self.actor.ping.remote(), timeout=5.0)
            return True
        except Exception:
            return False

    def heartbeat(self, timeout: float = 5.0) -> bool:
        return self.alive()

    def sync_to(self, dst: "RayWorkerHandle") -> int:
        """Weight hand-over to another job's engine hosted by the SAME actor."""
        import ray
        return ray.get(self.actor.sync.remote(self.key, dst.key))

    def kill(self) -> None:
        """Ends this job's engines; the actor stays for the GPU's other jobs."""
        import ray
        try:
            ray.get(self.actor.drop.remote(self.key), timeout=60.0)
        except Exception:
            pass

    def terminate(self) -> None:
        import ray
        ray.kill(self.actor, no_restart=True)


class RayRankPool:
    def __init__(self, world: int, master_port: int = 29500, colocate: bool = True,
                 placement: Optional[ColocatePlacement] = None):
        self.world, self.master_port, self.colocate = int(world), int(master_port), bool(colocate)
        self.placement = placement
        self.actors: Dict[int, Any] = {}
        self.master_addr: Optional[str] = None
        self._ids = 0
        self._lock = threading.Lock()

    def _actor(self, rank: int):
        import ray
        with self._lock:
            if self.placement is None:
                self.placement = create_colocate_placement(self.world)
            a = self.actors.get(rank)
            if a is None:
                opts = pg_scheduling_options(self.placement, rank, "training", colocate=False)
                a = ray.remote(_RayRankHost).options(**opts).remote()
                env = {"RANK": str(rank), "LOCAL_RANK": "0", "WORLD_SIZE": str(self.world),
                       "MASTER_PORT": str(self.master_port), "MASTER_ADDR": self.master_addr or "127.0.0.1"}
                if rank == 0:
                    self.master_addr = ray.get(a.setup.remote({k: v for k, v in env.items() if k != "MASTER_ADDR"}))
                    ray.get(a.setup.remote({"MASTER_ADDR": self.master_addr}))
                else:
                    if self.master_addr is None:
                        raise RuntimeError("rank 0 is created first: it names the rendezvous host")
                    ray.get(a.setup.remote(env))
                self.actors[rank] = a
            return a

    def factory(self, job_config: Dict[str, Any], rank: int, world: int) -> RayWorkerHandle:
        job_type = job_config.get("job_type", "training")
        if rank >= self.world:
            raise ValueError(f"{job_type} job wants rank {rank} but the pool has {self.world} actors")
        if job_type != "sampling" and world != self.world:
            raise ValueError(f"a {job_type} job forms a process group over the whole pool: it needs {self.world} "
                             f"ranks, not {world}")
        import ray
        if rank > 0 and 0 not in self.actors:
            self._actor(0)
        actor = self._actor(rank)
        with self._lock:
            self._ids += 1
            key = f"{job_type}-{self._ids}"
        ray.get(actor.create.remote(key))
        return RayWorkerHandle(actor, key, rank)

    def shutdown(self) -> None:
        import ray
        with self._lock:
            actors, self.actors = list(self.actors.values()), {}
        for a in actors:
            try:
                ray.kill(a, no_restart=True)
            except Exception:
                pass
