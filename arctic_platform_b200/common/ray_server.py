"""The job server behind the Ray protocol: a state object that owns jobs and workers, and an async facade with the
body-style signatures Ray callers use.

* ``ArcticRLRayServerState`` owns the job table and every worker.  With Ray it lives in a 0-GPU actor
  (``create_arctic_rl_ray_server_state``), so the driver process holds only a handle and several clients can attach to
  one deployment; without Ray the same object lives in the caller's process.  Besides the job lifecycle
  (``initialize``, ``destroy``, sampler sleep / wake / cache reset) it answers the bookkeeping questions a server
  facade asks: ``get_jobs``, ``get_next_job_id``, ``get_colocate``, ``get_weight_sync_ready``.
* ``ArcticRLRayServer`` is the data-plane facade: coroutines that take a job id and a ``body`` dict (``step(job_id,
  {"learning_rate": ...})``, ``save(job_id, {"path", "step", "export_hf"})``, ``generate(job_id, {"prompts",
  "sampling_params"})``, ...), verify the job's kind, and run the call on the state.  Long calls run in a worker
  thread, so one event loop serves a trainer and a rollout caller at the same time.

Both sit on ``common.server.ArcticRLServerCore`` (job table, rank fan-out, batch split / merge, metric reduction,
weight hand-over strategies) -- the HTTP server exposes that same core as routes.  Counterpart of
arctic_platform/common/ray_server.py:113-1214 in the reference.
"""
from __future__ import annotations

import asyncio
from typing import Any, Dict, List, Optional, Sequence, Union

from .server import ArcticRLServerCore, JobError


class ArcticRLRayServerState(ArcticRLServerCore):
    """The core plus the accessors of the reference's state actor.  Plain methods: behind Ray every method call is
    already asynchronous for the caller; in process they are cheap look-ups."""

    def get_jobs(self) -> Dict[int, Dict[str, Any]]:
        with self._lock:
            return {j.job_id: {"job_id": j.job_id, "job_type": j.job_type, "status": j.status, "num_devices": len(j.workers)}
                    for j in self.jobs.values()}

    def get_next_job_id(self) -> int:
        with self._lock:
            return max(self.jobs, default=0) + 1

    def get_colocate(self) -> bool:
        return bool(getattr(self, "colocate", False))

    def _workers_of(self, kind: str) -> List[Any]:
        job = self.find_job(kind)
        return list(job.workers) if job is not None else []

    def get_training_workers(self) -> List[Any]:
        return self._workers_of("training")

    def get_log_prob_workers(self) -> List[Any]:
        return self._workers_of("log_prob")

    def get_sampling_pool(self) -> List[List[Any]]:
        """Sampler replicas, each a list of its tensor-parallel ranks."""
        job = self.find_job("sampling")
        return self._replicas(job) if job is not None else []

    def get_weight_sync_ready(self) -> bool:
        return self.find_job("training") is not None and self.find_job("sampling") is not None


def create_arctic_rl_ray_server_state(**kwargs):
    """The state in a detached 0-GPU actor when Ray is importable, else in this process."""
    from ..rl.ray_client import _RayCoreProxy, ray_available
    if not ray_available():
        return ArcticRLRayServerState(**kwargs)
    import ray
    if not ray.is_initialized():
        ray.init(ignore_reinit_error=True)
    return _RayCoreProxy(ray.remote(num_gpus=0)(ArcticRLRayServerState).remote(**kwargs))


def _body(body: Any, default_key: Optional[str] = None) -> Dict[str, Any]:
    """Callers pass a dict, nothing, or (for one-argument calls) the bare value."""
    if body is None:
        return {}
    if isinstance(body, dict):
        return body
    if default_key is None:
        raise JobError(400, f"expected a JSON object, got {type(body).__name__}")
    return {default_key: body}


class ArcticRLRayServer:
    def __init__(self, arctic_rl_ray_server_state):
        self.state = arctic_rl_ray_server_state

    async def _run(self, fn, *args, **kwargs):
        return await asyncio.to_thread(fn, *args, **kwargs)

    def _verify_job(self, job_id: int, expected_types: Union[str, Sequence[str]]) -> None:
        kinds = (expected_types,) if isinstance(expected_types, str) else tuple(expected_types)
        info = self.state.get_job_status(job_id)                    # raises 404 for an unknown id
        if info.get("job_type") not in kinds:
            raise JobError(400, f"job {job_id} is a {info.get('job_type')} job, expected {' or '.join(kinds)}")

    # ---------------------------------------------------------------------------------------- lifecycle
    async def health(self) -> Dict[str, str]:
        return {"status": "ok"}

    async def initialize(self, job_config: Dict[str, Any]) -> Dict[str, Any]:
        return await self._run(self.state.initialize, job_config)

    async def destroy(self, job_id: Optional[int] = None, job_type: Optional[str] = None) -> Dict[str, Any]:
        if job_id is not None and job_type is not None:
            self._verify_job(job_id, job_type)
        return await self._run(self.state.destroy, job_id)

    async def status(self) -> Dict[str, Any]:
        return self.state.status()

    async def get_job_status(self, job_id: int) -> Dict[str, Any]:
        return self.state.get_job_status(job_id)

    # ---------------------------------------------------------------------------------------- training
    async def forward_backward(self, job_id: int, batch: Dict[str, Any]) -> Dict[str, Any]:
        self._verify_job(job_id, "training")
        return await self._run(self.state.forward_backward, job_id, batch)

    async def forward(self, job_id: int, batch: Dict[str, Any]) -> Dict[str, Any]:
        self._verify_job(job_id, ("training", "log_prob"))
        return await self._run(self.state.forward, job_id, batch)

    async def step(self, job_id: int, body: Any = None) -> Dict[str, Any]:
        self._verify_job(job_id, "training")
        return await self._run(self.state.step, job_id, _body(body, "learning_rate").get("learning_rate"))

    async def empty_training_cache(self, job_id: int) -> Dict[str, Any]:
        self._verify_job(job_id, ("training", "log_prob"))
        return await self._run(self.state.empty_training_cache, job_id)

    async def save(self, job_id: int, body: Any = None) -> Dict[str, Any]:
        self._verify_job(job_id, "training")
        b = _body(body, "path")
        return await self._run(self.state.save, job_id, b.get("path"), b.get("step"), bool(b.get("export_hf", False)),
                               b.get("save_total_limit"))

    async def load_checkpoint(self, job_id: int, body: Any = None) -> Dict[str, Any]:
        self._verify_job(job_id, "training")
        b = _body(body, "path")
        return await self._run(self.state.load_checkpoint, job_id, b.get("path"), b.get("step"))

    async def sleep_training(self, job_id: int, body: Any = None) -> Dict[str, Any]:
        self._verify_job(job_id, ("training", "log_prob"))
        return await self._run(self.state.sleep_training, job_id, _body(body, "mode").get("mode", "all"))

    async def wake_training(self, job_id: int, body: Any = None) -> Dict[str, Any]:
        self._verify_job(job_id, ("training", "log_prob"))
        return await self._run(self.state.wake_training, job_id)

    async def sleep_log_prob(self, job_id: int) -> Dict[str, Any]:
        self._verify_job(job_id, "log_prob")
        return await self._run(self.state.sleep_training, job_id, "all")

    async def wake_log_prob(self, job_id: int) -> Dict[str, Any]:
        self._verify_job(job_id, "log_prob")
        return await self._run(self.state.wake_training, job_id)

    # ---------------------------------------------------------------------------------------- sampling
    async def generate(self, job_id: int, request: Dict[str, Any]) -> Dict[str, Any]:
        self._verify_job(job_id, "sampling")
        r = _body(request)
        if not isinstance(r.get("prompts"), list):
            raise JobError(400, "generate needs a list of prompts")
        return await self._run(self.state.generate, job_id, r["prompts"], r.get("sampling_params"), r.get("routing_key"),
                               bool(r.get("strict", False)))

    async def log_probs(self, job_id: int, request: Dict[str, Any]) -> Dict[str, Any]:
        r = _body(request)
        return await self._run(self.state.log_probs, job_id, r.get("prompts") or [], r.get("completions") or [],
                               int(r.get("top_k", 1)))

    async def sleep_inference(self, job_id: int, body: Any = None) -> Dict[str, Any]:
        self._verify_job(job_id, "sampling")
        return await self._run(self.state.sleep_inference, job_id, int(_body(body, "level").get("level", 1)))

    async def wake_inference(self, job_id: int, body: Any = None) -> Dict[str, Any]:
        self._verify_job(job_id, "sampling")
        b = {"tags": body} if isinstance(body, list) else _body(body)
        return await self._run(self.state.wake_inference, job_id, b.get("tags"))

    async def reset_prefix_cache(self, job_id: int, body: Any = None) -> Dict[str, Any]:
        self._verify_job(job_id, "sampling")
        return await self._run(self.state.reset_prefix_cache, job_id)

    # ---------------------------------------------------------------------------------------- trainer -> sampler
    async def weight_sync(self, job_id: int, body: Dict[str, Any]) -> Dict[str, Any]:
        """``body``: ``{"source_sub_job_id"?, "target_sub_job_ids", "cuda_ipc"?, "low_memory"?}``; the source defaults
        to ``job_id`` (a training job)."""
        b = _body(body)
        src = int(b.get("source_sub_job_id", job_id))
        self._verify_job(src, "training")
        targets = [int(t) for t in (b.get("target_sub_job_ids") or [])]
        if not targets:
            raise JobError(400, "weight_sync needs target_sub_job_ids")
        return await self._run(self.state.weight_sync, src, targets, b.get("cuda_ipc"), b.get("low_memory"))

    async def weight_norm(self, training_job_id: Optional[int] = None, sampling_job_id: Optional[int] = None) -> Dict[str, Any]:
        return await self._run(self.state.weight_norm, training_job_id, sampling_job_id)

    async def operation(self, job_id: int, body: Dict[str, Any]) -> Dict[str, Any]:
        b = _body(body)
        if "operation_type" not in b:
            raise JobError(400, "operation needs operation_type")
        return await self._run(self.state.operation, b["operation_type"], int(b.get("sub_job_id", job_id)), b.get("payload"))
