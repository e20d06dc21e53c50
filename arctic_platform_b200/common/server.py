"""Job server core: what sits behind the HTTP routes, the Ray methods and the in-process client.

A *job* is a set of engine workers of one kind -- ``training``, ``sampling`` or ``log_prob`` -- created by
``initialize(job_config)``; every later call names a job id.  The method set and the return shapes follow
the reference's servers (arctic_platform/common/ray_server.py:551-1209, common/http_server.py:140-970):
``forward_backward -> {job_id, metrics, avg_loss}``, ``forward -> {job_id, batch, metrics, avg_loss}``,
``step -> {job_id, metrics: {last_lr, grad_norm}, batch}``, ``generate -> {results: [...]}``,
``weight_norm``, ``weight_sync``, ``sleep/wake`` for each engine kind, ``status`` / ``get_job_status``.

Workers are reached through a tiny actor interface (``call(method, *args)``) with three implementations:
in-process (this file), spawned local processes (``local_actors.py``) and Ray actors when Ray is
importable.  Failure handling is host-side: a worker that raises during ``initialize`` makes the server
destroy every worker it already created for that job (all-or-nothing, as
arctic_platform/common/deepspeed_worker.py:89-104), heartbeats mark a job ``FAILED``.
"""
from __future__ import annotations

import itertools
import threading
import os
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch

from .utils.batch import merge_dict_shards, restore_batch_order, split_batch_for_ranks
from .utils.metrics import finalize_fwd_bwd_metrics


class JobError(RuntimeError):
    """Carries an HTTP-like status code: 404 unknown job, 409 conflicting state, 400 bad request."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def route_prompts(prompts, n_replicas: int, routing_key=None, strict: bool = False) -> List[int]:
    """Replica index per prompt.  ``routing_key`` (one key, or one per prompt) pins equal keys to one replica by a
    stable hash -- conversations or prompt families that share a prefix stay together; ``strict`` is plain
    round-robin; the default gives every replica one contiguous slice (equal load, neighbours together)."""
    import zlib
    P = len(prompts)
    if routing_key is not None:
        keys = list(routing_key) if isinstance(routing_key, (list, tuple)) else [routing_key] * P
        if len(keys) != P:
            raise JobError(400, f"routing_key has {len(keys)} entries for {P} prompts")
        return [zlib.crc32(repr(k).encode()) % n_replicas for k in keys]
    if strict:
        return [i % n_replicas for i in range(P)]
    per = (P + n_replicas - 1) // n_replicas
    return [i // per for i in range(P)]


class InProcessActor:
    """Actor facade over an object living in this process."""

    def __init__(self, obj):
        self.obj = obj

    def call(self, method: str, *args, **kwargs):
        return getattr(self.obj, method)(*args, **kwargs)

    def kill(self) -> None:
        try:
            self.obj.destroy()
        except Exception:
            pass


@dataclass
class Job:
    job_id: int
    job_type: str
    config: Dict[str, Any]
    workers: List[Any]
    status: str = "RUNNING"
    created: float = field(default_factory=time.time)
    last_heartbeat: float = field(default_factory=time.time)
    info: Dict[str, Any] = field(default_factory=dict)


class RanksLost(RuntimeError):
    """A rank of a job died, or failed while its peers were left waiting for it in a collective; the peers were
    stopped.  The job cannot continue (recovery = restart from the last checkpoint)."""


def _hard_stop(worker) -> None:
    """Stops a rank that is stuck behind a failed peer.  Normally the rank's process is terminated.  When the job
    runs its kernels on NVSwitch multicast (``APB_MULTIMEM=1``) the rank's buffers are bound to a multicast object
    shared with the surviving ranks, and ending a process in that state can fault the other GPUs: the rank is then
    only ASKED to shut down (``destroy``), and what ends its wait is the bounded device wait (1 s, status word) and
    the process group's timeout."""
    from ..parallel.symm import multimem_enabled
    try:
        if multimem_enabled():
            if hasattr(worker, "request_destroy"):
                worker.request_destroy()
            else:
                worker.kill()               # in-process and spawned actors: kill() asks the worker to destroy itself
        elif hasattr(worker, "terminate"):
            worker.terminate()
        else:
            worker.kill()
    except Exception:
        pass


def call_all(workers: Sequence[Any], method: str, per_worker_args: Optional[Sequence[tuple]] = None, *shared_args,
             peer_grace_s: Optional[float] = 30.0) -> List[Any]:
    """Calls ``method`` on every worker AT THE SAME TIME and returns the results in worker order.  The ranks of a
    job run collectives inside these calls (process-group set-up, ZeRO-3 gathers, the optimizer's reduce-scatter),
    so a rank-by-rank loop would block on the first rank for ever; it would also serialise the ranks' compute.

    When one rank fails, its peers may be stuck in a collective that the failed rank will never join.  They get
    ``peer_grace_s`` seconds to return on their own (none when the rank died outright); those still busy are then
    stopped and :class:`RanksLost` is raised.  If everybody returned, the first failure is raised as it is.
    ``peer_grace_s=None`` is for workers that never wait for one another (sampler replicas): nobody is stopped."""
    args = [tuple(a) for a in per_worker_args] if per_worker_args is not None else [tuple(shared_args)] * len(workers)
    if len(workers) == 1:
        return [workers[0].call(method, *args[0])]
    from concurrent.futures import FIRST_EXCEPTION, ThreadPoolExecutor, wait
    from .local_actors import ActorDied
    pool = ThreadPoolExecutor(max_workers=len(workers))
    try:
        futs = [pool.submit(w.call, method, *a) for w, a in zip(workers, args)]
        done, pending = wait(futs, return_when=FIRST_EXCEPTION)
        stopped = []
        if pending:
            died = any(isinstance(f.exception(), ActorDied) for f in done if f.exception() is not None)
            if peer_grace_s is None:
                _d, pending = wait(pending)
            else:
                _d, pending = wait(pending, timeout=0.0 if died else peer_grace_s)
            for w, f in zip(workers, futs):
                if f in pending:
                    _hard_stop(w)
                    stopped.append(w)
            wait(pending, timeout=30.0)
        results, first = [], None
        for w, f in zip(workers, futs):
            exc = f.exception() if f.done() else TimeoutError("worker did not return after it was stopped")
            results.append(None if exc is not None else f.result())
            if exc is not None and first is None and w not in stopped:      # a stopped peer's error is a consequence
                first = exc
    finally:
        pool.shutdown(wait=False)
    if stopped:
        raise RanksLost(f"{method}: a rank failed ({type(first).__name__}: {str(first)[:300]}); "
                        f"{len(stopped)} waiting peer(s) were stopped") from first
    if first is not None:
        raise first
    return results


def _free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def default_worker_factory(job_config: Dict[str, Any], rank: int, world: int):
    from ..engine.worker import EngineWorker
    return InProcessActor(EngineWorker())


class ArcticRLServerCore:
    def __init__(self, worker_factory: Optional[Callable] = None, training_gpus: int = 0,
                 sampling_gpus: int = 0, log_prob_gpus: int = 0, colocate: bool = False,
                 heartbeat_timeout: float = 0.0, master_port: Optional[int] = None,
                 log_prob_engine: str = "deepspeed"):
        self.gpus = {"training": training_gpus, "sampling": sampling_gpus, "log_prob": log_prob_gpus}
        # which engine serves log-prob jobs: "deepspeed" = a forward-only training engine (ZeRO shards, packed
        # layout), "vllm" = the sampler's engine and weights layout (arctic_platform/common/ray_server.py:141-201)
        if log_prob_engine not in ("deepspeed", "vllm"):
            raise ValueError(f"log_prob_engine must be 'deepspeed' or 'vllm', got {log_prob_engine!r}")
        self.log_prob_engine = log_prob_engine
        self.pool = None
        if worker_factory is None:
            ranks = max(int(training_gpus or 0), int(log_prob_gpus or 0))
            if ranks > 1:
                # more than one rank per job: one long-lived process per GPU hosting that GPU's engines of every
                # job (the ranks need a process group; colocated engines need to share a process)
                from .ray_cluster import ray_available
                ray_up = False
                if ray_available():
                    import ray
                    ray_up = ray.is_initialized()
                if ray_up:                        # a Ray cluster is attached: one actor per GPU, placed by Ray
                    from .ray_actors import RayRankPool
                    self.pool = RayRankPool(ranks, master_port or _free_port(), colocate=colocate)
                else:
                    from .local_actors import RankProcessPool
                    self.pool = RankProcessPool(ranks, master_port or _free_port(), colocate=colocate)
                worker_factory = self.pool.factory
            else:
                worker_factory = default_worker_factory
        self.worker_factory = worker_factory
        self.colocate = colocate
        self.jobs: Dict[int, Job] = {}
        self._ids = itertools.count(1)
        self._lock = threading.RLock()
        self.heartbeat_timeout = heartbeat_timeout
        self._watchdog = None

    # ------------------------------------------------------------------ lifecycle
    def initialize(self, job_config: Dict[str, Any]) -> Dict[str, Any]:
        job_type = job_config.get("job_type", "training")
        if job_type not in ("training", "sampling", "log_prob"):
            raise JobError(400, f"unknown job_type {job_type!r}")
        if job_type == "log_prob":
            job_config = {**job_config, "log_prob_engine": job_config.get("log_prob_engine") or self.log_prob_engine}
        n = int(job_config.get("num_devices") or self.gpus.get(job_type) or 1)
        tp = int((job_config.get("vllm_config") or {}).get("tensor_parallel_size", 1) or 1) if job_type == "sampling" else 1
        # (an SPMD launch -- one client and one in-process worker per rank -- forms its replicas over the launcher's
        # world: the worker checks the division there)
        spmd = n == 1 and int(os.environ.get("WORLD_SIZE", "1") or 1) > 1
        if tp > 1 and n % tp and not spmd:
            raise JobError(400, f"tensor_parallel_size={tp} does not divide the sampling job's {n} devices")
        with self._lock:
            for j in self.jobs.values():
                if j.job_type == job_type and j.status == "RUNNING" and not job_config.get("allow_multiple"):
                    raise JobError(409, f"a {job_type} job is already running (job {j.job_id})")
            job_id = next(self._ids)
        workers: List[Any] = []
        try:
            for rank in range(n):
                w = self.worker_factory(job_config, rank, n)
                workers.append(w)
            if any(ok is False for ok in call_all(workers, "initialize", None, job_config)):
                raise RuntimeError("worker.initialize returned False")
        except Exception as exc:
            for w in workers:          # all-or-nothing: no half-initialised job survives
                try:
                    w.kill()
                except Exception:
                    pass
            raise JobError(500, f"{job_type} job failed to initialise: {exc}") from exc
        ckpt = job_config.get("checkpoint_path")
        info = {"job_id": job_id, "job_type": job_type, "model_name": job_config.get("model_name"),
                "status": "RUNNING", "num_devices": n,
                "checkpoint_path": f"{ckpt}/arctic_rl_job_{job_id}" if ckpt else None,
                "cuda_ipc": bool(job_config.get("cuda_ipc")), "low_memory": bool(job_config.get("low_memory")),
                "engine": "b200"}
        with self._lock:
            self.jobs[job_id] = Job(job_id, job_type, dict(job_config), workers, info=info)
        return info

    def destroy(self, job_id: Optional[int] = None) -> Dict[str, Any]:
        with self._lock:
            ids = [job_id] if job_id is not None else list(self.jobs)
            jobs = [self.jobs.pop(i) for i in ids if i in self.jobs]
        if job_id is not None and not jobs:
            raise JobError(404, f"unknown job {job_id}")
        for j in jobs:
            for w in j.workers:
                w.kill()
            j.status = "DESTROYED"
        if job_id is None and self.pool is not None:
            self.pool.shutdown()                  # everything was destroyed: the rank processes go too
        return {"destroyed": [j.job_id for j in jobs]}

    def _job(self, job_id: int, kinds=None) -> Job:
        with self._lock:
            j = self.jobs.get(int(job_id)) if job_id is not None else None
        if j is None:
            raise JobError(404, f"unknown job {job_id}")
        if j.status != "RUNNING":
            raise JobError(409, f"job {job_id} is {j.status}")
        if kinds and j.job_type not in kinds:
            raise JobError(400, f"job {job_id} is a {j.job_type} job, expected one of {kinds}")
        if self.heartbeat_timeout and time.time() - j.last_heartbeat > self.heartbeat_timeout:
            j.status = "FAILED"
            raise JobError(409, f"job {job_id} missed its heartbeat deadline")
        j.last_heartbeat = time.time()      # any call on the job is a sign of life from its client
        return j

    def heartbeat(self, job_id: int) -> None:
        with self._lock:
            j = self.jobs.get(int(job_id))
            if j is None:
                raise JobError(404, f"unknown job {job_id}")
            j.last_heartbeat = time.time()

    def find_job(self, job_type: str) -> Optional[Job]:
        with self._lock:
            for j in self.jobs.values():
                if j.job_type == job_type and j.status == "RUNNING":
                    return j
        return None

    # ------------------------------------------------------------------ training / scoring
    def _fail_job(self, job: Job, why: str) -> None:
        """Host-side failure handling: the job is marked FAILED and every worker of it is stopped."""
        job.status = "FAILED"
        job.info["failure"] = why
        for w in job.workers:
            _hard_stop(w)

    def _call_job(self, job: Job, method: str, per_worker_args=None, *shared):
        from .local_actors import ActorDied
        try:
            return call_all(job.workers, method, per_worker_args, *shared)
        except (ActorDied, RanksLost) as exc:
            self._fail_job(job, str(exc))
            raise JobError(500, f"job {job.job_id} FAILED: {exc}") from exc

    def recover(self, job_id: int, path: Optional[str] = None, step: Optional[int] = None) -> Dict[str, Any]:
        """Checkpoint + restart, the platform's recovery path: tears the (failed) job down, starts a new job from the
        same configuration on fresh worker processes and loads the newest checkpoint of the OLD job (or ``path``).
        Returns the new job's info with ``recovered_from`` and the restored ``global_steps`` (0 = no checkpoint)."""
        with self._lock:
            old = self.jobs.get(int(job_id))
        if old is None:
            raise JobError(404, f"unknown job {job_id}")
        cfg, ckpt = dict(old.config), path or old.info.get("checkpoint_path")
        for w in old.workers:
            _hard_stop(w)
        with self._lock:
            self.jobs.pop(old.job_id, None)
        old.status = "DESTROYED"
        info = dict(self.initialize(cfg))
        steps = 0
        if ckpt and old.job_type == "training":
            import os
            if os.path.isdir(ckpt):
                steps = self.load_checkpoint(info["job_id"], ckpt, step)["global_steps"]
        info.update(recovered_from=old.job_id, global_steps=steps)
        return info

    def start_worker_watchdog(self, period_s: float = 10.0) -> None:
        """Background liveness check of every running job's workers; a job that lost a worker is marked FAILED and
        torn down without waiting for the client's next call."""
        if self._watchdog is not None:
            return
        stop = threading.Event()

        def loop():
            while not stop.wait(period_s):
                with self._lock:
                    ids = [j.job_id for j in self.jobs.values() if j.status == "RUNNING"]
                for jid in ids:
                    try:
                        self.check_workers(jid)
                    except JobError:
                        pass
        t = threading.Thread(target=loop, name="apb-worker-watchdog", daemon=True)
        t.start()
        self._watchdog = (t, stop)

    def stop_worker_watchdog(self) -> None:
        if self._watchdog is not None:
            self._watchdog[1].set()
            self._watchdog[0].join(timeout=5.0)
            self._watchdog = None

    def check_workers(self, job_id: int, timeout: float = 5.0) -> Dict[str, Any]:
        """Liveness probe of every worker of a job (for a watchdog or an operator): a job with a worker that does
        not answer is marked FAILED and torn down."""
        job = self._job(job_id)
        # process liveness where the worker offers it (never blocks behind a long call), else a round trip
        alive = [bool(w.alive()) if hasattr(w, "alive") else (bool(w.heartbeat(timeout)) if hasattr(w, "heartbeat") else True)
                 for w in job.workers]
        if not all(alive):
            self._fail_job(job, f"workers {[i for i, a in enumerate(alive) if not a]} do not answer")
        return {"job_id": job.job_id, "alive": alive, "status": job.status}

    def _fan_out(self, job: Job, method: str, payload: Dict[str, Any]) -> List[Dict[str, Any]]:
        batch = payload.get("batch")
        meta = dict(payload.get("meta") or {})
        processing = payload.get("processing")
        n = len(job.workers)
        sp = int(((job.config.get("ds_worker_config") or {}).get("sequence_parallel", 1)) or 1)
        if sp > 1:
            # ranks [k*sp, (k+1)*sp) form one sequence-parallel group: they all get data shard k and split its tokens
            if n % sp:
                raise JobError(400, f"sequence_parallel={sp} does not divide the job's {n} ranks")
            shards, order = split_batch_for_ranks(batch, meta, n // sp)
            shards = [shards[r // sp] for r in range(n)]
        else:
            shards, order = split_batch_for_ranks(batch, meta, n)
        results = self._call_job(job, method, [(shard, meta, processing) for shard in shards])
        if sp > 1:
            # tensors come back complete from every rank of a group: keep the group leader's copy; metrics are sums
            # over the rows each rank scored, so they all count
            for r, res in enumerate(results):
                if r % sp and isinstance(res, dict) and "batch" in res:
                    res["batch"] = None
        return results, order

    def forward_backward(self, job_id: int, payload: Dict[str, Any]) -> Dict[str, Any]:
        job = self._job(job_id, ("training",))
        results, _ = self._fan_out(job, "forward_backward", payload)
        metrics, avg_loss = finalize_fwd_bwd_metrics(results)
        return {"job_id": job.job_id, "metrics": metrics, "avg_loss": avg_loss}

    def forward(self, job_id: int, payload: Dict[str, Any]) -> Dict[str, Any]:
        job = self._job(job_id, ("training", "log_prob"))
        results, order = self._fan_out(job, "forward_no_grad", payload)
        metrics, avg_loss = finalize_fwd_bwd_metrics(results)
        merged = merge_dict_shards([r["batch"] for r in results if r.get("batch")])
        if order is not None:
            merged = restore_batch_order(merged, order)
        return {"job_id": job.job_id, "batch": merged, "metrics": metrics, "avg_loss": avg_loss}

    def step(self, job_id: int, learning_rate: Optional[float] = None) -> Dict[str, Any]:
        job = self._job(job_id, ("training",))
        outs = self._call_job(job, "step", None, learning_rate)
        return {"job_id": job.job_id, "metrics": outs[0]["metrics"], "batch": {}}

    def empty_training_cache(self, job_id: int) -> Dict[str, Any]:
        job = self._job(job_id, ("training", "log_prob"))
        call_all(job.workers, "empty_cache")
        return {"job_id": job.job_id, "status": "ok"}

    # ------------------------------------------------------------------ checkpoints
    def save(self, job_id: int, path: Optional[str] = None, step: Optional[int] = None, export_hf: bool = False,
             save_total_limit: Optional[int] = None) -> Dict[str, Any]:
        """``<root>/checkpoint-<step>/`` is a complete engine checkpoint directory (``latest``, ``global_step<N>/``,
        optional ``hf/``); ``<root>/latest`` holds the integer step; old ``checkpoint-*`` children are pruned under
        ``root`` (arctic_platform/common/ray_server.py:765-789 in the reference)."""
        from .utils.checkpoint import prune_checkpoint_dirs, resolve_checkpoint_save_paths
        job = self._job(job_id, ("training",))
        root = path or job.info.get("checkpoint_path")
        if not root:
            raise JobError(400, "no checkpoint path configured")
        save_dir, prune_root = resolve_checkpoint_save_paths(root, step)
        os.makedirs(save_dir, exist_ok=True)
        outs = self._call_job(job, "save_checkpoint", None, save_dir, None, export_hf)
        if step is not None:
            with open(os.path.join(prune_root, "latest"), "w", encoding="utf-8") as f:
                f.write(str(int(step)))
        if save_total_limit and int(save_total_limit) > 0:
            prune_checkpoint_dirs(prune_root, int(save_total_limit))
        first = outs[0] if outs and isinstance(outs[0], dict) else {}
        return {"job_id": job.job_id, "path": save_dir, "hf_path": first.get("hf_path"),
                "global_step": first.get("global_step"), "tag": first.get("tag"), "files": first.get("files", [])}

    def load_checkpoint(self, job_id: int, path: Optional[str] = None, step: Optional[int] = None) -> Dict[str, Any]:
        from .utils.checkpoint import resolve_checkpoint_load_path
        job = self._job(job_id, ("training",))
        root = path or job.info.get("checkpoint_path")
        if not root:
            raise JobError(400, "no checkpoint path configured")
        ckpt = resolve_checkpoint_load_path(root, step, explicit_path=path is not None)
        # an explicit path or step that holds no checkpoint is an error, never a silent restart from step 0
        strict = path is not None or step is not None
        try:
            steps = self._call_job(job, "load_checkpoint", None, ckpt, None, strict)
        except FileNotFoundError as exc:
            raise JobError(404, str(exc)) from exc
        n = int(steps[0] or 0)
        return {"job_id": job.job_id, "path": ckpt, "global_step": n, "global_steps": n}

    # ------------------------------------------------------------------ rollout
    def generate(self, job_id: int, prompts, sampling_params=None, routing_key=None, strict: bool = False):
        job = self._job(job_id, ("sampling",))
        replicas = self._replicas(job)
        n = len(replicas)

        def on_replica(r, method, *args):
            # the ranks of a tensor-parallel replica run the call together and return the same thing
            if len(replicas[r]) == 1:
                return replicas[r][0].call(method, *args)
            return call_all(replicas[r], method, None, *args)[0]

        if n == 1:
            return {"job_id": job.job_id, "results": on_replica(0, "generate", prompts, sampling_params)}
        # replica data parallelism: every prompt goes to ONE replica with all its samples (so the replica shares the
        # prompt's KV among them); replicas run concurrently and the results come back in prompt order
        assign = route_prompts(prompts, n, routing_key, strict)
        groups: Dict[int, List[int]] = {}
        for i, r in enumerate(assign):
            groups.setdefault(r, []).append(i)

        def run(item):
            r, idxs = item
            out = on_replica(r, "generate", [prompts[i] for i in idxs], sampling_params)
            for o in out:
                o["prompt_index"] = idxs[o["prompt_index"]]
            return out

        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=len(groups)) as pool:
            parts = list(pool.map(run, sorted(groups.items())))
        results = sorted((o for part in parts for o in part), key=lambda o: o["prompt_index"])   # stable: sample order kept
        return {"job_id": job.job_id, "results": results}

    @staticmethod
    def _replicas(job: Job) -> List[List[Any]]:
        """Workers of a sampling job grouped into replicas: ``tensor_parallel_size`` consecutive ranks each."""
        tp = int((job.config.get("vllm_config") or {}).get("tensor_parallel_size", 1) or 1)
        ws = list(job.workers)
        if tp <= 1 or len(ws) < tp:
            return [[w] for w in ws]
        return [ws[i:i + tp] for i in range(0, len(ws), tp)]

    def log_probs(self, job_id: int, prompts, completions, top_k: int = 1) -> Dict[str, Any]:
        job = self._job(job_id, ("sampling", "log_prob", "training"))
        if len(prompts) != len(completions):
            raise JobError(400, f"{len(prompts)} prompts but {len(completions)} completions")
        if job.job_type == "sampling":
            # scored with the sampler's own weights (the reference's ``log_prob_engine = vllm``): the requests are
            # spread over the replicas, each scores its share in one packed pass
            replicas = self._replicas(job)
            n = len(replicas)
            share = [list(range(r, len(prompts), n)) for r in range(n)]
            active = [(ws, idx) for ws, idx in zip(replicas, share) if idx]
            flat = [(w, idx) for ws, idx in active for w in ws]          # all ranks of a replica score the same share
            outs = call_all([w for w, _ in flat], "score_completions",
                            [([prompts[i] for i in idx], [completions[i] for i in idx], int(top_k)) for _, idx in flat],
                            peer_grace_s=None)
            firsts, k = [], 0
            for ws, _idx in active:
                firsts.append(outs[k])
                k += len(ws)
            rows = [None] * len(prompts)
            tops = [None] * len(prompts)
            for (_, idx), res in zip(active, firsts):
                lp_rows, top_rows = (res["log_probs"], res["top_log_probs"]) if isinstance(res, dict) else (res, None)
                for j, i in enumerate(idx):
                    rows[i] = lp_rows[j]
                    if top_rows is not None:
                        tops[i] = top_rows[j]
            out = {"job_id": job.job_id, "log_probs": rows}
            if int(top_k) > 1:
                out["top_log_probs"] = tops
            return out
        if int(top_k) > 1:
            # the k most likely tokens per position need the whole distribution: one packed pass on every rank's share
            share = [list(range(r, len(prompts), len(job.workers))) for r in range(len(job.workers))]
            outs = call_all(job.workers, "score_completions",
                            [([prompts[i] for i in idx], [completions[i] for i in idx], int(top_k)) for idx in share])
            rows, tops = [None] * len(prompts), [None] * len(prompts)
            for idx, res in zip(share, outs):
                for j, i in enumerate(idx):
                    rows[i], tops[i] = res["log_probs"][j], res["top_log_probs"][j]
            return {"job_id": job.job_id, "log_probs": rows, "top_log_probs": tops}
        rows = []
        P = max(len(p) for p in prompts)
        R = max(len(c) for c in completions)
        ids = torch.zeros((len(prompts), P + R), dtype=torch.int64)
        mask = torch.zeros_like(ids)
        for i, (p, c) in enumerate(zip(prompts, completions)):
            ids[i, P - len(p):P] = torch.tensor(p)
            mask[i, P - len(p):P] = 1
            ids[i, P:P + len(c)] = torch.tensor(c)
            mask[i, P:P + len(c)] = 1
        out = self.forward(job.job_id, {"batch": {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, P:]},
                                        "meta": {"response_length": R, "zorro_train_enable": True}})
        lp = out["batch"]["log_probs"]
        for i, c in enumerate(completions):
            rows.append(lp[i, :len(c)].tolist())
        return {"job_id": job.job_id, "log_probs": rows}

    # ------------------------------------------------------------------ weights
    def weight_sync(self, source_job_id: int, target_job_ids: List[int], cuda_ipc: Optional[bool] = None,
                    low_memory: Optional[bool] = None) -> Dict[str, Any]:
        src = self._job(source_job_id, ("training",))
        t0 = time.perf_counter()
        total = 0
        from .utils.weight_sync import sync_pair
        strategies = set()
        stage = int(((src.config.get("ds_config") or {}).get("zero_optimization") or {}).get("stage", 1))
        sharded = stage >= 3 and len(src.workers) > 1
        for tid in target_job_ids:
            dst = self._job(tid, ("sampling", "log_prob"))
            from .utils.weight_sync import same_rank_process
            paired = len(dst.workers) == len(src.workers) and all(
                same_rank_process(sw, dw) for sw, dw in zip(src.workers, dst.workers))
            if len(src.workers) > 1 and paired and cuda_ipc is not False:
                # trainer rank r and sampler replica r share a process: every rank runs the in-process kernel at
                # the same time (under stage 3 it gathers the peers' shards, a collective)
                from concurrent.futures import ThreadPoolExecutor
                with ThreadPoolExecutor(max_workers=len(src.workers)) as pool:
                    outs = list(pool.map(lambda p: sync_pair(p[0], p[1], cuda_ipc=cuda_ipc), zip(src.workers, dst.workers)))
                total += sum(o["num_tensors"] for o in outs)
                strategies.update(o["strategy"] for o in outs)
                continue
            if sharded and not all(getattr(w, "obj", None) is not None for w in list(src.workers) + list(dst.workers)):
                # parameters exist only as shards spread over the source ranks: every rank takes part in the
                # gather, rank 0 hands the full tensors over, every target loads them
                from .utils.weight_sync import load_staged
                weights = call_all(src.workers, "get_weights", None, 0)[0]
                for dw in dst.workers:
                    total += load_staged(dw, weights)
                strategies.add("gather_bulk")
                continue
            for i, dw in enumerate(dst.workers):
                sw = src.workers[i % len(src.workers)]
                r = sync_pair(sw, dw, cuda_ipc=cuda_ipc, low_memory=low_memory,
                              via_file=bool(src.config.get("weight_sync_via_file")))
                total += r["num_tensors"]
                strategies.add(r["strategy"])
        return {"status": "ok", "num_tensors": total, "seconds": time.perf_counter() - t0,
                "strategies": sorted(strategies)}

    def weight_norm(self, training_job_id: Optional[int] = None, sampling_job_id: Optional[int] = None) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        if training_job_id is not None:
            r = call_all(self._job(training_job_id).workers, "weight_norm")[0]      # sharded engines: a collective
            out["training_norm"], out["training_num_params"] = r["norm"], r["num_params"]
        if sampling_job_id is not None:
            r = call_all(self._replicas(self._job(sampling_job_id))[0], "weight_norm")[0]   # a replica's ranks together
            out["sampling_norm"], out["sampling_num_params"] = r["norm"], r["num_params"]
        return out

    # ------------------------------------------------------------------ sleep / wake
    def sleep_inference(self, job_id: int, level: int = 1) -> Dict[str, Any]:
        job = self._job(job_id, ("sampling",))
        call_all(job.workers, "sleep_inference", None, level, peer_grace_s=None)
        return {"job_id": job.job_id, "status": "sleeping"}

    def wake_inference(self, job_id: int, tags=None) -> Dict[str, Any]:
        job = self._job(job_id, ("sampling",))
        if self.colocate:
            # the sampler is about to take its weights / KV memory back: return what the training engines of the same
            # GPUs only hold as allocator cache first (arctic_platform/common/ray_server.py:266-288)
            with self._lock:
                trainers = [j for j in self.jobs.values() if j.job_type in ("training", "log_prob") and j.status == "RUNNING"]
            for tj in trainers:
                try:
                    call_all(tj.workers, "empty_cache")
                except Exception:
                    pass
        call_all(job.workers, "wake_inference", None, tags, peer_grace_s=None)
        return {"job_id": job.job_id, "status": "awake"}

    def reset_prefix_cache(self, job_id: int) -> Dict[str, Any]:
        job = self._job(job_id, ("sampling",))
        call_all(job.workers, "reset_prefix_cache", peer_grace_s=None)
        return {"job_id": job.job_id, "status": "ok"}

    def sleep_training(self, job_id: int, mode: str = "all") -> Dict[str, Any]:
        job = self._job(job_id, ("training", "log_prob"))
        method = {"all": "offload_to_cpu", "non_lp": "offload_non_lp_states", "lp_params": "offload_lp_params"}.get(mode)
        if method is None:
            raise JobError(400, f"unknown sleep mode {mode!r}")
        call_all(job.workers, method)
        return {"job_id": job.job_id, "status": "sleeping", "mode": mode}

    def wake_training(self, job_id: int) -> Dict[str, Any]:
        job = self._job(job_id, ("training", "log_prob"))
        call_all(job.workers, "backload_to_gpu")
        return {"job_id": job.job_id, "status": "awake"}

    def operation(self, operation_type: str, sub_job_id: int, payload: Optional[dict] = None) -> Dict[str, Any]:
        payload = payload or {}
        if operation_type == "weight-sync":
            return self.weight_sync(payload.get("source_sub_job_id", sub_job_id), payload.get("target_sub_job_ids", []))
        if operation_type == "reset-prefix-cache":
            return self.reset_prefix_cache(sub_job_id)
        if operation_type == "sleep-inference":
            return self.sleep_inference(sub_job_id, payload.get("level", 1))
        if operation_type == "wake-inference":
            return self.wake_inference(sub_job_id, payload.get("tags"))
        raise JobError(400, f"unknown operation {operation_type!r}")

    # ------------------------------------------------------------------ status
    def status(self) -> Dict[str, Any]:
        with self._lock:
            return {"jobs": [dict(j.info, status=j.status) for j in self.jobs.values()]}

    def get_job_status(self, job_id: int) -> Dict[str, Any]:
        with self._lock:
            j = self.jobs.get(int(job_id))
        if j is None:
            raise JobError(404, f"unknown job {job_id}")
        return dict(j.info, status=j.status)
