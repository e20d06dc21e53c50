"""Spawned-process actors: the stand-in for Ray actors on machines without Ray.

``SpawnedActor`` starts one Python process per worker (``multiprocessing`` spawn context), optionally pinned to
one GPU through ``CUDA_VISIBLE_DEVICES`` and given the ``RANK`` / ``WORLD_SIZE`` / ``MASTER_*`` variables of a
``torch.distributed`` job, and forwards ``call(method, *args)`` over a pipe.  Exceptions in the worker come back
as ``ActorError``; a worker that dies or does not answer within ``timeout`` raises ``ActorDied`` -- the host-side
failure signal the job server turns into all-or-nothing teardown.  ``heartbeat()`` is a cheap liveness probe.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import threading
import traceback
from typing import Any, Callable, Dict, Optional


class ActorError(RuntimeError):
    pass


class ActorDied(RuntimeError):
    pass


def _exit_with_parent(parent_pid: int, period_s: float = 2.0) -> None:
    """A worker must not outlive the server that owns it (it may sit in a collective for ever and hold a GPU): when
    the parent is gone the process ends itself."""
    def watch():
        import time
        while True:
            time.sleep(period_s)
            if os.getppid() != parent_pid:
                os._exit(1)
    threading.Thread(target=watch, name="apb-parent-watch", daemon=True).start()


def _serve(conn, factory: Callable[[], Any], env: Dict[str, str]) -> None:
    os.environ.update(env)
    _exit_with_parent(os.getppid())
    try:
        obj = factory()
        conn.send(("ready", None))
    except BaseException as exc:  # noqa: BLE001 - reported to the parent
        conn.send(("error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
        return
    while True:
        try:
            msg = conn.recv()
        except EOFError:
            return
        if msg is None:
            return
        method, args, kwargs = msg
        try:
            if method == "__heartbeat__":
                conn.send(("ok", True))
                continue
            conn.send(("ok", getattr(obj, method)(*args, **kwargs)))
        except BaseException as exc:  # noqa: BLE001
            conn.send(("error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))


class SpawnedActor:
    def __init__(self, factory: Callable[[], Any], env: Optional[Dict[str, str]] = None, gpu: Optional[int] = None,
                 start_timeout: float = 600.0):
        ctx = mp.get_context("spawn")
        self._conn, child = ctx.Pipe()
        env = dict(env or {})
        if gpu is not None:
            env["CUDA_VISIBLE_DEVICES"] = str(gpu)
        self._lock = threading.Lock()         # one request on the pipe at a time (several jobs may share a process)
        self._proc = ctx.Process(target=_serve, args=(child, factory, env), daemon=True)
        self._proc.start()
        child.close()
        kind, payload = self._recv(start_timeout)
        if kind != "ready":
            self.kill()
            raise ActorError(f"actor failed to start: {payload}")

    def _recv(self, timeout: Optional[float]):
        try:
            if not self._conn.poll(timeout):
                raise ActorDied(f"no answer from actor pid {self._proc.pid} within {timeout}s")
            return self._conn.recv()
        except (EOFError, ConnectionResetError, OSError, ValueError) as exc:    # pipe closed: process gone or stopped
            raise ActorDied(f"actor pid {self._proc.pid} exited (code {self._proc.exitcode})") from exc

    def call(self, method: str, *args, timeout: Optional[float] = None, **kwargs):
        if not self.alive():
            raise ActorDied(f"actor pid {self._proc.pid} is not running (code {self._proc.exitcode})")
        with self._lock:
            try:
                self._conn.send((method, args, kwargs))
            except (BrokenPipeError, OSError) as exc:
                raise ActorDied(f"actor pid {self._proc.pid} is gone") from exc
            kind, payload = self._recv(timeout)
        if kind == "error":
            raise ActorError(payload)
        return payload

    def alive(self) -> bool:
        """Whether the process exists -- never blocks, also while a long call is in flight.  Decided from the process
        sentinel (readable once the process has exited), not from ``Process.is_alive()``: that one reaps the child
        with ``waitpid``, and when two threads ask at the same moment (the watchdog and a caller that is tearing the
        job down) the loser of the race is told "no such child" and reports a dead process as alive."""
        from multiprocessing.connection import wait
        try:
            return not wait([self._proc.sentinel], timeout=0)
        except (ValueError, OSError):            # closed process object
            return False

    def heartbeat(self, timeout: float = 5.0) -> bool:
        try:
            return bool(self.call("__heartbeat__", timeout=timeout))
        except (ActorDied, ActorError):
            return False

    def terminate(self) -> None:
        self.kill(grace_s=0.0)

    def request_destroy(self) -> None:
        """Posts the shutdown message and returns: the process ends by itself once its current call comes back (a
        bounded device wait or the process group's timeout ends a call stuck behind a failed peer).  Used instead of
        ``terminate`` while the ranks' buffers are bound to an NVSwitch multicast object."""
        try:
            self._conn.send(None)
        except Exception:
            pass

    def kill(self, grace_s: float = 2.0) -> None:
        try:
            if self.alive() and grace_s > 0:
                try:
                    self._conn.send(None)
                except Exception:
                    pass
                self._proc.join(grace_s)
            if self.alive():
                self._proc.terminate()
                self._proc.join(5.0)
            if self.alive():                     # the sentinel, not is_alive(): never signal a pid that was reaped
                self._proc.kill()
        finally:
            self._conn.close()


def _make_engine_worker():
    from ..engine.worker import EngineWorker
    return EngineWorker()


def spawned_worker_factory(master_port: int = 29500):
    """``worker_factory`` for ``ArcticRLServerCore``: one spawned process per rank, rank r on GPU r."""
    def factory(job_config: Dict[str, Any], rank: int, world: int):
        import torch
        # every rank sees all GPUs and takes the one named by LOCAL_RANK (as under torchrun): peer mappings of
        # the symmetric buffers need the peers' devices visible.  Each job type rendezvouses on its own port;
        # sampler replicas form no group at all.
        offset = {"training": 0, "log_prob": 1, "sampling": 2}.get(job_config.get("job_type", "training"), 0)
        env = {"RANK": str(rank), "LOCAL_RANK": str(rank if torch.cuda.is_available() else 0), "WORLD_SIZE": str(world),
               "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(master_port + offset)}
        return SpawnedActor(_make_engine_worker, env=env)
    return factory


# ----------------------------------------------------------------------------- one process per GPU, many jobs
class _RankHost:
    """Lives inside a rank's process and owns the engine workers of every job placed on that rank, so that a
    training engine and a sampling engine of the same GPU are in ONE process: the weight hand-over between them is
    the in-process kernel (no copy through the host), and sleep / wake trade the same device memory."""

    def __init__(self) -> None:
        self.workers: Dict[str, Any] = {}

    def create(self, key: str) -> bool:
        from ..engine.worker import EngineWorker
        self.workers[key] = EngineWorker()
        return True

    def invoke(self, key: str, method: str, *args, **kwargs):
        return getattr(self.workers[key], method)(*args, **kwargs)

    def drop(self, key: str) -> bool:
        w = self.workers.pop(key, None)
        if w is not None:
            w.destroy()
        return w is not None

    def sync(self, src_key: str, dst_key: str) -> int:
        return self.workers[src_key].sync_weights_to(self.workers[dst_key])

    def keys(self):
        return sorted(self.workers)


class RankWorkerHandle:
    """What the job server holds for one (rank process, job) pair: the actor interface of a single worker."""

    def __init__(self, actor: SpawnedActor, key: str, rank: int, owns_process: bool = False):
        self.actor, self.key, self.rank, self.owns_process = actor, key, rank, owns_process

    def call(self, method: str, *args, timeout: Optional[float] = None, **kwargs):
        return self.actor.call("invoke", self.key, method, *args, timeout=timeout, **kwargs)

    def heartbeat(self, timeout: float = 5.0) -> bool:
        return self.actor.heartbeat(timeout)

    def alive(self) -> bool:
        return self.actor.alive()

    def sync_to(self, dst: "RankWorkerHandle") -> int:
        """Weight hand-over to another job's engine in the SAME rank process (the in-process kernel runs there)."""
        return self.actor.call("sync", self.key, dst.key)

    def request_destroy(self) -> None:
        self.actor.request_destroy()

    def terminate(self) -> None:
        """Stops the rank's process outright (the job is lost: a peer failed while this rank may be waiting for it
        in a collective, where a polite request would never be read)."""
        self.actor.kill()

    def kill(self) -> None:
        """Ends this job's worker; the rank's process stays for the other jobs (the pool ends processes)."""
        try:
            self.actor.call("drop", self.key, timeout=60.0)
        except (ActorDied, ActorError):
            pass
        if self.owns_process:
            self.actor.kill()


class RankProcessPool:
    """``world`` long-lived rank processes (rank r on GPU r, all GPUs visible, one rendezvous), created on first
    use.  ``factory`` is a ``worker_factory`` for ``ArcticRLServerCore``: jobs whose ranks form a process group
    (training, log-prob) must span the whole pool; sampler jobs may use any prefix of it."""

    def __init__(self, world: int, master_port: int = 29500, colocate: bool = True):
        self.world, self.master_port, self.colocate = int(world), int(master_port), bool(colocate)
        self.actors: Dict[int, SpawnedActor] = {}
        self._ids = 0
        self._lock = threading.Lock()

    def _actor(self, rank: int) -> SpawnedActor:
        with self._lock:
            a = self.actors.get(rank)
            if a is not None and not a.alive():       # the rank's process was lost (or stopped with a failed job)
                a = None
            if a is None:
                import torch
                env = {"RANK": str(rank), "LOCAL_RANK": str(rank if torch.cuda.is_available() else 0),
                       "WORLD_SIZE": str(self.world), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(self.master_port)}
                a = self.actors[rank] = SpawnedActor(_RankHost, env=env)
            return a

    def factory(self, job_config: Dict[str, Any], rank: int, world: int) -> RankWorkerHandle:
        job_type = job_config.get("job_type", "training")
        if job_type == "sampling" and not self.colocate:
            # split placement: sampler replica r gets a process of its own on the GPU after the trainer's GPUs
            import torch
            env = {"RANK": "0", "WORLD_SIZE": "1",
                   "LOCAL_RANK": str(self.world + rank if torch.cuda.is_available() else 0)}
            actor = SpawnedActor(_RankHost, env=env)
            actor.call("create", "sampling", timeout=600.0)
            return RankWorkerHandle(actor, "sampling", rank, owns_process=True)
        if rank >= self.world:
            raise ValueError(f"{job_type} job wants rank {rank} but the pool has {self.world} rank processes")
        if job_type != "sampling" and world != self.world:
            raise ValueError(f"a {job_type} job forms a process group over the whole pool: it needs {self.world} "
                             f"ranks, not {world}")
        with self._lock:
            self._ids += 1
            key = f"{job_type}-{self._ids}"
        actor = self._actor(rank)
        actor.call("create", key, timeout=600.0)
        return RankWorkerHandle(actor, key, rank)

    def shutdown(self) -> None:
        with self._lock:
            actors, self.actors = list(self.actors.values()), {}
        for a in actors:
            a.kill()
