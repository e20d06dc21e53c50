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
import traceback
from typing import Any, Callable, Dict, Optional


class ActorError(RuntimeError):
    pass


class ActorDied(RuntimeError):
    pass


def _serve(conn, factory: Callable[[], Any], env: Dict[str, str]) -> None:
    os.environ.update(env)
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
        self._proc = ctx.Process(target=_serve, args=(child, factory, env), daemon=True)
        self._proc.start()
        child.close()
        kind, payload = self._recv(start_timeout)
        if kind != "ready":
            self.kill()
            raise ActorError(f"actor failed to start: {payload}")

    def _recv(self, timeout: Optional[float]):
        if not self._conn.poll(timeout):
            raise ActorDied(f"no answer from actor pid {self._proc.pid} within {timeout}s")
        try:
            return self._conn.recv()
        except (EOFError, ConnectionResetError) as exc:
            raise ActorDied(f"actor pid {self._proc.pid} exited (code {self._proc.exitcode})") from exc

    def call(self, method: str, *args, timeout: Optional[float] = None, **kwargs):
        if not self._proc.is_alive():
            raise ActorDied(f"actor pid {self._proc.pid} is not running (code {self._proc.exitcode})")
        try:
            self._conn.send((method, args, kwargs))
        except (BrokenPipeError, OSError) as exc:
            raise ActorDied(f"actor pid {self._proc.pid} is gone") from exc
        kind, payload = self._recv(timeout)
        if kind == "error":
            raise ActorError(payload)
        return payload

    def heartbeat(self, timeout: float = 5.0) -> bool:
        try:
            return bool(self.call("__heartbeat__", timeout=timeout))
        except (ActorDied, ActorError):
            return False

    def kill(self) -> None:
        try:
            if self._proc.is_alive():
                try:
                    self._conn.send(None)
                except Exception:
                    pass
                self._proc.join(2.0)
            if self._proc.is_alive():
                self._proc.terminate()
                self._proc.join(5.0)
            if self._proc.is_alive():
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
