"""Ray transport of the unified client: the job server core lives in a 0-GPU Ray actor and every request is an
actor method call -- no HTTP, no wire encoding.

What the reference's ``RayTransport`` offers (arctic_platform/client/transports/onprem_ray.py:28-146) and how it is
done here:

* **one private event loop** for all synchronous calls (created once, not per call).  A synchronous call made from a
  thread whose own loop is running (an async framework calling the sync API) hops to a helper thread instead of
  nesting ``run_until_complete``;
* **asynchronous calls** wait for the actor's reply without blocking the caller's loop (the blocking ``ray.get``
  runs in the loop's default executor);
* **picklable**: the transport travels inside a client object that frameworks ship to other actors (verl hands a
  reconnected backend to its rollout server actor); the loop is dropped on pickling and rebuilt on the other side,
  the actor handle is what addresses the running server;
* **reconnect**: given an existing state actor (plus job ids in the config) the transport attaches to the running
  jobs, creates nothing and -- not owning the jobs -- destroys nothing on ``shutdown``;
* the op -> method table is checked against the server core up front, so a missing method fails at construction and
  not in the middle of a training run.

Without Ray installed ``create_arctic_rl_ray_server_state`` hosts the core in this process and the same transport
works on it (calls are then plain method calls).
"""
from __future__ import annotations

import asyncio
import concurrent.futures
from typing import Any, Optional

from ...common.server import ArcticRLServerCore, JobError
from ..config import ArcticRLClientConfig
from ..transport import JobHandles, Request, Transport, unresolved_ops
from .onprem import dispatch_to_core

RAY_JOB_ORDER = ("training", "sampling", "log_prob")


class RayTransport(Transport):
    def __init__(self, config: ArcticRLClientConfig, server_state: Any = None):
        self.config = config
        self._reconnect = server_state is not None
        if server_state is None:
            from ...rl.ray_client import create_arctic_rl_ray_server_state
            server_state = create_arctic_rl_ray_server_state(colocate=getattr(config.backend, "colocate", False))
        self._state = server_state
        missing = unresolved_ops(ArcticRLServerCore)
        if missing:
            raise RuntimeError(f"server core lacks methods for ops {missing}")
        self.jobs = JobHandles.from_config(config)
        self._loop = asyncio.new_event_loop()

    # -- pickling: everything but the loop --------------------------------------------------------------------
    def __getstate__(self) -> dict:
        state = dict(self.__dict__)
        state.pop("_loop", None)
        return state

    def __setstate__(self, state: dict) -> None:
        self.__dict__.update(state)
        self._loop = asyncio.new_event_loop()

    def get_server_state(self) -> Any:
        """The state actor (or in-process core): hand it to another process's ``RayTransport`` to reattach."""
        return self._state

    # -- jobs ---------------------------------------------------------------------------------------------------
    def initialize(self) -> JobHandles:
        if self.jobs.any_set:
            return self.jobs                                   # reconnect: the jobs exist on the shared state
        if self._reconnect:
            raise ValueError("reconnecting to a server state needs the job ids in the client config")
        for jt in RAY_JOB_ORDER:
            if self.config.gpus_for(jt) > 0:
                self.jobs.set(jt, self._state.initialize(self.config.to_onprem(jt))["job_id"])
        return self.jobs

    # -- calls --------------------------------------------------------------------------------------------------
    def _run_on_loop(self, coro):
        try:
            asyncio.get_running_loop()
        except RuntimeError:
            return self._loop.run_until_complete(coro)
        # the calling thread already runs a loop: this one cannot be driven from here
        with concurrent.futures.ThreadPoolExecutor(max_workers=1) as pool:
            return pool.submit(self._loop.run_until_complete, coro).result()

    async def _dispatch(self, request: Request) -> dict:
        loop = asyncio.get_running_loop()
        return await loop.run_in_executor(None, dispatch_to_core, self._state, request)

    def call(self, request: Request) -> dict:
        return self._run_on_loop(self._dispatch(request))

    async def acall(self, request: Request) -> dict:
        return await self._dispatch(request)

    def shutdown(self) -> None:
        try:
            if not self._reconnect:                            # a reattached transport does not own the jobs
                try:
                    self._state.destroy()
                except JobError:
                    pass
        finally:
            if not self._loop.is_closed():
                self._loop.close()
