"""On-prem transports: in-process server core (``local`` / ``ray``) and HTTP.

``CoreTransport`` hands a request straight to an ``ArcticRLServerCore`` (in this process, or behind a Ray
actor proxy); ``HttpTransport`` speaks to ``common/http_server.py`` with DSSST1 frames for tensor bodies,
optionally launching the server as a subprocess (with ``server_cuda_visible_devices``) and failing fast if
it dies during start-up.  Contract of arctic_platform/client/transports/onprem*.py.
"""
from __future__ import annotations

import os
import subprocess
import sys
import time
from typing import Any, Dict, Optional

from ... import wire
from ...common.server import ArcticRLServerCore, JobError
from ..config import ArcticRLClientConfig
from ..transport import JOB_CREATE_ORDER, JobHandles, Request, Transport

_ROUTES = {"forward-backward": "/forward-backward", "forward": "/forward", "step": "/step", "save": "/save",
           "load-checkpoint": "/load-checkpoint", "generate": "/generate", "log-probs": "/log-probs",
           "operation": "/operation", "sleep-inference": "/sleep-inference", "wake-inference": "/wake-inference",
           "sleep-training": "/sleep-training", "wake-training": "/wake-training"}


def dispatch_to_core(core, req: Request) -> dict:
    """One canonical op against a server core (or a proxy with the same methods)."""
    b, j = req.body, req.job_id
    if req.op == "forward-backward":
        return core.forward_backward(j, b)
    if req.op == "forward":
        return core.forward(j, b)
    if req.op == "step":
        return core.step(j, b.get("learning_rate"))
    if req.op == "save":
        return core.save(j, b.get("path"), b.get("step"), b.get("export_hf", False), b.get("save_total_limit"))
    if req.op == "load-checkpoint":
        return core.load_checkpoint(j, b.get("path"), b.get("step"))
    if req.op == "generate":
        return core.generate(j, b["prompts"], b.get("sampling_params"), b.get("routing_key"), b.get("strict", False))
    if req.op == "log-probs":
        return core.log_probs(j, b["prompts"], b["completions"], b.get("top_k", 1))
    if req.op == "operation":
        return core.operation(b["operation_type"], b.get("sub_job_id", j), b.get("payload"))
    if req.op == "sleep-inference":
        return core.sleep_inference(j, b.get("level", 1))
    if req.op == "wake-inference":
        return core.wake_inference(j, b.get("tags"))
    if req.op == "sleep-training":
        return core.sleep_training(j, b.get("mode", "all"))
    if req.op == "wake-training":
        return core.wake_training(j)
    raise ValueError(f"unknown op {req.op!r}")


class CoreTransport(Transport):
    def __init__(self, config: ArcticRLClientConfig, server_state: Any = None):
        self.config = config
        self.core = server_state or ArcticRLServerCore(colocate=getattr(config.backend, "colocate", False))
        self.jobs = JobHandles.from_config(config)

    def initialize(self) -> JobHandles:
        if self.jobs.any_set:
            return self.jobs
        order = ("training", "sampling", "log_prob") if self.config.backend.protocol == "ray" else JOB_CREATE_ORDER
        for jt in order:
            if self.config.gpus_for(jt) > 0:
                body = self.config.to_onprem(jt)
                if self.config.backend.protocol == "local":
                    body["num_devices"] = 1
                self.jobs.set(jt, self.core.initialize(body)["job_id"])
        return self.jobs

    def call(self, request: Request) -> dict:
        return dispatch_to_core(self.core, request)

    async def acall(self, request: Request) -> dict:
        return self.call(request)

    def shutdown(self) -> None:
        try:
            self.core.destroy()
        except JobError:
            pass


class HttpTransport(Transport):
    def __init__(self, config: ArcticRLClientConfig, session=None):
        import requests
        self.config = config
        self.backend = config.backend
        self.base = f"http://{self.backend.host}:{self.backend.port}"
        self.session = session or requests.Session()
        self.jobs = JobHandles.from_config(config)
        self._proc: Optional[subprocess.Popen] = None

    # -- server process ------------------------------------------------------------------------------
    def _healthy(self) -> bool:
        try:
            return self.session.get(f"{self.base}/health", timeout=2).status_code == 200
        except Exception:
            return False

    def _launch(self) -> None:
        c = self.config
        env = dict(os.environ)
        if self.backend.server_cuda_visible_devices is not None:
            env["CUDA_VISIBLE_DEVICES"] = self.backend.server_cuda_visible_devices
        cmd = [sys.executable, "-m", "arctic_platform_b200.common.http_server", "--host", self.backend.host, "--port",
               str(self.backend.port), "--training-gpus", str(c.training_gpus), "--sampling-gpus",
               str(c.sampling_gpus), "--log-prob-gpus", str(c.log_prob_gpus)]
        if self.backend.colocate:
            cmd.append("--colocate")
        self._proc = subprocess.Popen(cmd, env=env)
        deadline = time.time() + self.backend.startup_timeout
        while time.time() < deadline:
            if self._proc.poll() is not None:
                code = self._proc.returncode
                self._proc = None
                raise RuntimeError(f"launched server exited with code {code} before becoming healthy")
            if self._healthy():
                return
            time.sleep(0.5)
        self.shutdown()
        raise TimeoutError(f"launched server not healthy after {self.backend.startup_timeout}s")

    def initialize(self) -> JobHandles:
        if self.jobs.any_set:
            return self.jobs
        if self.backend.launch_local_server and not self._healthy():
            self._launch()
        for jt in JOB_CREATE_ORDER:
            if self.config.gpus_for(jt) > 0:
                r = self.session.post(f"{self.base}/initialize", json=self.config.to_onprem(jt),
                                      timeout=self.config.job_ready_timeout)
                self._raise(r)
                self.jobs.set(jt, r.json()["job_id"])
        return self.jobs

    @staticmethod
    def _raise(resp) -> None:
        if resp.status_code >= 400:
            try:
                detail = resp.json().get("detail")
            except ValueError:
                detail = resp.text
            raise RuntimeError(f"server returned {resp.status_code}: {detail}")

    def call(self, request: Request) -> dict:
        url = self.base + _ROUTES[request.op]
        params = {"job_id": request.job_id} if request.job_id is not None else None
        timeout = self.config.request_timeout
        if request.binary:
            r = self.session.post(url, params=params, data=wire.dumps(request.body),
                                  headers={"Content-Type": "application/octet-stream"}, timeout=timeout)
            self._raise(r)
            return wire.loads(r.content)
        body: Any = request.body
        if request.op == "wake-inference":
            body = request.body.get("tags")
        elif request.op in ("sleep-inference", "sleep-training"):
            params = {**(params or {}), **request.body}
            body = None
        r = self.session.post(url, params=params, json=body, timeout=timeout)
        self._raise(r)
        return r.json()

    async def acall(self, request: Request) -> dict:
        import asyncio
        return await asyncio.get_running_loop().run_in_executor(None, self.call, request)

    def shutdown(self) -> None:
        try:
            if self.jobs.any_set:
                self.session.post(f"{self.base}/destroy", timeout=60)
        except Exception:
            pass
        p, self._proc = self._proc, None
        if p is not None and p.poll() is None:
            p.terminate()
            try:
                p.wait(10)
            except subprocess.TimeoutExpired:
                p.kill()
