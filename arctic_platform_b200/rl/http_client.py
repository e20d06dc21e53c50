"""HTTP client of the job server: DSSST1 frames on the tensor routes, JSON elsewhere.

Same surface as the in-process client and as the reference's ``ArcticRLHttpClient``
(arctic_platform/rl/http_client.py:68-729): optional launch of a local server subprocess with
``/health`` polling bounded by ``startup_timeout`` (fail fast when the subprocess dies), stale-job
clean-up, job initialisation in the order sampling -> log_prob -> training, ``RUNNING`` polling bounded by
``job_ready_timeout``, SIGTERM -> wait -> SIGKILL shutdown and an ``atexit`` hook.
"""
from __future__ import annotations

import atexit
import subprocess
import sys
import time
from typing import Any, Dict, List, Optional

import requests

from ..utils.record_replay import record_replay_generation
from .. import wire
from .config import ArcticRLClientConfig
from .local_client import job_config_from, run_sync

OCTET = {"Content-Type": "application/octet-stream"}
HTTP_JOB_ORDER = ("sampling", "log_prob", "training")


class ServerLaunchError(RuntimeError):
    pass


class ArcticRLHttpClient:
    def __init__(self, config: ArcticRLClientConfig, session: Optional[requests.Session] = None):
        self.config = config
        self.base = f"http://{config.host}:{config.port}"
        self._session = session or requests.Session()
        self._proc: Optional[subprocess.Popen] = None
        self.job_ids: Dict[str, Optional[int]] = {"training": config.training_job_id,
                                                  "sampling": config.sampling_job_id,
                                                  "log_prob": config.log_prob_job_id}
        if config.training_job_id is None and config.sampling_job_id is None and config.log_prob_job_id is None:
            if config.backend == "local" and not self._healthy():
                self._launch_local_server()
            self._cleanup_stale_jobs()
            self._initialize_jobs()
            self._wait_for_jobs_running()

    # ------------------------------------------------------------------ server process
    def _healthy(self) -> bool:
        try:
            return self._session.get(f"{self.base}/health", timeout=2).status_code == 200
        except requests.RequestException:
            return False

    def _launch_local_server(self) -> None:
        c = self.config
        cmd = [sys.executable, "-m", "arctic_platform_b200.common.http_server", "--host", str(c.host), "--port",
               str(c.port), "--training-gpus", str(c.training_gpus), "--sampling-gpus", str(c.sampling_gpus),
               "--log-prob-gpus", str(c.log_prob_gpus), "--log-prob-engine", c.log_prob_engine]
        if c.colocate:
            cmd.append("--colocate")
        out = None if c.server_logs else subprocess.DEVNULL
        self._proc = subprocess.Popen(cmd, stdout=out, stderr=out)
        atexit.register(self._kill_server)
        deadline = time.time() + c.startup_timeout
        while time.time() < deadline:
            if self._proc.poll() is not None:
                raise ServerLaunchError(f"local server exited with code {self._proc.returncode} during start-up")
            if self._healthy():
                return
            time.sleep(c.health_check_interval)
        self._kill_server()
        raise ServerLaunchError(f"local server did not become healthy within {c.startup_timeout}s")

    def _kill_server(self) -> None:
        p = self._proc
        if p is None or p.poll() is not None:
            return
        p.terminate()
        try:
            p.wait(10)
        except subprocess.TimeoutExpired:
            p.kill()
        self._proc = None

    def _cleanup_stale_jobs(self) -> None:
        try:
            jobs = self._session.get(f"{self.base}/status", timeout=10).json().get("jobs", [])
        except (requests.RequestException, ValueError):
            return
        for j in jobs:
            self._session.post(f"{self.base}/destroy", params={"job_id": j["job_id"]}, timeout=60)

    def _initialize_jobs(self) -> None:
        counts = {"training": self.config.training_gpus, "sampling": self.config.sampling_gpus,
                  "log_prob": self.config.log_prob_gpus}
        for kind in HTTP_JOB_ORDER:
            if counts[kind] > 0:
                r = self._session.post(f"{self.base}/initialize", json=job_config_from(self.config, kind, counts[kind]),
                                       timeout=self.config.job_ready_timeout)
                self._raise(r)
                self.job_ids[kind] = r.json()["job_id"]

    def _wait_for_jobs_running(self) -> None:
        deadline = time.time() + self.config.job_ready_timeout
        for kind, jid in self.job_ids.items():
            while jid is not None:
                st = self._session.get(f"{self.base}/job/{jid}", timeout=10).json().get("status")
                if st == "RUNNING":
                    break
                if st in ("FAILED", "DESTROYED") or time.time() > deadline:
                    raise RuntimeError(f"{kind} job {jid} is {st}")
                time.sleep(self.config.health_check_interval)

    # ------------------------------------------------------------------ plumbing
    @staticmethod
    def _raise(resp) -> None:
        if resp.status_code >= 400:
            try:
                detail = resp.json().get("detail")
            except ValueError:
                detail = resp.text
            raise RuntimeError(f"server returned {resp.status_code}: {detail}")

    # job ids as attributes (arctic_platform/rl/http_client.py:323-341 in the reference)
    @property
    def training_job_id(self) -> Optional[int]:
        return self.job_ids.get("training")

    @property
    def sampling_job_id(self) -> Optional[int]:
        return self.job_ids.get("sampling")

    @property
    def log_prob_job_id(self) -> Optional[int]:
        return self.job_ids.get("log_prob")

    def _need(self, kind: str) -> int:
        jid = self.job_ids.get(kind)
        if jid is None:
            raise RuntimeError(f"no {kind} job")
        return jid

    def _octet(self, route: str, job_id: int, obj: Any) -> Any:
        r = self._session.post(f"{self.base}{route}", params={"job_id": job_id}, data=wire.dumps(obj), headers=OCTET)
        self._raise(r)
        return wire.loads(r.content)

    def _json(self, route: str, params=None, body=None) -> Any:
        r = self._session.post(f"{self.base}{route}", params=params, json=body)
        self._raise(r)
        return r.json()

    # ------------------------------------------------------------------ API
    async def fwd_bwd(self, batch: Dict[str, Any], processing: Optional[dict] = None, router_replay=None):
        payload = batch if "batch" in batch else {"batch": batch}
        if processing is not None:
            payload = {**payload, "processing": processing}
        return self._octet("/forward-backward", self._need("training"), payload)

    async def fwd_no_grad(self, batch: Dict[str, Any], reference_model: bool = False):
        payload = batch if "batch" in batch else {"batch": batch}
        kind = "log_prob" if (reference_model and self.job_ids.get("log_prob") is not None) else "training"
        return self._octet("/forward", self._need(kind), payload)

    async def step(self, learning_rate: Optional[float] = None):
        return self._json("/step", {"job_id": self._need("training")}, {"learning_rate": learning_rate})

    async def save_checkpoint(self, path=None, step=None, export_hf=False, save_total_limit=None):
        return self._json("/save", {"job_id": self._need("training")},
                          {"path": path, "step": step, "export_hf": export_hf, "save_total_limit": save_total_limit})

    async def load_checkpoint(self, path=None, step=None):
        return self._json("/load-checkpoint", {"job_id": self._need("training")}, {"path": path, "step": step})

    async def recover_training(self, path=None, step=None):
        """Checkpoint + restart of the training job after a failure; this client follows the job to its new id."""
        out = self._json("/recover", {"job_id": self._need("training")}, {"path": path, "step": step})
        self.job_ids["training"] = out["job_id"]
        return out

    async def save_weights(self, path: str):
        return self._json("/save", {"job_id": self._need("training")}, {"path": path, "export_hf": True})

    async def empty_training_cache(self):
        return self._json("/empty-training-cache", {"job_id": self._need("training")})

    @record_replay_generation
    async def generate(self, prompts: List[Any], sampling_params: Optional[dict] = None) -> List[dict]:
        return self._octet("/generate", self._need("sampling"), {"prompts": prompts, "sampling_params": sampling_params})["results"]

    async def log_probs(self, prompts, completions, top_k: int = 1):
        # the scorer: the log-prob job, else the trainer, else (a sampling-only client) the sampler's own replicas
        kind = next((k for k in ("log_prob", "training", "sampling") if self.job_ids.get(k) is not None), "log_prob")
        return self._json("/log-probs", {"job_id": self._need(kind)},
                          {"prompts": prompts, "completions": completions, "top_k": top_k})

    async def sleep_inference(self, level: int = 1):
        return self._json("/sleep-inference", {"job_id": self._need("sampling"), "level": level})

    async def wake_inference(self, tags: Optional[List[str]] = None):
        return self._json("/wake-inference", {"job_id": self._need("sampling")}, tags)

    async def reset_prefix_cache(self):
        return self._json("/reset-prefix-cache", {"job_id": self._need("sampling")})

    async def sleep_training(self, mode: str = "all"):
        return self._json("/sleep-training", {"job_id": self._need("training"), "mode": mode})

    async def wake_training(self):
        return self._json("/wake-training", {"job_id": self._need("training")})

    async def sleep_log_prob(self):
        if self.job_ids.get("log_prob") is None:
            return {"status": "no_log_prob_job"}
        return self._json("/sleep-log-prob", {"job_id": self.job_ids["log_prob"]})

    async def wake_log_prob(self):
        if self.job_ids.get("log_prob") is None:
            return {"status": "no_log_prob_job"}
        return self._json("/wake-log-prob", {"job_id": self.job_ids["log_prob"]})

    async def sync_weights(self, cuda_ipc: Optional[bool] = None, low_memory: Optional[bool] = None):
        sid = self._need("sampling")
        self._json("/wake-inference", {"job_id": sid}, ["weights"])
        out = self._json("/weight-sync", None, {"source_sub_job_id": self._need("training"), "target_sub_job_ids": [sid],
                                                "cuda_ipc": cuda_ipc, "low_memory": low_memory})
        self._json("/wake-inference", {"job_id": sid}, ["kv_cache"])
        self._json("/reset-prefix-cache", {"job_id": sid})
        return out

    async def weight_norm(self):
        return self._json("/weight-norm", None, {"training_job_id": self.job_ids.get("training"),
                                                 "sampling_job_id": self.job_ids.get("sampling")})

    def reconnect_config(self) -> ArcticRLClientConfig:
        cfg = self.config.model_copy()
        cfg.training_job_id = self.job_ids.get("training")
        cfg.sampling_job_id = self.job_ids.get("sampling")
        cfg.log_prob_job_id = self.job_ids.get("log_prob")
        return cfg

    def get_server_state(self):
        return self._session.get(f"{self.base}/status", timeout=10).json()

    async def shutdown(self) -> None:
        try:
            self._session.post(f"{self.base}/destroy", timeout=60)
        except requests.RequestException:
            pass
        self._kill_server()

    def call(self, name: str, *args, **kwargs):
        return run_sync(getattr(self, name)(*args, **kwargs))
