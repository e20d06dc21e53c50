"""Unified RL client: synchronous ``SyncArcticRLClient`` and asynchronous ``ArcticRLClient`` over one
transport abstraction (arctic_platform/client/client.py:38-427 in the reference).  Every public method is
lowered to a canonical ``Request``; the transport (in-process / Ray, HTTP, Cortex) only delivers it."""
from __future__ import annotations

from typing import Any, List, Optional

from ..utils.record_replay import record_replay_generation
from .config import ArcticRLClientConfig, CortexConfig
from .transport import JobHandles, Request, Transport, initialize_or_cleanup


def make_transport(config: ArcticRLClientConfig, server_state: Any = None) -> Transport:
    if isinstance(config.backend, CortexConfig):
        from .transports.cortex import CortexTransport
        return CortexTransport(config)
    if config.backend.protocol == "http":
        from .transports.onprem import HttpTransport
        return HttpTransport(config)
    if config.backend.protocol == "ray":
        from .transports.ray_actor import RayTransport
        return RayTransport(config, server_state)
    from .transports.onprem import CoreTransport
    return CoreTransport(config, server_state)


# ----------------------------------------------------------------------------- request builders
def _payload(batch: dict) -> dict:
    return batch if "batch" in batch else {"batch": batch}


def _fwd_bwd_request(jobs: JobHandles, batch: dict, processing=None, router_replay=None) -> Request:
    body = dict(_payload(batch))
    if processing is not None:
        body["processing"] = processing
    if router_replay is not None:
        body["router_replay"] = router_replay
    return Request("forward-backward", jobs.require("training"), body, binary=True)


def _fwd_no_grad_request(jobs: JobHandles, batch: dict, reference_model: bool = False) -> Request:
    jt = "log_prob" if (reference_model and jobs.log_prob is not None) else "training"
    return Request("forward", jobs.require(jt), dict(_payload(batch)), binary=True)


def _step_request(jobs: JobHandles, learning_rate=None) -> Request:
    return Request("step", jobs.require("training"), {"learning_rate": learning_rate})


def _save_request(jobs, path=None, step=None, export_hf=False, save_total_limit=None) -> Request:
    return Request("save", jobs.require("training"), {"path": path, "step": step, "export_hf": export_hf,
                                                       "save_total_limit": save_total_limit})


def _load_request(jobs, path=None, step=None) -> Request:
    return Request("load-checkpoint", jobs.require("training"), {"path": path, "step": step})


def _generate_request(jobs, prompts, sampling_params=None, routing_key=None, strict=False) -> Request:
    return Request("generate", jobs.require("sampling"), {"prompts": prompts, "sampling_params": sampling_params,
                                                           "routing_key": routing_key, "strict": strict}, binary=True)


def _log_probs_request(jobs, prompts, completions=None, top_k=1) -> Request:
    # the scorer: the log-prob job, else the trainer, else (a sampling-only client) the sampler's own replicas
    jt = next((k for k in ("log_prob", "training", "sampling") if getattr(jobs, k, None) is not None), "log_prob")
    return Request("log-probs", jobs.require(jt), {"prompts": prompts, "completions": completions or [], "top_k": top_k})


def _sync_weights_requests(jobs, cuda_ipc=None, low_memory=None) -> List[Request]:
    s = jobs.require("sampling")
    return [
        Request("wake-inference", s, {"tags": ["weights"]}),
        Request("operation", jobs.require("training"),
                {"operation_type": "weight-sync", "sub_job_id": jobs.require("training"),
                 "payload": {"source_sub_job_id": jobs.require("training"), "target_sub_job_ids": [s],
                             "cuda_ipc": cuda_ipc, "low_memory": low_memory}}),
        Request("wake-inference", s, {"tags": ["kv_cache"]}),
        Request("operation", s, {"operation_type": "reset-prefix-cache", "sub_job_id": s, "payload": {}}),
    ]


def _reconnect_config(config: ArcticRLClientConfig, jobs: JobHandles) -> ArcticRLClientConfig:
    cfg = config.model_copy()
    cfg.training_job_id, cfg.sampling_job_id, cfg.log_prob_job_id = jobs.training, jobs.sampling, jobs.log_prob
    return cfg


class SyncArcticRLClient:
    def __init__(self, config: ArcticRLClientConfig, server_state: Any = None, transport: Optional[Transport] = None):
        self.config = config
        self.transport = transport or make_transport(config, server_state)
        self.jobs = initialize_or_cleanup(self.transport)

    def fwd_bwd(self, batch: dict, processing: Optional[dict] = None, router_replay: Any = None) -> dict:
        return self.transport.call(_fwd_bwd_request(self.jobs, batch, processing, router_replay))

    def fwd_no_grad(self, batch: dict, reference_model: bool = False) -> dict:
        return self.transport.call(_fwd_no_grad_request(self.jobs, batch, reference_model))

    def step(self, learning_rate: Optional[float] = None) -> dict:
        return self.transport.call(_step_request(self.jobs, learning_rate))

    def save_checkpoint(self, path=None, *, step=None, export_hf=False, save_total_limit=None) -> dict:
        return self.transport.call(_save_request(self.jobs, path, step, export_hf, save_total_limit))

    def load_checkpoint(self, path=None, *, step=None) -> dict:
        return self.transport.call(_load_request(self.jobs, path, step))

    @record_replay_generation
    def generate(self, prompts: list, sampling_params: Optional[dict] = None, routing_key=None, strict=False) -> list:
        return self.transport.call(_generate_request(self.jobs, prompts, sampling_params, routing_key, strict))["results"]

    def log_probs(self, prompts: list, completions: Optional[list] = None, top_k: int = 1) -> dict:
        return self.transport.call(_log_probs_request(self.jobs, prompts, completions, top_k))

    def sync_weights(self, cuda_ipc=None, low_memory=None) -> dict:
        out = {}
        for i, r in enumerate(_sync_weights_requests(self.jobs, cuda_ipc, low_memory)):
            res = self.transport.call(r)
            if i == 1:
                out = res
        return out

    def reset_prefix_cache(self, drain: bool = True, timeout_s: float = 60.0, retry_interval_s: float = 0.1) -> dict:
        s = self.jobs.require("sampling")
        return self.transport.call(Request("operation", s, {"operation_type": "reset-prefix-cache", "sub_job_id": s,
                                                            "payload": {"drain": drain, "timeout_s": timeout_s,
                                                                        "retry_interval_s": retry_interval_s}}))

    def sleep_inference(self, level: int = 1) -> dict:
        return self.transport.call(Request("sleep-inference", self.jobs.require("sampling"), {"level": level}))

    def wake_inference(self, tags: Optional[list] = None) -> dict:
        return self.transport.call(Request("wake-inference", self.jobs.require("sampling"), {"tags": tags}))

    def sleep_training(self, mode: str = "all") -> dict:
        return self.transport.call(Request("sleep-training", self.jobs.require("training"), {"mode": mode}))

    def wake_training(self) -> dict:
        return self.transport.call(Request("wake-training", self.jobs.require("training"), {}))

    def reconnect_config(self) -> ArcticRLClientConfig:
        return _reconnect_config(self.config, self.jobs)

    def get_server_state(self) -> Any:
        return getattr(self.transport, "core", None)

    def shutdown(self) -> None:
        self.transport.shutdown()

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.shutdown()


class ArcticRLClient:
    """Async twin: same methods as coroutines, delivered with ``transport.acall``."""

    def __init__(self, config: ArcticRLClientConfig, server_state: Any = None, transport: Optional[Transport] = None):
        self.config = config
        self.transport = transport or make_transport(config, server_state)
        self.jobs = initialize_or_cleanup(self.transport)

    async def fwd_bwd(self, batch, processing=None, router_replay=None):
        return await self.transport.acall(_fwd_bwd_request(self.jobs, batch, processing, router_replay))

    async def fwd_no_grad(self, batch, reference_model=False):
        return await self.transport.acall(_fwd_no_grad_request(self.jobs, batch, reference_model))

    async def step(self, learning_rate=None):
        return await self.transport.acall(_step_request(self.jobs, learning_rate))

    async def save_checkpoint(self, path=None, *, step=None, export_hf=False, save_total_limit=None):
        return await self.transport.acall(_save_request(self.jobs, path, step, export_hf, save_total_limit))

    async def load_checkpoint(self, path=None, *, step=None):
        return await self.transport.acall(_load_request(self.jobs, path, step))

    @record_replay_generation
    async def generate(self, prompts, sampling_params=None, routing_key=None, strict=False):
        return (await self.transport.acall(_generate_request(self.jobs, prompts, sampling_params, routing_key, strict)))["results"]

    async def log_probs(self, prompts, completions=None, top_k=1):
        return await self.transport.acall(_log_probs_request(self.jobs, prompts, completions, top_k))

    async def sync_weights(self, cuda_ipc=None, low_memory=None):
        out = {}
        for i, r in enumerate(_sync_weights_requests(self.jobs, cuda_ipc, low_memory)):
            res = await self.transport.acall(r)
            if i == 1:
                out = res
        return out

    async def reset_prefix_cache(self, drain=True, timeout_s=60.0, retry_interval_s=0.1):
        s = self.jobs.require("sampling")
        return await self.transport.acall(Request("operation", s, {"operation_type": "reset-prefix-cache",
                                                                   "sub_job_id": s, "payload": {"drain": drain}}))

    async def sleep_inference(self, level=1):
        return await self.transport.acall(Request("sleep-inference", self.jobs.require("sampling"), {"level": level}))

    async def wake_inference(self, tags=None):
        return await self.transport.acall(Request("wake-inference", self.jobs.require("sampling"), {"tags": tags}))

    async def sleep_training(self, mode="all"):
        return await self.transport.acall(Request("sleep-training", self.jobs.require("training"), {"mode": mode}))

    async def wake_training(self):
        return await self.transport.acall(Request("wake-training", self.jobs.require("training"), {}))

    def reconnect_config(self) -> ArcticRLClientConfig:
        return _reconnect_config(self.config, self.jobs)

    def get_server_state(self) -> Any:
        return getattr(self.transport, "core", None)

    async def shutdown(self) -> None:
        await self.transport.aclose()
        self.transport.shutdown()

    async def __aenter__(self):
        return self

    async def __aexit__(self, *exc) -> None:
        await self.shutdown()


def create_arctic_rl_client(config: ArcticRLClientConfig, *, blocking_calls: bool = False, server_state: Any = None):
    return SyncArcticRLClient(config, server_state) if blocking_calls else ArcticRLClient(config, server_state)
