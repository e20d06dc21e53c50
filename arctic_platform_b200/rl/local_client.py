"""In-process RL client: the public client surface driving engines that live in the calling process.

Method set and return shapes are those of the reference's async clients
(arctic_platform/rl/http_client.py:343-729, rl/ray_client.py:214-480): ``fwd_bwd``, ``fwd_no_grad``, ``step``,
``generate``, ``sync_weights``, ``weight_norm``, ``log_probs``, ``sleep_*`` / ``wake_*``, ``save_checkpoint``,
``load_checkpoint``, ``reconnect_config``, ``shutdown``.  Calls are coroutines like the reference's; the
``*_sync`` twins run them to completion for scripts and benchmarks.

Under ``torchrun`` every rank builds its own client over its own GPU: training ranks meet inside the
engine's fused gradient kernels, sampler replicas are independent, and the batch handed to ``fwd_bwd`` is
the rank's shard (``meta['dp_size']`` and the global normalisers are filled in from the process group).
"""
from __future__ import annotations

import asyncio
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils.record_replay import record_replay_generation
from ..common.server import ArcticRLServerCore
from .config import ArcticRLClientConfig

JOB_ORDER = ("training", "sampling", "log_prob")


def job_config_from(cfg: ArcticRLClientConfig, job_type: str, num_devices: int) -> Dict[str, Any]:
    """The ``JobConfig`` body a client sends to ``/initialize`` for one engine kind."""
    return {
        "model_name": cfg.model_name, "job_type": job_type, "num_devices": num_devices,
        "ds_config": cfg.ds_config, "training_config": cfg.training_config,
        "log_prob_config": cfg.log_prob_ds_config, "ds_worker_config": cfg.ds_worker_config,
        "vllm_config": cfg.vllm_config, "checkpoint_path": cfg.checkpoint_path,
        "arctic_inference_config": cfg.arctic_inference_config, "full_determinism": cfg.full_determinism,
        "seed": cfg.seed, "cuda_ipc": cfg.cuda_ipc, "low_memory": cfg.low_memory,
    }


class ArcticRLLocalClient:
    def __init__(self, config: ArcticRLClientConfig, server: Optional[ArcticRLServerCore] = None):
        self.config = config
        self.server = server or ArcticRLServerCore(colocate=config.colocate)
        self.job_ids: Dict[str, Optional[int]] = {"training": config.training_job_id,
                                                  "sampling": config.sampling_job_id,
                                                  "log_prob": config.log_prob_job_id}
        if config.training_job_id is None:
            self._initialize_jobs()

    @property
    def spmd_world(self) -> int:
        """Ranks of the SPMD job this client is one rank of.  Read when needed: the process group may be created by
        the caller before the client exists, or by the first engine during job initialisation."""
        return dist.get_world_size() if dist.is_initialized() else 1

    def _initialize_jobs(self) -> None:
        counts = {"training": self.config.training_gpus, "sampling": self.config.sampling_gpus,
                  "log_prob": self.config.log_prob_gpus}
        for kind in JOB_ORDER:
            if counts[kind] > 0:
                # in-process engines: this process contributes ONE device per job (SPMD ranks add the rest)
                info = self.server.initialize(job_config_from(self.config, kind, 1))
                self.job_ids[kind] = info["job_id"]

    # ------------------------------------------------------------------ helpers
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
            raise RuntimeError(f"no {kind} job (set {kind}_gpus > 0)")
        return jid

    def _with_global_meta(self, payload: Dict[str, Any]) -> Dict[str, Any]:
        """SPMD: ``dp_size`` and the global token / sample counts come from the process group."""
        payload = dict(payload)
        meta = dict(payload.get("meta") or {})
        batch = payload.get("batch")
        if self.spmd_world > 1 and isinstance(batch, dict):
            meta.setdefault("dp_size", self.spmd_world)
            dev = "cuda" if torch.cuda.is_available() else "cpu"
            if "batch_num_tokens" not in meta and "response_mask" in batch:
                t = torch.tensor([float(batch["response_mask"].sum()), float(batch["input_ids"].shape[0])],
                                 dtype=torch.float64, device=dev)
                dist.all_reduce(t)
                meta["batch_num_tokens"], meta["global_batch_size"] = float(t[0]), float(t[1])
        payload["meta"] = meta
        return payload

    # ------------------------------------------------------------------ training
    async def fwd_bwd(self, batch: Dict[str, Any], processing: Optional[dict] = None, router_replay=None) -> Dict[str, Any]:
        payload = batch if "batch" in batch else {"batch": batch}
        if processing is not None:
            payload = {**payload, "processing": processing}
        return self.server.forward_backward(self._need("training"), self._with_global_meta(payload))

    async def fwd_no_grad(self, batch: Dict[str, Any], reference_model: bool = False) -> Dict[str, Any]:
        payload = batch if "batch" in batch else {"batch": batch}
        kind = "log_prob" if (reference_model and self.job_ids.get("log_prob") is not None) else "training"
        return self.server.forward(self._need(kind), self._with_global_meta(payload))

    async def step(self, learning_rate: Optional[float] = None) -> Dict[str, Any]:
        return self.server.step(self._need("training"), learning_rate)

    async def save_checkpoint(self, path: Optional[str] = None, step: Optional[int] = None, export_hf: bool = False,
                              save_total_limit: Optional[int] = None) -> Dict[str, Any]:
        return self.server.save(self._need("training"), path, step, export_hf, save_total_limit)

    async def load_checkpoint(self, path: Optional[str] = None, step: Optional[int] = None) -> Dict[str, Any]:
        return self.server.load_checkpoint(self._need("training"), path, step)

    async def recover_training(self, path: Optional[str] = None, step: Optional[int] = None) -> Dict[str, Any]:
        """Checkpoint + restart of the training job after a failure; this client follows the job to its new id."""
        out = self.server.recover(self._need("training"), path, step)
        self.job_ids["training"] = out["job_id"]
        return out

    async def save_weights(self, path: str) -> Dict[str, Any]:
        """Hugging Face safetensors export of the current training weights."""
        return self.server.save(self._need("training"), path, None, True, None)

    async def empty_training_cache(self) -> Dict[str, Any]:
        return self.server.empty_training_cache(self._need("training"))

    # ------------------------------------------------------------------ rollout
    @record_replay_generation
    async def generate(self, prompts: List[List[int]], sampling_params: Optional[dict] = None) -> List[dict]:
        return self.server.generate(self._need("sampling"), prompts, sampling_params)["results"]

    async def log_probs(self, prompts, completions, top_k: int = 1) -> Dict[str, Any]:
        # the scorer: the log-prob job, else the trainer, else (a sampling-only client) the sampler's own replicas
        kind = next((k for k in ("log_prob", "training", "sampling") if self.job_ids.get(k) is not None), "log_prob")
        return self.server.log_probs(self._need(kind), prompts, completions, top_k)

    async def sleep_inference(self, level: int = 1) -> Dict[str, Any]:
        return self.server.sleep_inference(self._need("sampling"), level)

    async def wake_inference(self, tags: Optional[List[str]] = None) -> Dict[str, Any]:
        return self.server.wake_inference(self._need("sampling"), tags)

    async def reset_prefix_cache(self) -> Dict[str, Any]:
        return self.server.reset_prefix_cache(self._need("sampling"))

    async def sleep_training(self, mode: str = "all") -> Dict[str, Any]:
        return self.server.sleep_training(self._need("training"), mode)

    async def wake_training(self) -> Dict[str, Any]:
        return self.server.wake_training(self._need("training"))

    async def sleep_log_prob(self) -> Dict[str, Any]:
        if self.job_ids.get("log_prob") is None:
            return {"status": "no_log_prob_job"}
        return self.server.sleep_training(self.job_ids["log_prob"], "all")

    async def wake_log_prob(self) -> Dict[str, Any]:
        if self.job_ids.get("log_prob") is None:
            return {"status": "no_log_prob_job"}
        return self.server.wake_training(self.job_ids["log_prob"])

    # ------------------------------------------------------------------ weights
    async def sync_weights(self, cuda_ipc: Optional[bool] = None, low_memory: Optional[bool] = None) -> Dict[str, Any]:
        """wake(weights) -> weight sync -> wake(kv_cache) -> reset prefix cache (the staging the reference's
        HTTP client performs, arctic_platform/rl/http_client.py:625-678)."""
        targets = [self._need("sampling")]
        self.server.wake_inference(targets[0], ["weights"])
        out = self.server.weight_sync(self._need("training"), targets, cuda_ipc, low_memory)
        self.server.wake_inference(targets[0], ["kv_cache"])
        self.server.reset_prefix_cache(targets[0])
        return out

    async def weight_norm(self) -> Dict[str, Any]:
        return self.server.weight_norm(self.job_ids.get("training"), self.job_ids.get("sampling"))

    # ------------------------------------------------------------------ session
    def reconnect_config(self) -> ArcticRLClientConfig:
        cfg = self.config.model_copy()
        cfg.training_job_id = self.job_ids.get("training")
        cfg.sampling_job_id = self.job_ids.get("sampling")
        cfg.log_prob_job_id = self.job_ids.get("log_prob")
        return cfg

    def get_server_state(self) -> ArcticRLServerCore:
        return self.server

    async def shutdown(self) -> None:
        self.server.destroy()

    # blocking twins
    def call(self, name: str, *args, **kwargs):
        return run_sync(getattr(self, name)(*args, **kwargs))


def run_sync(coro):
    try:
        loop = asyncio.get_running_loop()
    except RuntimeError:
        loop = None
    if loop is None:
        return asyncio.run(coro)
    raise RuntimeError("run_sync called from a running event loop; await the coroutine instead")
