"""Flat SFT client configuration (arctic_platform/sft/config.py:39-148 in the reference): a training job
is mandatory, a checkpoint path is required unless reconnecting, ``to_rl_config()`` lowers it to the
unified RL client configuration."""
from __future__ import annotations

from typing import Any, Dict, Literal, Optional

from pydantic import BaseModel, ConfigDict, Field, model_validator

from ..client.config import ArcticRLClientConfig, OnPremConfig, SamplingConfig, TrainingConfig


class ArcticSFTClientConfig(BaseModel):
    model_config = ConfigDict(extra="forbid", protected_namespaces=())
    backend: Literal["onprem"] = "onprem"
    comm_protocol: Literal["http", "ray", "local"] = "http"
    model_name: str
    seed: Optional[int] = None
    max_seq_len: int = 2048
    training_gpus: int = Field(..., description="number of training GPUs (> 0)")
    sampling_gpus: int = 0
    colocate: bool = False
    cuda_ipc: bool = False
    low_memory: bool = False
    vllm_config: Optional[Dict[str, Any]] = None
    host: str = "localhost"
    port: int = 8000
    launch_local_server: bool = False
    server_cuda_visible_devices: Optional[str] = None
    startup_timeout: float = 600.0
    job_ready_timeout: float = 1800.0
    request_timeout: float = 1800.0
    ds_config: Optional[Dict[str, Any]] = None
    ds_worker_config: Optional[Dict[str, Any]] = None
    checkpoint_path: Optional[str] = None
    training_job_id: Optional[Any] = None
    sampling_job_id: Optional[Any] = None

    @model_validator(mode="after")
    def _check(self):
        if self.training_job_id is None:
            if self.training_gpus <= 0:
                raise ValueError("training_gpus must be > 0")
            if not self.checkpoint_path:
                raise ValueError("checkpoint_path is required (unless reconnecting with training_job_id)")
        return self

    def to_rl_config(self) -> ArcticRLClientConfig:
        return ArcticRLClientConfig(
            model_name=self.model_name, seed=42 if self.seed is None else self.seed, max_seq_len=self.max_seq_len,
            training_gpus=self.training_gpus, sampling_gpus=self.sampling_gpus,
            job_ready_timeout=self.job_ready_timeout, request_timeout=self.request_timeout,
            training=TrainingConfig(checkpoint_path=self.checkpoint_path, ds_config=self.ds_config or {},
                                    ds_worker_config=self.ds_worker_config, cuda_ipc=self.cuda_ipc,
                                    low_memory=self.low_memory),
            sampling=SamplingConfig(vllm=self.vllm_config or {}),
            backend=OnPremConfig(protocol=self.comm_protocol, host=self.host, port=self.port, colocate=self.colocate,
                                 launch_local_server=self.launch_local_server,
                                 server_cuda_visible_devices=self.server_cuda_visible_devices,
                                 startup_timeout=self.startup_timeout),
            training_job_id=self.training_job_id, sampling_job_id=self.sampling_job_id)
