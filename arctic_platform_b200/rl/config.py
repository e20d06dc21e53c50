"""Client-side configuration of an RL job (same field names and defaults as the reference's
``ArcticRLClientConfig``, arctic_platform/rl/config.py:28-165), plus ``comm_protocol="local"``:
engines run inside the calling process (one process per GPU, SPMD under ``torchrun`` for more than one
GPU), which is what benchmarks and single-node recipes use.
"""
from __future__ import annotations

import socket
from typing import Literal, Optional

from pydantic import BaseModel, Field, model_validator


def primary_ip() -> str:
    """This node's routable IPv4 address (falls back to loopback)."""
    try:
        with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as s:
            s.connect(("10.255.255.255", 1))
            return s.getsockname()[0]
    except OSError:
        return "127.0.0.1"


class ArcticRLClientConfig(BaseModel):
    backend: Literal["local", "dss-platform"] = "local"
    comm_protocol: Literal["http", "ray", "local"] = "http"
    checkpoint_path: Optional[str] = None
    host: Optional[str] = None
    port: Optional[int] = None

    model_name: str = Field(description="Preset name, Hugging Face id or checkpoint directory loaded on all engines.")
    ds_config: dict = Field(default_factory=dict, description="DeepSpeed-style config of the training engine.")
    training_config: Optional[dict] = None
    vllm_config: Optional[dict] = Field(default=None, description="Sampler overrides (max_model_len, max_num_seqs, ...).")
    log_prob_ds_config: Optional[dict] = None
    ds_worker_config: Optional[dict] = None
    arctic_inference_config: Optional[dict] = None
    full_determinism: bool = False
    seed: int = 42

    training_gpus: int = 0
    sampling_gpus: int = 0
    log_prob_gpus: int = 0
    log_prob_engine: Literal["vllm", "deepspeed"] = "vllm"
    colocate: bool = False
    cuda_ipc: bool = False
    low_memory: bool = False
    server_logs: bool = True
    ray_auto_attach: bool = True
    startup_timeout: float = 300.0
    health_check_interval: float = 2.0
    job_ready_timeout: float = 600.0

    # reconnect ids: when set the client attaches to running jobs instead of initialising new ones
    training_job_id: Optional[int] = Field(default=None, exclude=True)
    sampling_job_id: Optional[int] = Field(default=None, exclude=True)
    log_prob_job_id: Optional[int] = Field(default=None, exclude=True)

    @model_validator(mode="after")
    def _derive_host_port(self) -> "ArcticRLClientConfig":
        networked = self.comm_protocol == "http"
        if "host" not in self.model_fields_set:
            self.host = primary_ip() if networked else None
        if "port" not in self.model_fields_set:
            self.port = 7000 if networked else None
        return self

    @model_validator(mode="after")
    def _validate_local_gpu_counts(self) -> "ArcticRLClientConfig":
        if self.backend != "local" or self.training_job_id is not None:
            return self
        if self.training_gpus + self.sampling_gpus + self.log_prob_gpus <= 0:
            raise ValueError("Local backend requires at least one of training_gpus / sampling_gpus / log_prob_gpus > 0.")
        return self


class WeightSyncConfig(BaseModel):
    """Topology of a trainer -> sampler weight transfer for frameworks that own their training ranks."""
    training_sharding: str = Field(default="dp", description="'dp' or 'fsdp'")
    training_gpus: int = 1
    inference_replicas: int = 1
    inference_tp: int = 1
    base_port: int = 29500
    bucket_size: int = 256 * 1024 * 1024
