"""Unified client configuration (``extra="forbid"`` everywhere; backend chosen by a discriminated union on
``backend.type``).  Field names and defaults follow arctic_platform/client/config.py:45-312 in the
reference; ``OnPremConfig.protocol`` additionally accepts ``"local"`` for in-process engines.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Literal, Optional, Union

from pydantic import BaseModel, ConfigDict, Field, model_validator

JOB_TYPES = ("training", "sampling", "log_prob")


class OnPremConfig(BaseModel):
    model_config = ConfigDict(extra="forbid", validate_default=True)
    type: Literal["onprem"] = "onprem"
    protocol: Literal["http", "ray", "local"] = "http"
    host: str = "localhost"
    port: int = 8000
    colocate: bool = False
    launch_local_server: bool = False
    server_cuda_visible_devices: Optional[str] = None
    startup_timeout: float = 600.0


class CortexConfig(BaseModel):
    model_config = ConfigDict(extra="forbid", validate_default=True, populate_by_name=True)
    type: Literal["remote"] = "remote"
    protocol: Literal["cortex"] = "cortex"
    base_url: Optional[str] = None
    host: Optional[str] = None
    pat: Optional[str] = None
    pat_env_var: str = "CORTEX_PAT"
    database: str = ""
    schema_: str = Field("", alias="schema")
    endpoint: str = "cortex-training"
    max_retries: int = Field(10, ge=0)

    def resolve_pat(self) -> Optional[str]:
        return self.pat if self.pat is not None else os.environ.get(self.pat_env_var)

    @model_validator(mode="after")
    def _check(self):
        if not (self.base_url or self.host):
            raise ValueError("cortex: set base_url (direct URL) or host (PAT auth).")
        if self.host and not self.base_url:
            if not (self.database and self.schema_):
                raise ValueError("cortex: database + schema required for host/PAT auth.")
            if not self.resolve_pat():
                raise ValueError(f"cortex: no PAT — set `pat` or the '{self.pat_env_var}' env var for host auth.")
        return self


class SamplingConfig(BaseModel):
    model_config = ConfigDict(extra="forbid", validate_default=True)
    vllm: Dict[str, Any] = Field(default_factory=dict)
    arctic_inference_config: Optional[Dict[str, Any]] = None
    log_prob_engine: Literal["vllm", "deepspeed"] = "vllm"
    log_prob_ds_config: Optional[Dict[str, Any]] = None


class TrainingConfig(BaseModel):
    model_config = ConfigDict(extra="forbid", validate_default=True)
    full_determinism: bool = False
    checkpoint_path: Optional[str] = None
    ds_config: Dict[str, Any] = Field(default_factory=dict)
    ds_worker_config: Optional[Dict[str, Any]] = None
    cuda_ipc: bool = False
    low_memory: bool = False


class ArcticRLClientConfig(BaseModel):
    model_config = ConfigDict(extra="forbid", validate_default=True, protected_namespaces=())
    model_name: str
    seed: int = 42
    dtype: str = "bfloat16"
    max_seq_len: int = 8192
    training_gpus: int = 0
    sampling_gpus: int = 0
    log_prob_gpus: int = 0
    job_ready_timeout: float = 1800.0
    request_timeout: float = 1800.0
    training: TrainingConfig = Field(default_factory=TrainingConfig)
    sampling: SamplingConfig = Field(default_factory=SamplingConfig)
    backend: Union[OnPremConfig, CortexConfig] = Field(default_factory=OnPremConfig, discriminator="type")
    training_job_id: Optional[Any] = Field(default=None, exclude=True)
    sampling_job_id: Optional[Any] = Field(default=None, exclude=True)
    log_prob_job_id: Optional[Any] = Field(default=None, exclude=True)

    @model_validator(mode="after")
    def _need_a_job(self):
        reconnect = any(v is not None for v in (self.training_job_id, self.sampling_job_id, self.log_prob_job_id))
        if not reconnect and self.training_gpus + self.sampling_gpus + self.log_prob_gpus <= 0:
            raise ValueError("set at least one of training_gpus / sampling_gpus / log_prob_gpus > 0")
        return self

    def gpus_for(self, job_type: str) -> int:
        return int(getattr(self, f"{job_type}_gpus"))

    # ------------------------------------------------------------------ wire adapters
    def to_onprem(self, job_type: str) -> Dict[str, Any]:
        """The ``JobConfig`` body an on-prem server expects for ``job_type``."""
        vllm = dict(self.sampling.vllm)
        vllm.setdefault("max_model_len", self.max_seq_len)
        return {
            "model_name": self.model_name, "job_type": job_type, "num_devices": self.gpus_for(job_type),
            "ds_config": self.training.ds_config, "training_config": None,
            "log_prob_config": self.sampling.log_prob_ds_config, "ds_worker_config": self.training.ds_worker_config,
            "vllm_config": vllm, "checkpoint_path": self.training.checkpoint_path,
            "arctic_inference_config": self.sampling.arctic_inference_config,
            "full_determinism": self.training.full_determinism, "seed": self.seed,
            "cuda_ipc": self.training.cuda_ipc, "low_memory": self.training.low_memory,
        }

    def to_cortex(self) -> Dict[str, Any]:
        """Job-creation body of the Cortex (SnowAPI) protocol: one job with sub-jobs per engine kind."""
        sub = []
        for jt in JOB_TYPES:
            if self.gpus_for(jt) > 0:
                sub.append({"sub_job_type": jt, "num_devices": self.gpus_for(jt), "config": self.to_onprem(jt)})
        return {"model_name": self.model_name, "seed": self.seed, "dtype": self.dtype, "max_seq_len": self.max_seq_len,
                "sub_jobs": sub}
