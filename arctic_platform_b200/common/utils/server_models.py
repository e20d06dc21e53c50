"""Request / job models of the server API (field names and defaults of
arctic_platform/common/utils/server_models.py:30-165 in the reference)."""
from __future__ import annotations

from typing import Any, Dict, List, Literal, Optional

from pydantic import BaseModel, ConfigDict, Field, field_validator


class JobConfig(BaseModel):
    model_config = ConfigDict(extra="ignore", protected_namespaces=())
    model_name: str
    job_type: Literal["training", "sampling", "log_prob"] = "training"
    num_devices: int = 1
    ds_config: Dict[str, Any] = Field(default_factory=dict)
    training_config: Optional[Dict[str, Any]] = None
    log_prob_config: Optional[Dict[str, Any]] = None
    ds_worker_config: Optional[Dict[str, Any]] = None
    vllm_config: Optional[Dict[str, Any]] = None
    checkpoint_path: Optional[str] = None
    arctic_inference_config: Optional[Dict[str, Any]] = None
    full_determinism: bool = False
    seed: int = 42
    cuda_ipc: bool = False
    low_memory: bool = False

    @field_validator("seed", mode="before")
    @classmethod
    def _null_seed(cls, v):
        return 42 if v is None else v


class GenerateRequest(BaseModel):
    prompts: List[Any]
    sampling_params: Optional[Dict[str, Any]] = None
    routing_key: Optional[str] = None
    strict: bool = False


class LogProbsRequest(BaseModel):
    prompts: List[Any]
    completions: List[Any]
    top_k: int = 1


class StepRequest(BaseModel):
    learning_rate: Optional[float] = None


class SaveRequest(BaseModel):
    checkpoint_id: Optional[str] = None
    checkpoint_type: str = "resumable"
    path: Optional[str] = None
    step: Optional[int] = None
    export_hf: bool = False
    save_total_limit: Optional[int] = None
    stage_info: Optional[Dict[str, Any]] = None


class LoadCheckpointRequest(BaseModel):
    path: Optional[str] = None
    step: Optional[int] = None


class ResetPrefixCacheRequest(BaseModel):
    drain: bool = False
    timeout_s: float = 30.0
    retry_interval_s: float = 0.5


class WeightSyncRequest(BaseModel):
    source_sub_job_id: int
    target_sub_job_ids: List[int]
    cuda_ipc: Optional[bool] = None
    low_memory: Optional[bool] = None


class OperationRequest(BaseModel):
    operation_type: str
    sub_job_id: int
    sub_job_type: Optional[str] = None
    payload: Dict[str, Any] = Field(default_factory=dict)


class WeightNormRequest(BaseModel):
    training_job_id: Optional[int] = None
    sampling_job_id: Optional[int] = None


def parse_arctic_inference_rollout(ai_cfg: Optional[dict]) -> Dict[str, Any]:
    """``zorro_inference.enable`` -> ``use_fca`` (forest cascade attention), ``speculative_decoding.model`` ->
    ``spec_model``."""
    ai_cfg = ai_cfg or {}
    out: Dict[str, Any] = {}
    if "zorro_inference" in ai_cfg:
        out["use_fca"] = bool((ai_cfg["zorro_inference"] or {}).get("enable", False))
    spec = (ai_cfg.get("speculative_decoding") or {}).get("model")
    if spec:
        out["spec_model"] = spec
    return out


_SAMPLER_KEYS = {"max_model_len", "max_num_seqs", "kv_cache_tokens", "tensor_parallel_size", "gpu_memory_utilization",
                 "enable_sleep_mode", "eos_token_id", "dtype", "seed"}


def build_model_config(model_name: str, vllm_config: Optional[dict], ai_cfg: Optional[dict] = None) -> Dict[str, Any]:
    """Sampler configuration: known keys are kept at the top level, anything else goes to
    ``extra_engine_kwargs`` untouched."""
    cfg: Dict[str, Any] = {"model": model_name, "extra_engine_kwargs": {}}
    for k, v in (vllm_config or {}).items():
        if k in _SAMPLER_KEYS:
            cfg[k] = v
        else:
            cfg["extra_engine_kwargs"][k] = v
    cfg.update(parse_arctic_inference_rollout(ai_cfg))
    return cfg
