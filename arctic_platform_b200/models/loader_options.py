"""Validated ``ds_worker_config.loader_options``.

The reference validates the options of its MoE loader with a strict schema (unknown keys are errors, literals are
checked, the fused cross-entropy cannot be combined with an fp32 or chunked LM head) and hands them to the model
builder (arctic_platform/model/loaders/qwen3_5_moe.py:36-92,
arctic_platform/model/implementations/qwen35/config_validation.py:1-12).  The same keys are accepted here.  What
each one does in this build:

===============================  ====================================================================================
``ac_config``                    activation checkpointing (``mode``, ``freq``, ``targets``) and CPU offload of the saved
                                 boundaries (``offload_config``); ``router_replay_recompute`` is always on
``tiled_mlp_token_chunk_size``   dense MLP over row tiles of that many tokens
``weight_conversion_cache_dir``  node-local cache of converted checkpoints
``debug``                        ``random_init`` (skip the weight load), ``num_layers`` (truncate the depth),
                                 ``deterministic_algorithms``
``optimization_dtype``           parameter / compute dtype on CPU; on a GPU the kernels are bf16 and ``float32`` is refused
``fp32_lm_head`` / ``fused_*``   accepted: the LM-head kernel always accumulates in fp32 and never forms the logits
``seq_len``, ``attn``, ...       accepted, no effect (one attention kernel, no sequence-length specialisation)
===============================  ====================================================================================
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional, Union


def _strict(cls, d: Optional[Dict[str, Any]], what: str):
    d = dict(d or {})
    known = {f.name for f in fields(cls)}
    extra = sorted(set(d) - known)
    if extra:
        raise ValueError(f"{what}: unknown option(s) {extra}; known: {sorted(known)}")
    return cls(**d)


def _literal(value, allowed, what: str):
    if value not in allowed:
        raise ValueError(f"{what}={value!r}: expected one of {list(allowed)}")


@dataclass
class ActivationOffloadOptions:
    enabled: bool = False
    keep_last_n: int = 1
    use_streams: bool = True
    tensor_size_threshold: Optional[int] = None


@dataclass
class ActivationCheckpointOptions:
    mode: str = "full"
    freq: int = 1
    targets: List[str] = field(default_factory=lambda: ["norm"])
    offload_config: Any = field(default_factory=ActivationOffloadOptions)
    router_replay_recompute: bool = True

    def __post_init__(self) -> None:
        _literal(self.mode, ("full", "selective"), "ac_config.mode")
        if isinstance(self.offload_config, dict):
            self.offload_config = _strict(ActivationOffloadOptions, self.offload_config, "ac_config.offload_config")
        if int(self.freq) < 1:
            raise ValueError(f"ac_config.freq={self.freq}: expected >= 1")
        if self.offload_config.enabled and self.mode != "full":
            raise ValueError("Activation-checkpoint CPU offload (ac_config.offload_config.enabled=True) requires "
                             f"ac_config.mode='full', but the active mode is '{self.mode}'")

    def to_worker_dicts(self):
        """``(gradient_checkpointing dict, activation_offload dict or None)`` in the worker's own spelling."""
        gc = {"mode": self.mode, "freq": int(self.freq), "targets": list(self.targets)}
        off = self.offload_config
        ao = None
        if off.enabled:
            ao = {"keep_last": int(off.keep_last_n), "min_bytes": int(off.tensor_size_threshold or (1 << 20))}
        return gc, ao


@dataclass
class DebugOptions:
    random_init: bool = False
    num_layers: Optional[int] = None
    gradient_sample_max_numel: int = 0
    deterministic_algorithms: bool = False


@dataclass
class LoaderOptions:
    seq_len: int = 4096
    attn: str = "flash_attention_3"
    ep_comm_backend: str = "deepep"
    optimization_dtype: str = "bfloat16"
    reduce_dtype: str = "float32"
    moe_use_grouped_mm: bool = True
    fused_cross_entropy: Union[bool, str] = "liger"
    fused_lm_head_token_chunk_size: Union[int, str] = "disabled"
    fp32_lm_head: bool = False
    tiled_mlp_token_chunk_size: Optional[int] = None
    deepep_token_chunk_size: Optional[int] = None
    weight_conversion_cache_dir: Optional[str] = None
    ac_config: Any = None
    debug: Any = None
    patches: Optional[list] = None         # names registered with ``models.factory.register_patch``, applied in this order

    def __post_init__(self) -> None:
        if self.patches is not None and not (isinstance(self.patches, (list, tuple)) and all(isinstance(p, str) for p in self.patches)):
            raise ValueError("loader_options.patches: expected a list of patch names")
        _literal(self.ep_comm_backend, ("deepep",), "loader_options.ep_comm_backend")
        _literal(self.optimization_dtype, ("bfloat16", "float32"), "loader_options.optimization_dtype")
        _literal(self.reduce_dtype, ("bfloat16", "float32"), "loader_options.reduce_dtype")
        if not isinstance(self.fused_cross_entropy, bool):
            _literal(self.fused_cross_entropy, ("liger",), "loader_options.fused_cross_entropy")
        chunk = self.fused_lm_head_token_chunk_size
        if not (isinstance(chunk, int) and not isinstance(chunk, bool)):
            _literal(chunk, ("auto", "disabled"), "loader_options.fused_lm_head_token_chunk_size")
        if self.fused_cross_entropy and (self.fp32_lm_head or (isinstance(chunk, int) and not isinstance(chunk, bool))):
            raise ValueError("cannot combine fused_cross_entropy with fp32_lm_head or an integer "
                             "fused_lm_head_token_chunk_size")
        if self.tiled_mlp_token_chunk_size is not None and int(self.tiled_mlp_token_chunk_size) < 1:
            raise ValueError(f"loader_options.tiled_mlp_token_chunk_size={self.tiled_mlp_token_chunk_size}: expected >= 1")
        if isinstance(self.ac_config, dict):
            self.ac_config = _strict(ActivationCheckpointOptions, self.ac_config, "loader_options.ac_config")
        if isinstance(self.debug, dict):
            self.debug = _strict(DebugOptions, self.debug, "loader_options.debug")

    @staticmethod
    def from_dict(d: Optional[Dict[str, Any]]) -> "LoaderOptions":
        return _strict(LoaderOptions, d, "loader_options")
