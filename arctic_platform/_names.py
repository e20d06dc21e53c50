"""Names the reference uses for things this build calls differently, per reference module path.

``alias path -> {reference name: (module below arctic_platform_b200, attribute)}``.  When a module is imported through
the ``arctic_platform`` alias, the names of its entry are set on it (unless it already has them), so
``from arctic_platform.common.deepspeed_worker import DeepSpeedWorker`` gives this build's worker class.  Only
objects with the same role and a compatible call shape are listed; what has no counterpart (model patchers, DeepEP
buffer management, classes whose constructor differs such as the expert-parallel wrapper,
the action-mask and activation-offload holders, the Triton reconstruction kernel) is absent on purpose, and importing it fails loudly.
"""
from __future__ import annotations

_TRANSPORT = {n: ("client.transport", n) for n in ("JobHandles", "OPS", "Request", "Transport", "unresolved_ops")}
_WORKER = {"DeepSpeedWorker": ("engine.worker", "EngineWorker")}
_PROX = {"compute_prox_logp_approximations": ("rl.processors.functional", "proximal_logp_approximations"),
         "ProxLogpMethod": ("rl.processors.functional", "ProxLogpMethod"),
         "ProxApproxMethod": ("rl.processors.functional", "ProxApproxMethod")}
_ZORRO = {n: ("rl.zorro_train.api", n) for n in ("ZoRRoTrain", "ReconstructionInfo", "reconstruct_sequence",
                                                 "analyze_normal_batch_via_attention_mask")}
_LOADER_OPTIONS = {"ActivationOffloadConfig": ("models.loader_options", "ActivationOffloadOptions"),
                   "ActivationCheckpointConfig": ("models.loader_options", "ActivationCheckpointOptions"),
                   "DebugModelConfig": ("models.loader_options", "DebugOptions"),
                   "ModelConfig": ("models.loader_options", "LoaderOptions")}

COMPAT_NAMES = {
    "client": {**_TRANSPORT, "make_transport": ("client.client", "make_transport")},
    "common": dict(_WORKER),
    "common.deepspeed_worker": dict(_WORKER),
    "rl.deepspeed_worker": dict(_WORKER),
    "common.server": {"ArcticRLServerState": ("common.server", "ArcticRLServerCore")},
    "rl.server": {"ArcticRLServerState": ("common.server", "ArcticRLServerCore")},
    "common.utils.ray_pg": {"DEFAULT_BUNDLE_RESOURCES": ("common.utils.ray_pg", "BUNDLE")},
    "rl.utils.ray_pg": {"DEFAULT_BUNDLE_RESOURCES": ("common.utils.ray_pg", "BUNDLE")},
    "rl.http_client": {"ArcticRLHTTPClient": ("rl.http_client", "ArcticRLHttpClient")},
    "rl.processors.grpo": dict(_PROX),
    "rl.zorro_train.zorro_train": dict(_ZORRO),
    "rl.zorro_train.seqlen_balancing": {"get_reverse_idx": ("common.utils.batch", "get_reverse_idx")},
    "model.implementations.qwen35.config": dict(_LOADER_OPTIONS),
    "model.loaders.qwen3_5_moe": {"Qwen3_5MoeOptions": ("models.loader_options", "LoaderOptions")},
    "model.implementations.qwen35.conversion_cache": {
        "resolve_conversion_cache_path": ("models.conversion_cache", "resolve_cache_path"),
        "conversion_cache_ready": ("models.conversion_cache", "cache_ready"),
        "conversion_cache_is_node_local": ("models.conversion_cache", "cache_is_node_local")},
    "model.implementations.qwen35.models.layers.moe": {"relu2": ("models.latent_moe", "relu2")},
}
