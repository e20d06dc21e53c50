"""Step pipeline, packing, micro-batching, statistics and loss functions of the RL / SFT training calls.

The names the reference exports from ``arctic_platform.rl.processors`` (rl/processors/__init__.py:105-170) resolve
here; each is imported from its module on first use, so importing the package stays cheap and free of cycles
(``losses`` registers its functions in ``common.registry`` when it loads).
"""
from __future__ import annotations

import importlib
from typing import Any

_EXPORTS = {
    "pipeline": ("run_pipeline", "DEFAULT_PROCESSING", "pack_for_model", "response_length_of", "action_masks_of"),
    "packing": ("pack_sequences", "unpack_sequences", "pad_packed_for_model"),
    "padding": ("padded_tensor_2d_to_unpadded_tensor_1d", "padded_tensor_2d_dict_to_unpadded_tensor_1d_dict",
                "unpadded_tensor_1d_to_padded_tensor_2d", "unpadded_tensor_1d_dict_to_padded_tensor_2d_dict",
                "padded_tensor_2d_full_to_unpadded_tensor_1d_response", "unpadded_tensor_1d_response_to_padded_tensor_2d_full",
                "unpadded_tensor_1d_response_dict_to_padded_tensor_2d_full_dict", "compute_packing_info_for_batch"),
    "microbatch": ("DEFAULT_MAX_TOKENS_PER_MB", "MicroBatchSpec", "MicroBatchList", "ffd_allocate",
                   "split_padded_tensor_dict_into_mb_list"),
    "stats_tracker": ("DistributedStatsTracker", "ReduceType", "DEFAULT_TRACKER", "denominator", "stat", "scalar", "scope",
                      "export", "export_all", "get", "record_timing", "TRACKERS"),
    "functional": ("masked_sum", "masked_mean", "masked_normalization", "agg_loss", "kl_penalty", "kl_penalty_forward",
                   "ppo_clip_token_loss", "ppo_actor_loss_fn", "sapo_loss_fn", "m2po_mask", "proximal_logp_approximations",
                   "resolve_proximal_logp", "sequence_level_ratio_and_advantages", "ProxLogpMethod", "ProxApproxMethod",
                   "PROX_LOGP_METHOD_RECOMPUTE", "PROX_LOGP_METHOD_LOGLINEAR", "PROX_LOGP_METHOD_METRICS",
                   "PROX_APPROX_METHOD_LOGLINEAR", "PROX_APPROX_METHOD_LINEAR", "PROX_APPROX_METHOD_ROLLOUT",
                   "PROX_APPROX_METHODS_ALL", "compute_prox_logp_approximations", "_resolve_proximal_logp",
                   "_compute_sequence_level_ratio_and_advantages"),
    "losses": ("verl_grpo_loss", "grpo_loss", "sft_loss", "sft_ce_loss", "SFT_LOSS_FNS"),
    "../../sft/processor": ("LOGIT_LOSS_FNS", "run_sft_pipeline"),
}
_REGISTRY = ("LOSS_FNS", "POST_PROCESSORS", "register_loss_fn", "register_post_processor", "resolve_fn")
_WHERE = {name: mod for mod, names in _EXPORTS.items() for name in names}

__all__ = sorted(list(_WHERE) + list(_REGISTRY))


def __getattr__(name: str) -> Any:
    if name in _REGISTRY:
        from ...common import registry
        if name in ("LOSS_FNS", "POST_PROCESSORS"):
            importlib.import_module(f"{__name__}.losses")          # built-in functions register on import
            importlib.import_module(f"{__name__}.pipeline")
        value = getattr(registry, name)
    elif name in _WHERE:
        where = _WHERE[name]
        mod = importlib.import_module("...sft.processor", __name__) if where.startswith("../") else \
            importlib.import_module(f"{__name__}.{where}")
        value = getattr(mod, name)
    else:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    globals()[name] = value
    return value


def __dir__():
    return sorted(set(globals()) | set(__all__))
