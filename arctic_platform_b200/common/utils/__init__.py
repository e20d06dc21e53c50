"""Helpers shared by the servers and workers.  The names the reference re-exports from ``arctic_platform.common.utils``
(common/utils/__init__.py) resolve here on first use; nothing is imported when the package loads."""
from __future__ import annotations

import importlib

_EXPORTS = {
    ".server_models": ("GenerateRequest", "JobConfig", "LoadCheckpointRequest", "LogProbsRequest", "OperationRequest",
                       "ResetPrefixCacheRequest", "SaveRequest", "StepRequest", "WeightNormRequest", "WeightSyncRequest",
                       "build_model_config"),
    ".batch": ("http_split_batch", "ray_split_batch", "log_dp_shard_tokens", "merge_dict_shards", "shard_token_stats", "split_dict",
               "unpack_batch", "split_batch_for_ranks", "restore_batch_order"),
    ".metrics": ("combine_metric_microbatches", "combine_metric_shards", "finalize_fwd_bwd_metrics"),
    ".cuda_ipc": ("merge_cuda_ipc_payloads",),
    "...utils.debug": ("ProfilerContext", "SynchronizedWallClockTimerSimple"),
    "...utils.record_replay": ("record_replay_generation",),
}
_WHERE = {name: mod for mod, names in _EXPORTS.items() for name in names}

__all__ = sorted(_WHERE)


def __getattr__(name: str):
    if name not in _WHERE:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(_WHERE[name], __name__), name)
    globals()[name] = value
    return value
