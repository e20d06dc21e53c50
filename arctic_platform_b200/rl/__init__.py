"""RL client package.  The names the reference exports from ``arctic_platform.rl`` (rl/__init__.py:37-68) resolve
here; everything beyond the client factory and its configs is imported on first use."""
from __future__ import annotations

import importlib
from typing import Any

from .client import create_arctic_rl_client
from .config import ArcticRLClientConfig, WeightSyncConfig

_LAZY = {
    "WeightSyncCoordinator": ("weight_sync", "WeightSyncCoordinator"),
    "run_pipeline": ("processors", "run_pipeline"),
    "register_loss_fn": ("processors", "register_loss_fn"),
    "register_post_processor": ("processors", "register_post_processor"),
    "grpo_loss": ("processors", "grpo_loss"),
    "verl_grpo_loss": ("processors", "verl_grpo_loss"),
    "pack_sequences": ("processors", "pack_sequences"),
    "unpack_sequences": ("processors", "unpack_sequences"),
    "run_sft_pipeline": ("..sft", "run_sft_pipeline"),
    "sft_loss": ("..sft", "sft_loss"),
}

__all__ = ["ArcticRLClientConfig", "WeightSyncConfig", "create_arctic_rl_client", *sorted(_LAZY)]


def __getattr__(name: str) -> Any:
    if name not in _LAZY:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    mod, attr = _LAZY[name]
    target = importlib.import_module(mod if mod.startswith("..") else f".{mod}", __name__ if not mod.startswith("..") else __name__)
    value = getattr(target, attr)
    globals()[name] = value
    return value
