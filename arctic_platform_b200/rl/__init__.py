"""RL client package: ``ArcticRLClientConfig`` + ``create_arctic_rl_client`` (the names the reference exports
from ``arctic_platform.rl``, rl/__init__.py:37-41)."""
from .client import create_arctic_rl_client
from .config import ArcticRLClientConfig, WeightSyncConfig

__all__ = ["ArcticRLClientConfig", "WeightSyncConfig", "create_arctic_rl_client"]
