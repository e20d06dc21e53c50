"""Unified client package (``ArcticRLClientConfig`` / ``create_arctic_rl_client``, as exported by
``arctic_platform.client`` in the reference, client/__init__.py:1-5)."""
from .client import ArcticRLClient, SyncArcticRLClient, create_arctic_rl_client
from .config import ArcticRLClientConfig, CortexConfig, OnPremConfig, SamplingConfig, TrainingConfig

__all__ = ["ArcticRLClientConfig", "ArcticRLClient", "SyncArcticRLClient", "create_arctic_rl_client", "CortexConfig",
           "OnPremConfig", "SamplingConfig", "TrainingConfig"]
