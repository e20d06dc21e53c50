"""``create_arctic_rl_client``: picks the client implementation for ``config.comm_protocol``
(arctic_platform/rl/client.py:40-47 in the reference dispatches between its HTTP and Ray clients; the
in-process client is the third option here)."""
from __future__ import annotations

from .config import ArcticRLClientConfig


def create_arctic_rl_client(config: ArcticRLClientConfig, arctic_rl_server_state=None):
    if config.comm_protocol == "local":
        from .local_client import ArcticRLLocalClient
        return ArcticRLLocalClient(config, arctic_rl_server_state)
    if config.comm_protocol == "http":
        from .http_client import ArcticRLHttpClient
        return ArcticRLHttpClient(config)
    if config.comm_protocol == "ray":
        from .ray_client import ArcticRLRayClient
        return ArcticRLRayClient(config, arctic_rl_server_state)
    raise ValueError(f"unknown comm_protocol {config.comm_protocol!r}")
