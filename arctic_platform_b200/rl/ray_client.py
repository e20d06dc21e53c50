"""Ray-protocol client.

The reference runs the server state as a 0-GPU Ray actor and one Ray actor per training GPU
(arctic_platform/common/ray_server.py:113-131, rl/ray_client.py:63-184).  Ray is an optional dependency
here: when it is importable the job server core is hosted in a Ray actor and calls go through actor
handles; when it is not, the same class falls back to hosting the core in this process, which keeps the
``comm_protocol="ray"`` code path of client scripts working on machines without Ray.
"""
from __future__ import annotations

from typing import Optional

from ..common.server import ArcticRLServerCore
from .config import ArcticRLClientConfig
from .local_client import ArcticRLLocalClient


def ray_available() -> bool:
    try:
        import ray  # noqa: F401
        return True
    except Exception:
        return False


class _RayCoreProxy:
    """Forwards attribute calls to a Ray actor hosting an ``ArcticRLServerCore``."""

    def __init__(self, actor):
        self._actor = actor

    def __getattr__(self, name):
        import ray
        method = getattr(self._actor, name)

        def call(*args, **kwargs):
            return ray.get(method.remote(*args, **kwargs))
        return call


def create_arctic_rl_ray_server_state(**kwargs):
    """Server state hosted in a detached 0-GPU actor (Ray) or in-process (no Ray)."""
    from ..common.ray_server import create_arctic_rl_ray_server_state as create
    return create(**kwargs)


class ArcticRLRayClient(ArcticRLLocalClient):
    JOB_ORDER = ("training", "sampling", "log_prob")

    def __init__(self, config: ArcticRLClientConfig, arctic_rl_server_state=None):
        state = arctic_rl_server_state or create_arctic_rl_ray_server_state(
            training_gpus=config.training_gpus, sampling_gpus=config.sampling_gpus,
            log_prob_gpus=config.log_prob_gpus, colocate=config.colocate)
        super().__init__(config, state)
