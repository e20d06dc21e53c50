"""Server side shared by the RL and SFT services: job server, HTTP / Ray front ends, registry, helpers.

``EngineWorker``, ``init_ray_cluster`` and ``primary_ip`` are importable from the package (loaded on first use), as
the reference's ``arctic_platform.common`` offers its worker class and cluster helpers (common/__init__.py:30-60)."""
from __future__ import annotations

import importlib

_WHERE = {"EngineWorker": "..engine.worker", "init_ray_cluster": ".ray_cluster", "primary_ip": ".ray_cluster"}

__all__ = sorted(_WHERE)


def __getattr__(name: str):
    if name not in _WHERE:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(_WHERE[name], __name__), name)
    globals()[name] = value
    return value
