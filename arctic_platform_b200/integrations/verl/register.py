"""Lazy plugin registration.

verl imports the modules named in ``VERL_USE_EXTERNAL_MODULES`` at bootstrap; importing this one registers the
adapter under the backend name ``"arctic"`` -- in verl's ``RemoteBackendRegistry`` when verl is importable, and
always in the local ``BACKENDS`` table so the same lookup works in tests and in frameworks without a registry.
Nothing heavy is imported until ``resolve()`` is called.  Counterpart of
arctic_platform/integrations/verl/register.py:45-73.
"""
from __future__ import annotations

import importlib
from pathlib import Path
from typing import Callable, Dict

BACKENDS: Dict[str, Callable[[], type]] = {}
WORKERS: Dict[str, Callable[[], type]] = {}
ROLLOUTS: Dict[str, Callable[[], type]] = {}


def _lazy(module: str, attr: str) -> Callable[[], type]:
    return lambda: getattr(importlib.import_module(module, __package__), attr)


def config_search_path() -> str:
    """Directory to add to Hydra's search path (``hydra.searchpath+=[file://...]``) for ``remote_backend=arctic``."""
    return str(Path(__file__).resolve().parent / "config")


def register() -> Dict[str, bool]:
    BACKENDS["arctic"] = _lazy(".adapter", "ArcticRLClientWrapper")
    WORKERS["arctic"] = _lazy(".worker", "ArcticRLActorRolloutRefWorker")
    ROLLOUTS["arctic"] = _lazy(".rollout", "ArcticLLMServer")
    in_verl = False
    try:
        reg = importlib.import_module("verl.workers.remote_backend").RemoteBackendRegistry
        reg.register("arctic")(BACKENDS["arctic"]())
        in_verl = True
    except Exception:
        pass
    return {"local": True, "verl": in_verl}


def resolve(kind: str, name: str = "arctic") -> type:
    table = {"backend": BACKENDS, "worker": WORKERS, "rollout": ROLLOUTS}[kind]
    if name not in table:
        raise KeyError(f"no {kind} registered under '{name}' (import {__name__} first)")
    return table[name]()


STATUS = register()
