"""Prompt de-duplicated training ("ZoRRo"): layout tables, tensor-level views, the actor, sequence-length balancing.

``ZoRRoTrain`` / ``ReconstructionInfo`` (the reference's class-style entry points, ``api.py``), ``PackedBatch`` and
``DeduplicatedActor`` are importable from the package; each is loaded on first use."""
from __future__ import annotations

import importlib

_WHERE = {"ZoRRoTrain": "api", "ReconstructionInfo": "api", "PackedBatch": "layout", "build_packed_batch": "layout",
          "DeduplicatedActor": "actor"}

__all__ = sorted(_WHERE)


def __getattr__(name: str):
    if name not in _WHERE:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(f"{__name__}.{_WHERE[name]}"), name)
    globals()[name] = value
    return value
