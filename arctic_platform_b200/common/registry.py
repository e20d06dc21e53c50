"""Name -> callable registries for loss functions and output post-processors.

A request's ``processing`` dict (``{"pre": [...], "post": [...], "loss_fn": name, "loss_kwargs": {...}}``)
selects functions by name; an unknown name with dots in it is imported as ``package.module.attr``
(same contract as arctic_platform/common/registry.py:24-59).
"""
from __future__ import annotations

import importlib
from typing import Callable, Dict

LOSS_FNS: Dict[str, Callable] = {}
POST_PROCESSORS: Dict[str, Callable] = {}


def _register(table: Dict[str, Callable], name: str):
    def deco(fn: Callable) -> Callable:
        table[name] = fn
        return fn
    return deco


def register_loss_fn(name: str):
    return _register(LOSS_FNS, name)


def register_post_processor(name: str):
    return _register(POST_PROCESSORS, name)


def resolve_fn(name_or_fn, table: Dict[str, Callable]) -> Callable:
    if callable(name_or_fn):
        return name_or_fn
    if name_or_fn in table:
        return table[name_or_fn]
    if isinstance(name_or_fn, str) and "." in name_or_fn:
        mod, _, attr = name_or_fn.rpartition(".")
        try:
            return getattr(importlib.import_module(mod), attr)
        except (ImportError, AttributeError) as exc:
            raise KeyError(f"cannot import {name_or_fn!r}: {exc}") from exc
    raise KeyError(f"{name_or_fn!r} is not registered (known: {sorted(table)})")
