"""Checkpoint directory conventions: ``<root>/checkpoint-<step>`` tags and pruning of old ones
(arctic_platform/common/utils/checkpoint.py:27-62 in the reference)."""
from __future__ import annotations

import re
import shutil
from pathlib import Path
from typing import Optional, Tuple

_TAG = re.compile(r"^checkpoint-(\d+)$")


def resolve_checkpoint_save_paths(root: str, step: Optional[int]) -> Tuple[str, str]:
    """``(save_dir, prune_root)``.  With a step the checkpoint is a self-contained directory
    ``<root>/checkpoint-<step>`` (its own ``latest``, ``global_step<N>/`` and ``hf/`` inside); without one the
    engine writes straight into ``root``.  ``prune_root`` -- the parent of the ``checkpoint-*`` children -- is
    always ``root``."""
    root = str(root)
    return (str(Path(root) / f"checkpoint-{int(step)}"), root) if step is not None else (root, root)


def resolve_checkpoint_load_path(root: str, step: Optional[int], explicit_path: bool) -> str:
    """Directory handed to the engines' ``load_checkpoint``: ``<root>/checkpoint-<step>`` for a step; for the job's
    configured root (no explicit path) the child named by the integer in ``<root>/latest``; otherwise ``root``."""
    root = str(root)
    if step is not None:
        return str(Path(root) / f"checkpoint-{int(step)}")
    if not explicit_path:
        latest = Path(root) / "latest"
        if latest.is_file():
            try:
                return str(Path(root) / f"checkpoint-{int(latest.read_text().strip())}")
            except ValueError:
                pass                      # an engine-level ``latest`` (a tag): root itself is the checkpoint directory
    return root


def prune_checkpoint_dirs(parent: str, keep: int) -> list:
    """Deletes the oldest ``checkpoint-<step>`` directories so that at most ``keep`` remain; returns the
    removed paths.  ``keep <= 0`` keeps everything; other entries are never touched."""
    if keep is None or keep <= 0:
        return []
    p = Path(parent)
    if not p.is_dir():
        return []
    found = []
    for d in p.iterdir():
        m = _TAG.match(d.name)
        if d.is_dir() and m:
            found.append((int(m.group(1)), d))
    found.sort()
    removed = []
    for _, d in found[:-keep] if len(found) > keep else []:
        shutil.rmtree(d, ignore_errors=True)
        removed.append(str(d))
    return removed
