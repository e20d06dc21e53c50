"""Checkpoint directory conventions: ``<root>/checkpoint-<step>`` tags and pruning of old ones
(arctic_platform/common/utils/checkpoint.py:27-62 in the reference)."""
from __future__ import annotations

import re
import shutil
from pathlib import Path
from typing import Optional, Tuple

_TAG = re.compile(r"^checkpoint-(\d+)$")


def resolve_checkpoint_save_paths(root: str, step: Optional[int]) -> Tuple[str, Optional[str]]:
    """``(save_dir, tag)``: with a step the engine writes under ``root`` with tag ``checkpoint-<step>``;
    without one it uses its own default tag (``global_step<N>``)."""
    return (str(root), f"checkpoint-{int(step)}") if step is not None else (str(root), None)


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
