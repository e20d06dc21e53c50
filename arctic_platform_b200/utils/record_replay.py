"""Deterministic rollout record / replay for reproducing a failing training step without the sampler.

``@record_replay_generation`` wraps an async or sync ``generate``-like function.  Controlled by
``REPLAY_GENERATION_DIR`` (where the tape lives), ``REPLAY_GENERATION_MODE`` (``record`` | ``replay`` | unset)
and ``REPLAY_START_RECORD`` (first call index to put on tape); call ``i`` is stored as ``generate-{i}.json``.
Same switches as arctic_platform/common/utils/record_replay.py:26-183, with a JSON tape instead of pickle so a
tape is never executed on load."""
from __future__ import annotations

import asyncio
import functools
import json
import os
from pathlib import Path
from typing import Any, Callable


class ReplayMiss(RuntimeError):
    pass


def _settings():
    d = os.environ.get("REPLAY_GENERATION_DIR")
    mode = os.environ.get("REPLAY_GENERATION_MODE", "").lower()
    if mode == "load":                                   # the reference's word for replay
        mode = "replay"
    if os.environ.get("REPLAY_GENERATION") == "1" and not mode:
        mode = "replay"
    start = int(os.environ.get("REPLAY_START_RECORD", "0") or 0)
    return (Path(d) if d else None), mode, start


def _jsonable(obj):
    """Tensors / arrays inside a result (recorded expert choices) are taped as nested lists."""
    if hasattr(obj, "tolist"):
        return obj.tolist()
    raise TypeError(f"{type(obj).__name__} is not JSON serialisable")


def record_replay_generation(fn: Callable) -> Callable:
    counter = {"i": 0}

    def _path(d: Path, i: int) -> Path:
        return d / f"generate-{i}.json"

    def _before(args, kwargs):
        d, mode, start = _settings()
        i = counter["i"]
        counter["i"] += 1
        if d is None or mode not in ("record", "replay"):
            return None, None, i
        if mode == "replay":
            p = _path(d, i)
            if not p.exists():
                raise ReplayMiss(f"no recorded generation for call {i} under {d}")
            return json.loads(p.read_text())["result"], None, i
        return None, (d if i >= start else None), i

    def _after(d, i, result):
        if d is not None:
            d.mkdir(parents=True, exist_ok=True)
            _path(d, i).write_text(json.dumps({"call": i, "result": result}, default=_jsonable))
        return result

    if asyncio.iscoroutinefunction(fn):
        @functools.wraps(fn)
        async def awrapper(*args, **kwargs):
            replayed, d, i = _before(args, kwargs)
            if replayed is not None:
                return replayed
            return _after(d, i, await fn(*args, **kwargs))
        awrapper._replay_counter = counter
        return awrapper

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        replayed, d, i = _before(args, kwargs)
        if replayed is not None:
            return replayed
        return _after(d, i, fn(*args, **kwargs))
    wrapper._replay_counter = counter
    return wrapper


class RecordReplay:
    """Tape of whole batch dicts (tensors included), for loops that record what they fed the trainer rather than what
    the sampler returned: ``save_record(i, batch)`` in record mode, ``load_record(i)`` in load mode, ``skip_record(i)``
    for the leading records a replay should pass over.  Switches, read when the object is made:
    ``REPLAY_GENERATION=1`` (on), ``REPLAY_GENERATION_DIR``, ``REPLAY_GENERATION_MODE`` = ``record`` (default) |
    ``load``, ``REPLAY_START_RECORD``.  Records are DSSST1 frames (``generate-<i>.dssst1``): loading one parses
    tensors and JSON, it never runs code -- the reference stores pickles
    (arctic_platform/common/utils/record_replay.py:60-105)."""

    def __init__(self):
        self.enabled = os.environ.get("REPLAY_GENERATION", "").lower() in ("1", "true", "yes", "on")
        d = os.environ.get("REPLAY_GENERATION_DIR")
        self.dir = Path(d) if d else None
        self.mode = os.environ.get("REPLAY_GENERATION_MODE", "record").lower()
        if self.mode == "replay":
            self.mode = "load"
        if self.mode not in ("record", "load"):
            raise ValueError(f"REPLAY_GENERATION_MODE={self.mode!r}: expected record or load")
        try:
            self.start_record = max(0, int(os.environ.get("REPLAY_START_RECORD", "0") or 0))
        except ValueError:
            self.start_record = 0
        if self.is_record_mode():
            self.dir.mkdir(parents=True, exist_ok=True)
        elif self.is_replay_mode() and not self.dir.exists():
            raise FileNotFoundError(f"load mode needs the directory {self.dir}")

    def is_enabled(self) -> bool:
        return self.enabled and self.dir is not None

    def is_record_mode(self) -> bool:
        return self.is_enabled() and self.mode == "record"

    def is_replay_mode(self) -> bool:
        return self.is_enabled() and self.mode == "load"

    def skip_record(self, record_index: int) -> bool:
        return self.is_replay_mode() and record_index <= self.start_record

    def _path(self, record_index: int) -> Path:
        return self.dir / f"generate-{record_index}.dssst1"

    def save_record(self, record_index: int, batch_dict: dict) -> None:
        if self.is_record_mode():
            from .. import wire
            self._path(record_index).write_bytes(wire.dumps(batch_dict))

    def load_record(self, record_index: int):
        if not self.is_replay_mode():
            return None
        p = self._path(record_index)
        if not p.exists():
            raise FileNotFoundError(f"no record {record_index} under {self.dir}")
        from .. import wire
        return wire.loads(p.read_bytes())
