"""Helpers for tests and examples: capability decorators, seeding, tensor comparison, environment mocking,
port reservation and a cross-process GPU lock (subset of arctic_platform/testing_utils.py:102-1255 that the
platform's own tests rely on)."""
from __future__ import annotations

import contextlib
import fcntl
import functools
import importlib.util
import io
import os
import random
import socket
import sys
import tempfile
import unittest
from pathlib import Path
from typing import Dict, Iterator, Optional

import torch


def _skip_unless(cond: bool, reason: str):
    def deco(fn):
        return unittest.skipUnless(cond, reason)(fn)
    return deco


def require_torch_gpu(fn):
    return _skip_unless(torch.cuda.is_available(), "test requires a CUDA device")(fn)


def require_torch_multi_gpu(fn):
    return _skip_unless(torch.cuda.is_available() and torch.cuda.device_count() > 1, "test requires several GPUs")(fn)


def require_module(name: str):
    return _skip_unless(importlib.util.find_spec(name) is not None, f"test requires {name}")


require_ray = require_module("ray")
require_fastapi = require_module("fastapi")


def set_seed(seed: int = 42) -> None:
    random.seed(seed)
    try:
        import numpy as np
        np.random.seed(seed)
    except Exception:
        pass
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def torch_assert_equal(actual, expected, **kw) -> None:
    torch.testing.assert_close(actual, expected, rtol=0.0, atol=0.0, **kw)


def torch_assert_close(actual, expected, **kw) -> None:
    torch.testing.assert_close(actual, expected, **kw)


def torch_assert_safetensors_close(path_a, path_b, rtol: float = 1e-5, atol: float = 1e-6) -> None:
    from .models.hf_io import read_safetensors
    a, b = dict(read_safetensors(path_a)), dict(read_safetensors(path_b))
    assert a.keys() == b.keys(), f"tensor names differ: {sorted(set(a) ^ set(b))[:5]}"
    for k in a:
        torch.testing.assert_close(a[k].float(), b[k].float(), rtol=rtol, atol=atol, msg=lambda m: f"{k}: {m}")


class CaptureStd:
    """Context manager capturing stdout and/or stderr into ``.out`` / ``.err``."""

    def __init__(self, out: bool = True, err: bool = True):
        self._want_out, self._want_err = out, err
        self.out = self.err = ""

    def __enter__(self):
        if self._want_out:
            self._old_out, sys.stdout = sys.stdout, io.StringIO()
        if self._want_err:
            self._old_err, sys.stderr = sys.stderr, io.StringIO()
        return self

    def __exit__(self, *exc):
        if self._want_out:
            self.out, sys.stdout = sys.stdout.getvalue(), self._old_out
        if self._want_err:
            self.err, sys.stderr = sys.stderr.getvalue(), self._old_err
        return False


class CaptureStdout(CaptureStd):
    def __init__(self):
        super().__init__(err=False)


class CaptureStderr(CaptureStd):
    def __init__(self):
        super().__init__(out=False)


@contextlib.contextmanager
def mockenv_context(*remove: str, **update: str) -> Iterator[None]:
    """Temporarily sets / removes environment variables."""
    saved: Dict[str, Optional[str]] = {k: os.environ.get(k) for k in list(remove) + list(update)}
    try:
        for k in remove:
            os.environ.pop(k, None)
        os.environ.update(update)
        yield
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def mockenv(**update: str):
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **kw):
            with mockenv_context(**update):
                return fn(*a, **kw)
        return wrapper
    return deco


def get_unique_port_number(base: int = 10999, stride: int = 8) -> int:
    """Distinct base port per pytest-xdist worker (``gw3`` -> base + 3 * stride)."""
    wid = os.environ.get("PYTEST_XDIST_WORKER", "gw0")
    try:
        n = int(wid.replace("gw", ""))
    except ValueError:
        n = 0
    return base + stride * n


def reserve_free_port(host: str = "127.0.0.1") -> int:
    with socket.socket() as s:
        s.bind((host, 0))
        return s.getsockname()[1]


@contextlib.contextmanager
def gpu_serial_lock(name: str = "apb-gpu-serial") -> Iterator[None]:
    """Cross-process exclusive lock (flock) for tests that must not share the GPU with one another."""
    path = Path(tempfile.gettempdir()) / f"{name}.lock"
    with open(path, "w") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


class TestCasePlus(unittest.TestCase):
    """``unittest.TestCase`` with self-cleaning temporary directories."""

    def setUp(self):
        super().setUp()
        self._tmp = []

    def get_auto_remove_tmp_dir(self) -> str:
        d = tempfile.TemporaryDirectory()
        self._tmp.append(d)
        return d.name

    def tearDown(self):
        for d in self._tmp:
            d.cleanup()
        super().tearDown()
