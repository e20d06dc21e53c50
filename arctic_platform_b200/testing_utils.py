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


def apply_print_resets(buf: str) -> str:
    """What a terminal would show: on every line, whatever precedes the last carriage return is dropped (progress
    bars rewrite their line)."""
    import re
    return re.sub(r"^.*\r", "", buf, flags=re.M)


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


def gpu_partitioning_active() -> bool:
    """True when the test session gave every parallel test worker its own disjoint slice of the GPUs
    (``ARL_GPU_PARTITIONED=1``); the host-wide serial lock is then unnecessary."""
    return os.environ.get("ARL_GPU_PARTITIONED") == "1"


@contextlib.contextmanager
def gpu_serial_lock(name: str = "apb-gpu-serial") -> Iterator[None]:
    """Cross-process exclusive lock (flock) for tests that must not share the GPU with one another; a no-op when
    the workers' GPUs are partitioned."""
    if gpu_partitioning_active():
        yield
        return
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


def make_tied_lm_head_model(hidden_size: int, vocab_size: int, device: str = "cpu", dtype=torch.float32, seed: int = 0):
    """The smallest object the log-prob primitives accept as a model: ``.output_weight [vocab, hidden]`` (also
    reachable as ``.lm_head.weight`` and, tied, ``.embed``) and ``.config.vocab_size``."""
    from types import SimpleNamespace
    g = torch.Generator().manual_seed(seed)
    w = torch.nn.Parameter((torch.randn(vocab_size, hidden_size, generator=g) * hidden_size ** -0.5).to(device, dtype))
    return SimpleNamespace(output_weight=w, embed=w, lm_head=SimpleNamespace(weight=w),
                           config=SimpleNamespace(vocab_size=vocab_size, hidden_size=hidden_size))


class RunOutput:
    def __init__(self, returncode: int, stdout, stderr):
        self.returncode, self.stdout, self.stderr = returncode, stdout, stderr


async def _stream_subprocess(cmd, env, stdin, timeout, quiet, echo) -> RunOutput:
    import asyncio
    if echo:
        print("\nRunning:", " ".join(cmd))
    proc = await asyncio.create_subprocess_exec(cmd[0], *cmd[1:], stdin=stdin, stdout=asyncio.subprocess.PIPE,
                                                stderr=asyncio.subprocess.PIPE, env=env)
    out, err = [], []

    async def pump(stream, sink, label, target):
        while True:
            line = await stream.readline()
            if not line:
                return
            text = line.decode("utf-8", "replace").rstrip()
            sink.append(text)
            if not quiet:
                print(label, text, file=target)

    pumps = asyncio.gather(pump(proc.stdout, out, "stdout:", sys.stdout), pump(proc.stderr, err, "stderr:", sys.stderr))
    try:
        await asyncio.wait_for(asyncio.gather(pumps, proc.wait()), timeout=timeout)
    except asyncio.TimeoutError:
        proc.kill()                      # the exact child started above
        await proc.wait()
        raise RuntimeError(f"'{' '.join(cmd)}' did not finish within {timeout}s") from None
    return RunOutput(proc.returncode, out, err)


def execute_subprocess_async(cmd, env=None, stdin=None, timeout: float = 180, quiet: bool = False, echo: bool = True
                             ) -> RunOutput:
    """Runs ``cmd`` (a list), streaming its output line by line while capturing it.  Raises when the command fails,
    runs past ``timeout`` or prints nothing at all (a test that delegates its checks to the child must have seen
    the child say something)."""
    import asyncio
    loop = asyncio.new_event_loop()          # never the ambient loop: an earlier async test may have closed it
    try:
        result = loop.run_until_complete(_stream_subprocess(list(cmd), env, stdin, timeout, quiet, echo))
    finally:
        loop.close()
    if result.returncode != 0:
        raise RuntimeError(f"'{' '.join(cmd)}' failed with returncode {result.returncode}\n\n"
                           "stderr of the child:\n" + "\n".join(result.stderr))
    if not result.stdout and not result.stderr:
        raise RuntimeError(f"'{' '.join(cmd)}' produced no output.")
    return result


# ------------------------------------------------------------------------------------------------- environment flags
def parse_flag_from_env(key: str, default: bool = False) -> bool:
    """``yes/true/1/on`` and ``no/false/0/off`` (any case); anything else is an error, not a silent default."""
    raw = os.environ.get(key)
    if raw is None:
        return default
    word = raw.strip().lower()
    if word in ("1", "true", "yes", "y", "on"):
        return True
    if word in ("0", "false", "no", "n", "off", ""):
        return False
    raise ValueError(f"{key}={raw!r}: expected yes or no")


def parse_int_from_env(key: str, default: Optional[int] = None) -> Optional[int]:
    raw = os.environ.get(key)
    if raw is None:
        return default
    try:
        return int(raw)
    except ValueError as exc:
        raise ValueError(f"{key}={raw!r}: expected an integer") from exc


def is_torch_available() -> bool:
    return True


def is_deepspeed_available() -> bool:
    return importlib.util.find_spec("deepspeed") is not None


def get_gpu_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


# ------------------------------------------------------------------------------------------------- more decorators
def require_torch(fn):
    return fn


def require_torch_no_gpus(fn):
    return _skip_unless(get_gpu_count() == 0, "test requires a machine without GPUs")(fn)


def require_torch_non_multi_gpu(fn):
    return _skip_unless(get_gpu_count() < 2, "test requires zero or one GPU")(fn)


def require_torch_up_to_2_gpus(fn):
    return _skip_unless(get_gpu_count() < 3, "test requires at most two GPUs")(fn)


require_deepspeed = require_module("deepspeed")
require_flash_attn = require_module("flash_attn")
require_flash_attn_3 = require_module("flash_attn_interface")


# ------------------------------------------------------------------------------------------------- paths and files
def get_tests_dir(append_path: Optional[str] = None) -> str:
    """The ``tests`` directory of the checkout this module was imported from (``append_path`` joined onto it)."""
    root = Path(__file__).resolve().parents[1] / "tests"
    return str(root / append_path) if append_path else str(root)


@contextlib.contextmanager
def ExtendSysPath(path) -> Iterator[None]:
    """``sys.path`` with ``path`` in front for the duration of the block."""
    path = os.fspath(path)
    sys.path.insert(0, path)
    try:
        yield
    finally:
        try:
            sys.path.remove(path)
        except ValueError:
            pass


def write_file(file, content: str) -> None:
    Path(file).parent.mkdir(parents=True, exist_ok=True)
    Path(file).write_text(content, encoding="utf-8")


def read_json_file(file):
    import json
    return json.loads(Path(file).read_text(encoding="utf-8"))


def replace_str_in_file(file, text_to_search: str, replacement_text: str) -> int:
    """Replaces every occurrence in place; returns how many there were."""
    p = Path(file)
    text = p.read_text(encoding="utf-8")
    n = text.count(text_to_search)
    if n:
        p.write_text(text.replace(text_to_search, replacement_text), encoding="utf-8")
    return n


class CaptureLogger:
    """Collects what a ``logging`` logger emits inside the block: ``with CaptureLogger(log) as cl: ...; cl.out``."""

    def __init__(self, logger):
        import logging
        self.logger = logger
        self.io = io.StringIO()
        self.handler = logging.StreamHandler(self.io)
        self.out = ""

    def __enter__(self):
        self.logger.addHandler(self.handler)
        return self

    def __exit__(self, *exc):
        self.logger.removeHandler(self.handler)
        self.out = self.io.getvalue()

    def __repr__(self):
        return f"captured: {self.out}\n"


# ------------------------------------------------------------------------------------------------- pytest-xdist
def get_xdist_worker_id() -> int:
    """0 outside pytest-xdist, else the numeric part of ``gw<N>``."""
    worker = os.environ.get("PYTEST_XDIST_WORKER", "gw0")
    digits = "".join(c for c in worker if c.isdigit())
    return int(digits) if digits else 0


def get_xdist_worker_count() -> int:
    return parse_int_from_env("PYTEST_XDIST_WORKER_COUNT", 1) or 1


# ------------------------------------------------------------------------------------------------- pytest reports
def pytest_addoption_shared(parser) -> None:
    """``--make-reports=<id>``: write the terminal report's sections to ``reports/<id>/*.txt`` (call from a
    ``conftest.py``'s ``pytest_addoption``)."""
    try:
        parser.addoption("--make-reports", action="store", default=False,
                         help="write report files under reports/<id>/ (durations, failures, summary)")
    except ValueError:
        pass                                    # already added by another conftest


def pytest_terminal_summary_main(tr, id: str, root: Optional[str] = None) -> Dict[str, str]:
    """Writes ``durations.txt`` (slowest first), ``failures_line.txt`` (one line per failure), ``failures_long.txt``
    (tracebacks), ``passes.txt``, ``skipped.txt`` and ``stats.txt`` for a finished run.  ``tr`` is pytest's terminal
    reporter.  Returns ``{name: path}``."""
    out_dir = Path(root or "reports") / str(id)
    out_dir.mkdir(parents=True, exist_ok=True)
    stats = getattr(tr, "stats", {})
    files: Dict[str, str] = {}

    def emit(name: str, lines) -> None:
        path = out_dir / f"{name}.txt"
        path.write_text("".join(f"{ln}\n" for ln in lines), encoding="utf-8")
        files[name] = str(path)

    timed = [r for reps in stats.values() for r in reps if hasattr(r, "duration") and getattr(r, "when", "") == "call"]
    timed.sort(key=lambda r: r.duration, reverse=True)
    emit("durations", [f"{r.duration:9.3f}s {r.nodeid}" for r in timed if r.duration >= 0.005])
    failed = list(stats.get("failed", [])) + list(stats.get("error", []))
    emit("failures_line", [f"{r.nodeid}: {str(getattr(r, 'longreprtext', '')).strip().splitlines()[-1] if getattr(r, 'longreprtext', '') else ''}"
                           for r in failed])
    emit("failures_long", [f"==== {r.nodeid}\n{getattr(r, 'longreprtext', '')}" for r in failed])
    emit("passes", [r.nodeid for r in stats.get("passed", []) if getattr(r, "when", "call") == "call"])
    emit("skipped", [f"{r.nodeid}: {r.longrepr[-1] if isinstance(r.longrepr, tuple) else r.longrepr}" for r in stats.get("skipped", [])])
    emit("stats", [f"{k or 'other'}: {len(v)}" for k, v in sorted(stats.items(), key=lambda kv: str(kv[0]))])
    return files


# ------------------------------------------------------------------------------------------------- GPUs under pytest-xdist
def gpu_slice_for_worker(worker_id: int, n_workers: int, gpu_ids):
    """The GPUs one pytest-xdist worker may see: the list is cut into ``n_workers`` contiguous slices of equal size
    (the remainder stays unused so that every worker has the same number of devices); with more workers than GPUs,
    workers share round-robin, one GPU each."""
    ids = [str(g) for g in gpu_ids]
    if not ids or n_workers <= 1:
        return ids
    if n_workers >= len(ids):
        return [ids[worker_id % len(ids)]]
    per = len(ids) // n_workers
    return ids[worker_id * per:(worker_id + 1) * per]


def visible_gpu_ids():
    """GPU ids this process could use, WITHOUT initialising CUDA: ``CUDA_VISIBLE_DEVICES`` when set, else the device
    nodes the driver created."""
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible is not None:
        return [v.strip() for v in visible.split(",") if v.strip()]
    import glob
    import re
    return sorted((re.sub(r"\\D", "", p) for p in glob.glob("/dev/nvidia[0-9]*")), key=int)


def partition_gpus_for_xdist() -> Optional[str]:
    """Call before anything initialises CUDA (top of ``conftest.py``): under pytest-xdist, narrows
    ``CUDA_VISIBLE_DEVICES`` to this worker's slice and sets ``ARL_GPU_PARTITIONED=1``; returns the new value, or
    None when nothing was changed (no xdist, no GPUs, or already partitioned)."""
    if "PYTEST_XDIST_WORKER" not in os.environ or os.environ.get("ARL_GPU_PARTITIONED"):
        return None
    ids = visible_gpu_ids()
    if not ids:
        return None
    mine = gpu_slice_for_worker(get_xdist_worker_id(), get_xdist_worker_count(), ids)
    os.environ["CUDA_VISIBLE_DEVICES"] = ",".join(mine)
    os.environ["ARL_GPU_PARTITIONED"] = "1"
    return os.environ["CUDA_VISIBLE_DEVICES"]
