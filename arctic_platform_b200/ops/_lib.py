"""ctypes access to the two native libraries.

``cuda_lib()`` returns ``libapb200.so`` (kernels), ``rt_lib()`` returns
``libapb200_rt.so`` (host runtime).  Both are built in-tree by
:mod:`arctic_platform_b200._build`; if the shared object is missing and a
compiler is present it is built on first use.  On a machine with a GPU a
missing kernel library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path
from typing import Tuple

import torch

from .. import _build

_lock = threading.Lock()
_cuda = None
_rt = None


class NativeLibraryError(RuntimeError):
    pass


class KernelError(RuntimeError):
    """A kernel launch returned a non-zero code or the status word is set."""


class CollectiveTimeout(KernelError):
    """A bounded device-side wait ran out: a pipeline stage that never filled (codes 101-104) or a peer that never
    announced the expected epoch (105; ``peer``, ``expected_epoch`` and ``seen_epoch`` are then set)."""

    def __init__(self, message: str, code: int, expected_epoch: int = 0, peer: int = -1, seen_epoch: int = 0):
        super().__init__(message)
        self.code, self.expected_epoch, self.peer, self.seen_epoch = code, expected_epoch, peer, seen_epoch


TIMEOUT_CODES = {101: "a TMA stage never filled", 102: "a stage never drained", 103: "an accumulator never arrived",
                 104: "TMEM was never released", 105: "a flag never reached the expected epoch"}


def _load(path: Path, builder):
    if not path.exists():
        try:
            builder()
        except Exception as exc:  # pragma: no cover - depends on toolchain
            raise NativeLibraryError(f"{path.name} is missing and could not be built: {exc}") from exc
    try:
        return ctypes.CDLL(str(path))
    except OSError as exc:
        raise NativeLibraryError(f"cannot load {path}: {exc}") from exc


def cuda_lib() -> ctypes.CDLL:
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                lib = _load(_build.CUDA_LIB, _build.build_cuda)
                _declare_cuda(lib)
                _cuda = lib
    return _cuda


def rt_lib() -> ctypes.CDLL:
    global _rt
    if _rt is None:
        with _lock:
            if _rt is None:
                lib = _load(_build.RT_LIB, _build.build_runtime)
                _declare_rt(lib)
                _rt = lib
    return _rt


def cuda_available() -> bool:
    return torch.cuda.is_available()


def stream_ptr(stream=None) -> ctypes.c_void_p:
    """Raw handle of the launch stream.  Also binds the library's runtime to torch's current device
    in this thread (autograd worker threads start without one)."""
    s = stream if stream is not None else torch.cuda.current_stream()
    code = cuda_lib().apb_bind_device(s.device.index if s.device.index is not None else torch.cuda.current_device())
    if code != 0:
        raise KernelError(f"apb_bind_device failed with code {code}")
    return ctypes.c_void_p(s.cuda_stream)


def ptr(t) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError(f"a kernel argument lives on {t.device}, not on a CUDA device")
    return ctypes.c_void_p(t.data_ptr())


_LAUNCHES = 0


def check(code: int, what: str) -> None:
    """Raises on a non-zero launch code; also counts the call as one launch of this library's kernels."""
    global _LAUNCHES
    if code != 0:
        raise KernelError(f"{what} failed with code {code}")
    _LAUNCHES += 1


def launch_count() -> int:
    """Kernel entry points of this library called so far in this process (graph replays add the number
    recorded while the graph was captured)."""
    return _LAUNCHES


def add_launches(n: int) -> None:
    global _LAUNCHES
    _LAUNCHES += int(n)


def status_read() -> int:
    return int(cuda_lib().apb_status_read())


def status_clear() -> None:
    cuda_lib().apb_status_clear()


def status_record() -> Tuple[int, int, int, int]:
    """``(code, expected epoch, peer, epoch seen)`` of the current device."""
    fn = cuda_lib().apb_status_read4
    fn.argtypes, fn.restype = [ctypes.c_void_p], ctypes.c_int
    buf = (ctypes.c_int * 4)()
    if fn(ctypes.cast(buf, ctypes.c_void_p)) != 0:
        return (int(status_read()), 0, 0, 0)
    return tuple(int(x) for x in buf)            # type: ignore[return-value]


def check_status(what: str = "kernel") -> None:
    """Synchronises and raises if any kernel recorded an error: :class:`CollectiveTimeout` when a bounded wait ran
    out, :class:`KernelError` for everything else (bad arguments, routing entries outside the group)."""
    torch.cuda.synchronize()
    st = status_read()
    if st != 0:
        code, expected, peer, seen = status_record()
        status_clear()
        if st in TIMEOUT_CODES:
            detail = f" (peer {peer} holds epoch {seen}, expected {expected})" if st == 105 and expected else ""
            raise CollectiveTimeout(f"{what}: device status word = {st}: {TIMEOUT_CODES[st]}{detail}", st, expected,
                                    peer if expected else -1, seen)
        raise KernelError(f"{what}: device status word = {st}")


c_vp = ctypes.c_void_p
c_i = ctypes.c_int
c_ll = ctypes.c_longlong
c_f = ctypes.c_float
c_sz = ctypes.c_size_t


def _sig(lib, name, argtypes, restype=ctypes.c_int):
    fn = getattr(lib, name, None)
    if fn is None:
        return
    fn.argtypes = argtypes
    fn.restype = restype


def _declare_cuda(lib) -> None:
    _sig(lib, "apb_status_read", [])
    _sig(lib, "apb_status_clear", [])
    _sig(lib, "apb_version", [])
    _sig(lib, "apb_bind_device", [c_i])
    _sig(lib, "apb_fill_u32", [c_vp, c_sz, ctypes.c_uint32, c_vp])
    _sig(lib, "apb_gemm_bf16",
         [c_vp, c_vp, c_vp, c_i, c_i, c_i, c_ll, c_ll, c_ll, c_i, c_i, c_i, c_i, c_f, c_vp,
          c_vp, c_ll, c_vp, c_i, c_ll, c_i, c_i, c_vp])
    _sig(lib, "apb_rmsnorm_fwd", [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i, c_i, c_f, c_f, c_vp])
    _sig(lib, "apb_rmsnorm_bwd", [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i, c_i, c_f, c_vp])
    _sig(lib, "apb_qknorm_rope_fwd",
         [c_vp, c_ll, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i, c_i, c_i, c_i, c_i, c_f, c_vp])
    _sig(lib, "apb_qknorm_rope_bwd",
         [c_vp, c_ll, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_ll, c_vp, c_vp,
          c_i, c_i, c_i, c_i, c_i, c_f, c_vp])
    _sig(lib, "apb_swiglu_fwd", [c_vp, c_vp, c_ll, c_ll, c_vp])
    _sig(lib, "apb_swiglu_bwd", [c_vp, c_vp, c_vp, c_ll, c_ll, c_vp])
    # later kernels declare themselves from their wrapper modules through declare()


def declare(name: str, argtypes, restype=ctypes.c_int):
    """Declares the signature of an exported kernel entry point and returns it."""
    lib = cuda_lib()
    fn = getattr(lib, name, None)
    if fn is None:
        raise NativeLibraryError(f"{name} is not exported by {_build.CUDA_LIB.name}; rebuild the library")
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


def _declare_rt(lib) -> None:
    i32p = ctypes.POINTER(ctypes.c_int32)
    i64p = ctypes.POINTER(ctypes.c_int64)
    f64p = ctypes.POINTER(ctypes.c_double)
    _sig(lib, "apb_rt_pages_create", [ctypes.c_int32], c_vp)
    _sig(lib, "apb_rt_pages_destroy", [c_vp], None)
    _sig(lib, "apb_rt_pages_free_count", [c_vp], ctypes.c_int32)
    _sig(lib, "apb_rt_pages_alloc", [c_vp, ctypes.c_int32, i32p], ctypes.c_int32)
    _sig(lib, "apb_rt_pages_retain", [c_vp, ctypes.c_int32, i32p], ctypes.c_int32)
    _sig(lib, "apb_rt_pages_release", [c_vp, ctypes.c_int32, i32p], ctypes.c_int32)
    _sig(lib, "apb_rt_pages_refcount", [c_vp, ctypes.c_int32], ctypes.c_int32)
    _sig(lib, "apb_rt_ffd_pack", [i64p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, i32p],
         ctypes.c_int32)
    _sig(lib, "apb_rt_group_prompts", [i64p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, i32p],
         ctypes.c_int32)
    _sig(lib, "apb_rt_balance_groups", [f64p, i32p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, i32p],
         ctypes.c_int32)
    f = ctypes.c_float
    _sig(lib, "apb_rt_cpu_adamw", [c_vp, c_vp, c_vp, c_vp, c_vp, ctypes.c_int64, f, f, f, f, f, f, f, f, ctypes.c_int32],
         ctypes.c_int32)
    _sig(lib, "apb_rt_cpu_sumsq", [c_vp, ctypes.c_int64], ctypes.c_double)
    _sig(lib, "apb_rt_version", [], ctypes.c_int32)
