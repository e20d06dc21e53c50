"""Device buffers on the driver's virtual-memory management API: shareable between the processes of a node as file
descriptors, and with addresses that survive giving the physical memory back.

* ``VmmBuffer(device, nbytes)`` -- an address range backed by physical memory on ``device`` (``csrc/vmm.cu``).
  ``export_fd()`` returns a file descriptor of the physical allocation; ``release_physical()`` / ``remap()`` are the
  sleep / wake pair with a stable address; ``tensor(dtype, numel)`` views the range as a torch tensor (no copy).
* ``ImportedBuffer(device, fd, padded)`` -- another process's allocation mapped here; loads and stores go over NVLink.
* ``exchange_fds(rank, world, fd, sock_dir, barrier)`` -- every rank's descriptor to every other rank over Unix
  sockets (``SCM_RIGHTS``); only the ranks of one node can take part, which is also the reach of peer mappings.
* ``VmmSymmetricMemory(numel, dtype, device, group)`` -- the same-sized buffer on every rank with the table of
  per-rank addresses the peer-load / peer-store kernels take: the allocation behind ``SymmetricBuffer`` when
  ``APB_SYMM=vmm`` is set (default: ``torch.distributed._symmetric_memory``).

Status: the descriptor exchange and all argument handling are tested on CPU (``tests/test_vmm_cpu.py``); the driver
calls are compiled for sm_100a but have NOT been run on a GPU, which is why this backend is opt-in.  No NVSwitch
multicast object is created here (``multimem`` kernels keep needing the default backend).
"""
from __future__ import annotations

import ctypes
import os
import socket
import threading
import time
from typing import Callable, Dict, List, Optional

import torch

NO_DRIVER = -10          # csrc/vmm.cu: no usable CUDA driver
_FN: Dict[str, object] = {}


class VmmError(RuntimeError):
    def __init__(self, what: str, code: int):
        super().__init__(f"{what} failed with code {code}" + (" (no CUDA driver on this machine)" if code == NO_DRIVER else ""))
        self.code = code


def _fn(name: str):
    if not _FN:
        from ..ops import _lib
        c = ctypes
        vp, i, sz, u64 = c.c_void_p, c.c_int, c.c_size_t, c.c_ulonglong
        P = c.POINTER
        _FN["granularity"] = _lib.declare("apb_vmm_granularity", [i, P(sz)])
        _FN["alloc"] = _lib.declare("apb_vmm_alloc", [i, sz, P(vp), P(sz), P(u64)])
        _FN["export_fd"] = _lib.declare("apb_vmm_export_fd", [u64, P(i)])
        _FN["import_fd"] = _lib.declare("apb_vmm_import_fd", [i, i, sz, P(vp), P(u64)])
        _FN["release_physical"] = _lib.declare("apb_vmm_release_physical", [vp, sz, u64])
        _FN["remap"] = _lib.declare("apb_vmm_remap", [i, vp, sz, P(u64)])
        _FN["free"] = _lib.declare("apb_vmm_free", [vp, sz, u64])
    return _FN[name]


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise VmmError(what, rc)


def granularity(device: int) -> int:
    out = ctypes.c_size_t(0)
    _check(_fn("granularity")(int(device), ctypes.byref(out)), "apb_vmm_granularity")
    return int(out.value)


class _DeviceRange:
    """``__cuda_array_interface__`` over a raw device range, so that ``torch.as_tensor`` can view it."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}


_TYPESTR = {torch.float32: "<f4", torch.float16: "<f2", torch.int32: "<i4", torch.int64: "<i8", torch.uint8: "|u1",
            torch.int8: "|i1", torch.int16: "<i2", torch.float64: "<f8"}


def view_as_tensor(ptr: int, nbytes: int, dtype: torch.dtype, numel: int, device: int) -> torch.Tensor:
    """A tensor over ``[ptr, ptr + numel * itemsize)``; bf16 goes through int16 (the array interface has no bf16)."""
    item = torch.empty((), dtype=dtype).element_size()
    if numel * item > nbytes:
        raise ValueError(f"{numel} elements of {dtype} need {numel * item} bytes, the range holds {nbytes}")
    carrier = torch.int16 if dtype == torch.bfloat16 else dtype
    if carrier not in _TYPESTR:
        raise TypeError(f"no array-interface type for {dtype}")
    t = torch.as_tensor(_DeviceRange(ptr, (numel,), _TYPESTR[carrier]), device=torch.device("cuda", device))
    return t.view(dtype) if carrier is not dtype else t


class VmmBuffer:
    def __init__(self, device: int, nbytes: int):
        if nbytes <= 0:
            raise ValueError("nbytes must be positive")
        self.device = int(device)
        va, padded, handle = ctypes.c_void_p(0), ctypes.c_size_t(0), ctypes.c_ulonglong(0)
        _check(_fn("alloc")(self.device, int(nbytes), ctypes.byref(va), ctypes.byref(padded), ctypes.byref(handle)), "apb_vmm_alloc")
        self.ptr, self.padded, self.handle = int(va.value), int(padded.value), int(handle.value)
        self.nbytes = int(nbytes)

    @property
    def resident(self) -> bool:
        return self.handle != 0

    def tensor(self, dtype: torch.dtype, numel: int) -> torch.Tensor:
        if not self.resident:
            raise RuntimeError("the buffer's physical memory is released; call remap() first")
        return view_as_tensor(self.ptr, self.padded, dtype, numel, self.device)

    def export_fd(self) -> int:
        fd = ctypes.c_int(-1)
        _check(_fn("export_fd")(self.handle, ctypes.byref(fd)), "apb_vmm_export_fd")
        return int(fd.value)

    def release_physical(self) -> None:
        """Sleep: the pages go back to the driver, the addresses stay reserved; contents are lost."""
        if self.resident:
            _check(_fn("release_physical")(ctypes.c_void_p(self.ptr), self.padded, self.handle), "apb_vmm_release_physical")
            self.handle = 0

    def remap(self) -> None:
        """Wake: fresh pages under the same addresses (contents undefined)."""
        if not self.resident:
            h = ctypes.c_ulonglong(0)
            _check(_fn("remap")(self.device, ctypes.c_void_p(self.ptr), self.padded, ctypes.byref(h)), "apb_vmm_remap")
            self.handle = int(h.value)

    def free(self) -> None:
        if self.ptr:
            _fn("free")(ctypes.c_void_p(self.ptr), self.padded, self.handle)
            self.ptr, self.handle = 0, 0


class ImportedBuffer:
    def __init__(self, device: int, fd: int, padded: int):
        va, handle = ctypes.c_void_p(0), ctypes.c_ulonglong(0)
        _check(_fn("import_fd")(int(device), int(fd), int(padded), ctypes.byref(va), ctypes.byref(handle)), "apb_vmm_import_fd")
        self.device, self.ptr, self.padded, self.handle = int(device), int(va.value), int(padded), int(handle.value)

    def free(self) -> None:
        if self.ptr:
            _fn("free")(ctypes.c_void_p(self.ptr), self.padded, self.handle)
            self.ptr, self.handle = 0, 0


# ------------------------------------------------------------------------------------------------- descriptor exchange
def _sock_path(sock_dir: str, rank: int) -> str:
    return os.path.join(sock_dir, f"rank{rank}.sock")


def exchange_fds(rank: int, world: int, fd: int, sock_dir: str, barrier: Callable[[], None], timeout: float = 60.0,
                 payload: int = 0) -> Dict[int, tuple]:
    """Sends ``fd`` (and one integer ``payload``, e.g. the padded size) to every other rank and returns
    ``{peer: (received fd, payload)}``.  Every rank listens on ``sock_dir/rank<r>.sock``; ``barrier()`` must return
    only when every rank has called it (all listeners exist before anybody connects).  Received descriptors belong to
    the caller (close them after importing)."""
    if world <= 1:
        return {}
    os.makedirs(sock_dir, exist_ok=True)
    path = _sock_path(sock_dir, rank)
    try:
        os.unlink(path)
    except FileNotFoundError:
        pass
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    server.bind(path)
    server.listen(world)
    server.settimeout(timeout)
    got: Dict[int, tuple] = {}
    errors: List[BaseException] = []

    def accept_all():
        try:
            for _ in range(world - 1):
                conn, _addr = server.accept()
                with conn:
                    conn.settimeout(timeout)
                    msg, fds, _flags, _a = socket.recv_fds(conn, 32, 1)
                    if len(fds) != 1 or len(msg) != 16:
                        raise RuntimeError(f"rank {rank}: malformed descriptor message ({len(msg)} bytes, {len(fds)} descriptors)")
                    peer = int.from_bytes(msg[:8], "little")
                    got[peer] = (fds[0], int.from_bytes(msg[8:], "little"))
                    conn.sendall(b"k")                      # the sender may close its end only after we hold the descriptor
        except BaseException as exc:                        # reported by the calling thread
            errors.append(exc)

    t = threading.Thread(target=accept_all, name=f"apb-vmm-accept-{rank}", daemon=True)
    t.start()
    try:
        barrier()
        msg = int(rank).to_bytes(8, "little") + int(payload).to_bytes(8, "little")
        for peer in range(world):
            if peer == rank:
                continue
            deadline = time.time() + timeout
            while True:
                c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
                c.settimeout(timeout)
                try:
                    c.connect(_sock_path(sock_dir, peer))
                    break
                except (FileNotFoundError, ConnectionRefusedError):
                    c.close()
                    if time.time() > deadline:
                        raise TimeoutError(f"rank {rank}: rank {peer} is not listening on {_sock_path(sock_dir, peer)}")
                    time.sleep(0.02)
            with c:
                socket.send_fds(c, [msg], [fd])
                if c.recv(1) != b"k":
                    raise RuntimeError(f"rank {rank}: rank {peer} did not confirm the descriptor")
        t.join(timeout)
        if t.is_alive():
            raise TimeoutError(f"rank {rank}: received {len(got)} of {world - 1} descriptors within {timeout}s")
        if errors:
            raise errors[0]
        return got
    finally:
        server.close()
        try:
            os.unlink(path)
        except OSError:
            pass


def default_sock_dir() -> str:
    """One directory per job on this node: named after the rendezvous port so that two jobs never share it."""
    base = os.environ.get("APB_VMM_SOCK_DIR") or os.path.join("/tmp", f"apb-vmm-{os.getuid()}")
    return os.path.join(base, os.environ.get("MASTER_PORT", "0"))


class VmmSymmetricMemory:
    """The same-sized VMM buffer on every rank of ``group`` (all on one node), each mapped into every rank."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group=None, sock_dir: Optional[str] = None):
        import torch.distributed as dist
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        dev = device.index if device.index is not None else torch.cuda.current_device()
        item = torch.empty((), dtype=dtype).element_size()
        self.local = VmmBuffer(dev, max(1, numel) * item)
        self.tensor = self.local.tensor(dtype, numel)
        fd = self.local.export_fd()
        self.imported: Dict[int, ImportedBuffer] = {}
        try:
            got = exchange_fds(self.rank, self.world, fd, sock_dir or default_sock_dir(), lambda: dist.barrier(group=group),
                               payload=self.local.padded)
        finally:
            os.close(fd)
        for peer, (pfd, padded) in sorted(got.items()):
            try:
                self.imported[peer] = ImportedBuffer(dev, pfd, padded)
            finally:
                os.close(pfd)
        self.peer_ptrs = [self.local.ptr if r == self.rank else self.imported[r].ptr for r in range(self.world)]
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)

    def close(self) -> None:
        for b in self.imported.values():
            b.free()
        self.imported.clear()
        self.tensor = None
        self.local.free()
