"""Symmetric (peer-mapped) device buffers for the in-kernel NVLink paths.

A :class:`SymmetricBuffer` is the same-sized allocation on every rank of a process group,
mapped into every rank's address space, optionally also bound to an NVSwitch multicast
object.  Kernels receive the table of per-rank base pointers (and the multicast pointer)
and issue plain loads/stores or ``multimem`` instructions on them; ordering between ranks
uses the epoch flags of :class:`EpochFlags` with bounded waits on the device.

The allocation and handle exchange ride on ``torch.distributed._symmetric_memory`` (CUDA
VMM allocations whose handles are exchanged through the process group's store) -- that is
plumbing in the sense of one-process-per-GPU ``torch.distributed``; every byte that moves
afterwards is moved by this package's kernels.  With one rank, or on CPU (gloo), the
buffer is an ordinary tensor and the pointer table has one entry.

The reference has no counterpart: it reaches other GPUs only through NCCL collectives
inside DeepSpeed / DeepEP (arctic_platform/common/deepspeed_worker.py:155).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist


def multimem_enabled() -> bool:
    """NVSwitch multicast (``multimem.*``) is used only when explicitly enabled and NVLS is not
    switched off for NCCL; fault-handling tests run with it off (plain peer loads)."""
    if os.environ.get("NCCL_NVLS_ENABLE", "1") == "0":
        return False
    return os.environ.get("APB_MULTIMEM", "0") == "1"


def _keep_rendezvous_off_multicast() -> None:
    """Unless ``APB_MULTIMEM=1`` asks for ``multimem`` kernels, tell torch's symmetric-memory rendezvous not to bind
    the allocation to an NVSwitch multicast object at all (``TORCH_SYMM_MEM_DISABLE_MULTICAST``).  A binding that no
    kernel uses still ties every rank's memory into one multicast group, and a rank that ends while bound can raise
    NVLink faults on its peers' GPUs; with the binding off, stopping a rank leaves the others on plain peer
    mappings only."""
    if not multimem_enabled():
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


class SymmetricBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, device, group=None, zero: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and group is not False) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.numel = numel
        self.dtype = dtype
        self.multicast_ptr = 0
        self._handle = None
        dev = torch.device(device)
        if self.world > 1 and dev.type == "cuda" and os.environ.get("APB_SYMM", "torch") == "vmm" and not multimem_enabled():
            # this package's own allocation + descriptor exchange (parallel/vmm.py); opt-in
            from .vmm import VmmSymmetricMemory
            self._handle = VmmSymmetricMemory(numel, dtype, dev, group)
            self.tensor = self._handle.tensor
            if zero:
                self.tensor.zero_()
            self.peer_ptrs = [int(p) for p in self._handle.peer_ptrs]
            torch.cuda.synchronize(dev)
            dist.barrier(group=group)
        elif self.world > 1 and dev.type == "cuda":
            _keep_rendezvous_off_multicast()
            import torch.distributed._symmetric_memory as symm_mem

            self.tensor = symm_mem.empty(numel, dtype=dtype, device=dev)
            if zero:
                self.tensor.zero_()
            grp = group if group is not None else dist.group.WORLD
            self._handle = symm_mem.rendezvous(self.tensor, grp)
            self.peer_ptrs: List[int] = [int(p) for p in self._handle.buffer_ptrs]
            if multimem_enabled():
                try:
                    self.multicast_ptr = int(self._handle.multicast_ptr or 0)
                except Exception:
                    self.multicast_ptr = 0
            torch.cuda.synchronize(dev)
            dist.barrier(group=group)
        else:
            self.tensor = torch.zeros(numel, dtype=dtype, device=dev) if zero else torch.empty(numel, dtype=dtype,
                                                                                              device=dev)
            self.peer_ptrs = [self.tensor.data_ptr()]

    def ptr_table(self, byte_offset: int = 0):
        """ctypes array of per-rank base pointers (advanced by ``byte_offset``) for a kernel call."""
        arr = (ctypes.c_void_p * len(self.peer_ptrs))()
        for i, p in enumerate(self.peer_ptrs):
            arr[i] = p + byte_offset
        return arr

    def mc_ptr(self, byte_offset: int = 0) -> ctypes.c_void_p:
        return ctypes.c_void_p(self.multicast_ptr + byte_offset if self.multicast_ptr else 0)


class EpochFlags:
    """One int32 flag per peer in symmetric memory plus a host-side monotonically increasing epoch.
    Every rank advances the epoch identically (SPMD), so a flag value names one kernel of the sequence
    and a stale flag can never satisfy a later wait."""

    def __init__(self, device, group=None, slots: int = 64):
        self.buf = SymmetricBuffer(slots, torch.int32, device, group)
        self.epoch = 0

    def next(self) -> int:
        self.epoch += 1
        return self.epoch

    @property
    def world(self) -> int:
        return self.buf.world

    @property
    def rank(self) -> int:
        return self.buf.rank

    def ptr_table(self):
        return self.buf.ptr_table()
