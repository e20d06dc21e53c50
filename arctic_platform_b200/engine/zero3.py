"""ZeRO stage 3 for the training engine: bf16 parameters live ONLY as per-rank shards.

Layout.  Every parameter is cut into ``world`` equal flat pieces (row blocks of a weight matrix); rank ``r`` keeps
piece ``r`` of every parameter of a unit back to back in its shard buffer, which sits in symmetric memory so that
peers can read it.  The fp32 master weights and Adam moments have the same per-rank layout, so the fused optimizer
kernel updates master, moments and the bf16 shard in one pass without any all-gather.

Materialisation.  A unit (one decoder block) is rebuilt just in time by ``gather_shards_kernel``: every rank PULLS the
peers' pieces over NVLink with plain loads into a gather slot; a side stream prefetches the next unit (forward: i+1,
backward: i-1) while the current one computes, and module pre-hooks (forward and backward) wait for the slot.
Parameters of unit ``i`` are permanent views into slot ``i % n_slots``, so tensors autograd saved in the forward point
at the right bytes again once the backward hook has re-gathered the unit.  ``n_slots`` is 2 (every use re-gathers)
unless the gathered blocks may stay live (``stage3_max_live_parameters``; automatic when they take at most a tenth
of the device memory): then every block has a slot of its own and is gathered ONCE per optimizer step instead of
once per micro-batch pass -- with 16 micro-batches per step that removes 31 of 32 gathers per block.  The embedding /
lm-head and the final norm stay gathered (they are touched at both ends of every pass).

Gradients.  On GPUs with the fused kernels and ``overlap_comm`` (automatic: models whose full-size fp32 gradient
buffer would take more than a tenth of the device memory) a decoder block's gradient is reduced over the ranks right after the block's backward has been queued: its weight-gradient GEMMs accumulate into one of
three block-sized fp32 staging buffers in symmetric memory, a backward hook launches ``zero3_reduce_unit_kernel`` on a
side stream (every rank pulls ITS shard range from all ranks' staging buffers, adds it to its fp32 shard accumulator
and clears what it read), and the next block's backward runs meanwhile.  A rank therefore holds three blocks of full
gradient plus its 1/world shard accumulator instead of a full-size buffer -- what lets the 32B recipes fit.  Without
the overlap (small models, CPU / gloo, the collective baseline, activation checkpointing) gradients stay full-size
in fp32, accumulated locally over micro-batches, and are reduced piece by piece at the optimizer step -- one
reduction per step instead of one per micro-batch, which is the faster choice while the buffer fits.

CPU / gloo runs use the same bookkeeping with ``all_gather`` / ``all_reduce``, which is what the equivalence test
against stage 1 exercises.  The reference delegates all of this to DeepSpeed (``zero_optimization.stage: 3``,
arctic_platform/common/deepspeed_worker.py:208-324).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..parallel.symm import SymmetricBuffer


class Zero3State:
    def __init__(self, engine):
        self.e = engine
        W, r = engine.world, engine.rank
        dev, dt = engine.device, engine.param_dtype
        self.fused = engine.impl == "fused" and engine.on_cuda
        # ---- piece tables
        self.pieces: List[List[Tuple[str, int, int, int]]] = []     # per unit: (name, full_rel_off, piece_len, shard_rel_off)
        self.unit_shard_len: List[int] = []
        for u in engine.units:
            rows, off = [], 0
            if u.local_only:             # expert-parallel unit: already different on every rank, kept whole
                self.pieces.append([])
                self.unit_shard_len.append(0)
                continue
            for name, p in u.params:
                n = p.numel()
                if n % (8 * W):
                    raise ValueError(f"ZeRO-3: parameter {name} has {n} elements, not a multiple of 8 x world ({8 * W})")
                full_off = engine.param_slices[name][0] - u.offset
                rows.append((name, full_off, n // W, off))
                off += n // W
            self.pieces.append(rows)
            self.unit_shard_len.append(off)
        # two offset systems: ``unit_shard_off`` for the fp32 state (master, moments, reduced gradients), which also
        # holds the whole of every expert-parallel unit, and ``bf16_off`` for the bf16 shard buffer peers read
        engine.unit_shard_off = []
        self.bf16_off: List[int] = []
        acc32 = acc16 = 0
        for u, n in zip(engine.units, self.unit_shard_len):
            engine.unit_shard_off.append(acc32)
            self.bf16_off.append(acc16)
            acc32 += u.length if u.local_only else n
            acc16 += n
        engine.shard_total = acc32
        # ---- shard buffer (peers read it) filled from the model's current parameters
        self.shard_buf = SymmetricBuffer(max(acc16, 8), dt, dev, engine.group if self.fused else False)
        with torch.no_grad():
            for ui, u in enumerate(engine.units):
                base = self.bf16_off[ui]
                pmap = dict(u.params)
                for name, _fo, pl, so in self.pieces[ui]:
                    self.shard_buf.tensor[base + so:base + so + pl].copy_(pmap[name].data.reshape(-1)[r * pl:(r + 1) * pl])
        # ---- gather slots: blocks alternate between two, everything else stays resident
        self.is_block = [u.name.startswith("block") and not u.local_only for u in engine.units]
        block_lens = [u.length for u, b in zip(engine.units, self.is_block) if b]
        max_block = max(block_lens or [8])
        self.n_slots = self._choose_slot_count(block_lens, max_block, dt)
        self.slots = [torch.empty(max_block, dtype=dt, device=dev) for _ in range(self.n_slots)]
        self.slot_content = [-1] * self.n_slots
        self.resident: Dict[int, torch.Tensor] = {}
        self.block_rank: Dict[int, int] = {}
        k = 0
        for ui, u in enumerate(engine.units):
            if self.is_block[ui]:
                self.block_rank[ui] = k
                buf = self.slots[k % self.n_slots]
                k += 1
            else:
                buf = torch.zeros(u.length, dtype=dt, device=dev)
                self.resident[ui] = buf
            for name, p in u.params:
                o, n, shape = engine.param_slices[name]
                view = buf[o - u.offset:o - u.offset + n].view(shape)
                if u.local_only:
                    view.copy_(p.data)           # nothing to gather later: the rank's own values live here
                p.data = view
        self.side = torch.cuda.Stream(device=dev) if engine.on_cuda else None
        self.ready: List[Optional[torch.cuda.Event]] = [None] * self.n_slots
        self.gathers = 0
        self.gather_ctas = int(os.environ.get("APB_ZERO3_GATHER_CTAS", "128"))   # SMs lent to a prefetch
        for ui in self.resident:
            self._gather(ui, self.resident[ui])
        self.overlap = False               # set by enable_overlapped_reduce()
        self._install_hooks()

    def _choose_slot_count(self, block_lens: List[int], max_block: int, dt: torch.dtype) -> int:
        """Two alternating slots, or one per block when the gathered blocks may stay live between uses."""
        n = len(block_lens)
        if n <= 2:
            return 2
        limit = int(getattr(self.e.cfg, "zero3_max_live_parameters", -1))
        if os.environ.get("APB_ZERO3_LIVE_PARAMETERS"):
            limit = int(float(os.environ["APB_ZERO3_LIVE_PARAMETERS"]))
        need = n * max_block
        if limit >= 0:
            return n if need <= limit else 2
        if not self.e.on_cuda:
            return 2
        total = torch.cuda.get_device_properties(self.e.device).total_memory
        return n if need * torch.empty(0, dtype=dt).element_size() * 10 <= total else 2

    # ------------------------------------------------------------------ gather
    def _gather(self, ui: int, buf: torch.Tensor) -> None:
        """All pieces of unit ``ui`` from every rank into ``buf`` (full parameter-major layout of the unit)."""
        e = self.e
        W = e.world
        if e.units[ui].local_only:
            if buf.data_ptr() != self.resident[ui].data_ptr():
                buf.copy_(self.resident[ui])
            return
        base = self.bf16_off[ui]
        self.gathers += 1
        if self.fused:
            rows = self.pieces[ui]
            s = _lib.stream_ptr()
            for lo in range(0, len(rows), 24):                     # one launch per (up to) 24 parameters
                part = rows[lo:lo + 24]
                n = len(part)
                arr = ctypes.c_longlong * n
                _lib.check(_fused_gather()(self.shard_buf.ptr_table(base * 2), e.rank, W,
                                           arr(*[r[1] for r in part]), arr(*[r[2] for r in part]),
                                           arr(*[r[3] for r in part]), n, ctypes.c_void_p(buf.data_ptr()),
                                           self.gather_ctas, s), "apb_gather_unit")
            return
        for _name, fo, pl, so in self.pieces[ui]:
            mine = self.shard_buf.tensor[base + so:base + so + pl].contiguous()
            dst = buf[fo:fo + pl * W]
            if e.on_cuda:
                dist.all_gather_into_tensor(dst, mine, group=e.group)
            else:
                parts = [torch.empty_like(mine) for _ in range(W)]
                dist.all_gather(parts, mine, group=e.group)
                for i, p in enumerate(parts):
                    dst[i * pl:(i + 1) * pl].copy_(p)

    def gather_all_into(self, dst_flat: torch.Tensor) -> None:
        """Every unit into a full flat buffer with the engine's parameter-major layout (weight sync, checkpoints)."""
        for ui, u in enumerate(self.e.units):
            self._gather(ui, dst_flat[u.offset:u.offset + u.length])

    def ensure(self, ui: int) -> None:
        """Unit ``ui`` is in its slot when this returns (on the current stream)."""
        if not self.is_block[ui]:
            return
        k = self.block_rank[ui] % self.n_slots
        if self.slot_content[k] == ui:
            if self.ready[k] is not None:
                torch.cuda.current_stream(self.e.device).wait_event(self.ready[k])
                self.ready[k] = None
            return
        if self.ready[k] is not None:      # an unconsumed prefetch may still be writing this slot
            torch.cuda.current_stream(self.e.device).wait_event(self.ready[k])
        self._gather(ui, self.slots[k])
        self.slot_content[k] = ui
        self.ready[k] = None

    def prefetch(self, ui: int) -> None:
        """Starts gathering unit ``ui`` on the side stream; its slot may still be read by work already queued on the
        main stream (the unit two positions away), so the side stream first waits for the main stream."""
        if ui < 0 or ui >= len(self.e.units) or not self.is_block[ui]:
            return
        k = self.block_rank[ui] % self.n_slots
        if self.slot_content[k] == ui:
            return
        if self.side is None or not self.fused:
            return                       # collectives stay on the main stream: ensure() gathers on demand
        main = torch.cuda.current_stream(self.e.device)
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            self._gather(ui, self.slots[k])
            ev = torch.cuda.Event()
            ev.record(self.side)
        self.slot_content[k] = ui
        self.ready[k] = ev

    def invalidate(self) -> None:
        """After an optimizer step the shards changed: slots are stale, resident units are gathered again."""
        self.slot_content = [-1] * self.n_slots
        self.ready = [None] * self.n_slots
        for ui, buf in self.resident.items():
            self._gather(ui, buf)

    # ------------------------------------------------------------------ hooks
    def _install_hooks(self) -> None:
        blocks = self.e.model.blocks
        unit_of_block = [ui for ui, b in enumerate(self.is_block) if b]

        def fwd_pre(i):
            def hook(_mod, _args):
                ui = unit_of_block[i]
                self.ensure(ui)
                if i + 1 < len(unit_of_block):
                    self.prefetch(unit_of_block[i + 1])
            return hook

        def bwd_pre(i):
            def hook(_mod, _grad_out):
                ui = unit_of_block[i]
                if self.overlap:
                    self._before_block_backward(ui)
                self.ensure(ui)
                if i - 1 >= 0:
                    self.prefetch(unit_of_block[i - 1])
            return hook

        def bwd_post(i):
            def hook(_mod, _grad_in, _grad_out):
                if self.overlap:
                    self.reduce_block_async(unit_of_block[i])
            return hook

        for i, blk in enumerate(blocks):
            blk.register_forward_pre_hook(fwd_pre(i))
            if not self.e.forward_only:
                blk.register_full_backward_pre_hook(bwd_pre(i))
                blk.register_full_backward_hook(bwd_post(i))

    # ------------------------------------------------------------------ gradient reduction overlapped with backward
    def enable_overlapped_reduce(self) -> None:
        """Called by the engine once the staging buffers exist.  The reductions run on their own stream with their
        own flag set: epochs are compared with ``>=``, so kernels of two streams must never share one counter."""
        from ..parallel.symm import EpochFlags
        e = self.e
        self.overlap = True
        self.side_r = torch.cuda.Stream(device=e.device)
        self.flags_r = EpochFlags(e.device, e.group)
        self.reduce_done: Dict[int, torch.cuda.Event] = {}       # block unit -> its reduction has finished here
        self.pass_done: Optional[torch.cuda.Event] = None        # every rank finished the previous pass's reductions
        self._unit_of_rank = {k: ui for ui, k in self.block_rank.items()}
        self._wait_fn = None

    def begin_backward(self) -> None:
        if self.overlap:
            self.reduce_done = {}

    def _before_block_backward(self, ui: int) -> None:
        """Block ``ui`` is about to accumulate into staging buffer ``rank % 3``.  Its previous user -- the block three
        positions later in this pass, or a block of the previous pass -- has been read and cleared by ALL ranks once
        this rank's reduction of the block TWO positions later has finished (every rank enters that kernel's barrier
        only after its own earlier reductions), or, at the start of a pass, once the end-of-pass barrier has."""
        main = torch.cuda.current_stream(self.e.device)
        k = self.block_rank[ui]
        ev = self.reduce_done.get(self._unit_of_rank.get(k + 2, -1))
        if ev is not None:
            main.wait_event(ev)
        elif self.pass_done is not None:
            main.wait_event(self.pass_done)

    def reduce_block_async(self, ui: int) -> None:
        e = self.e
        W, r = e.world, e.rank
        main = torch.cuda.current_stream(e.device)
        ready = torch.cuda.Event()
        ready.record(main)
        self.side_r.wait_event(ready)
        fn = _fused_reduce()
        base = e.unit_shard_off[ui]
        rows = self.pieces[ui]
        gp = e.unit_grad_table(ui)
        with torch.cuda.stream(self.side_r):
            s = _lib.stream_ptr(self.side_r)
            for lo in range(0, len(rows), 24):
                part = rows[lo:lo + 24]
                n = len(part)
                arr = ctypes.c_longlong * n
                _lib.check(fn(gp, self.flags_r.ptr_table(), r, W, self.flags_r.next(),
                              arr(*[p[1] + r * p[2] for p in part]), arr(*[p[2] for p in part]),
                              arr(*[base + p[3] for p in part]), n, 1.0 / W, _lib.ptr(e.reduced), None, 1, s),
                           "apb_zero3_reduce_unit")
            done = torch.cuda.Event()
            done.record(self.side_r)
        self.reduce_done[ui] = done

    def finish_backward(self) -> None:
        """End of a backward pass: one more barrier on the reduction stream (all ranks have finished reading and
        clearing every staging buffer), and the main stream joins it -- the optimizer step, or the next pass's first
        blocks, must see the completed shard accumulator / cleared buffers."""
        if not self.overlap:
            return
        e = self.e
        from .trainer import _fused_fns
        with torch.cuda.stream(self.side_r):
            _lib.check(_fused_fns()["wait"](self.flags_r.ptr_table(), e.rank, e.world, self.flags_r.next(),
                                            _lib.stream_ptr(self.side_r)), "apb_epoch_wait")
            ev = torch.cuda.Event()
            ev.record(self.side_r)
        self.pass_done = ev
        torch.cuda.current_stream(e.device).wait_event(ev)

    # ------------------------------------------------------------------ optimizer step
    def reduce_pieces_fused(self, fn_r, flags_tbl, s) -> None:
        e = self.e
        W, r = e.world, e.rank
        fn = _fused_reduce()
        for ui, u in enumerate(e.units):
            if u.local_only or (self.overlap and self.is_block[ui]):
                continue
            base = e.unit_shard_off[ui]
            rows = self.pieces[ui]
            gp = e.unit_grad_table(ui)
            for lo in range(0, len(rows), 24):                     # one launch (one flag barrier) per 24 parameters
                part = rows[lo:lo + 24]
                n = len(part)
                arr = ctypes.c_longlong * n
                _lib.check(fn(gp, flags_tbl, r, W, e.flags.next(), arr(*[p[1] + r * p[2] for p in part]),
                              arr(*[p[2] for p in part]), arr(*[base + p[3] for p in part]), n, 1.0 / W,
                              _lib.ptr(e.reduced), _lib.ptr(e.sumsq), 0, s), "apb_zero3_reduce_unit")

    def reduced_pieces_collective(self) -> List[torch.Tensor]:
        """Per unit: this rank's shard of the averaged gradient (shard layout)."""
        e = self.e
        W, r = e.world, e.rank
        out = []
        for ui, u in enumerate(e.units):
            gu = e.unit_grad_tensor(ui)
            if u.local_only:
                out.append(gu / W)               # complete on this rank
                continue
            dist.all_reduce(gu, group=e.group)
            parts = [gu[fo + r * pl:fo + (r + 1) * pl] for _n, fo, pl, _so in self.pieces[ui]]
            out.append(torch.cat(parts) / W)
        return out


_GATHER = None
_REDUCE = None


def _fused_reduce():
    global _REDUCE
    if _REDUCE is None:
        c = ctypes
        _REDUCE = _lib.declare("apb_zero3_reduce_unit", [c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_void_p,
                                                          c.c_void_p, c.c_void_p, c.c_int, c.c_float, c.c_void_p,
                                                          c.c_void_p, c.c_int, c.c_void_p])
    return _REDUCE


def _fused_gather():
    global _GATHER
    if _GATHER is None:
        c = ctypes
        _GATHER = _lib.declare("apb_gather_unit", [c.c_void_p, c.c_int, c.c_int, c.c_void_p, c.c_void_p, c.c_void_p,
                                                    c.c_int, c.c_void_p, c.c_int, c.c_void_p])
    return _GATHER
