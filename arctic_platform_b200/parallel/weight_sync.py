"""Trainer -> sampler weight synchronisation.

The reference has four routes (NCCL broadcast groups, CUDA-IPC bulk, CUDA-IPC streaming, CPU file:
arctic_platform/common/utils/weight_sync.py:47-187, common/ray_server.py:1099-1165), all of which first
all-gather every ZeRO-3 parameter one by one on the sender and then copy ~310 tensors one at a time.
Here the sampler keeps its parameters in ONE flat bf16 buffer with exactly the trainer's layout
(:func:`flatten_like`), so a sync is a single kernel (``sync_weights_flat_kernel`` in ``optim.cu``):
every 16-byte piece of the destination is read from the rank that owns it -- through the NVLink peer
mapping when the trainer state is ZeRO-sharded -- and written once.  Optional block-scaled fp8
(e4m3, 128 x 128 blocks) copies of the matrix weights are produced by ``quant_fp8_block128_kernel``.

When the sampler's layout differs from the trainer's -- a tensor-parallel replica keeps head / column shards, an
fp8 sampler keeps block-scaled e4m3 matrices -- the sync is still ONE kernel, driven by a table
(:class:`SyncPlan`, ``sync_weights_table_kernel``): every 128 x 128 tile of every destination slice is read once
from the rank that owns it (ZeRO-3 pieces over NVLink, or a replicated buffer), written as bf16 and / or quantised
to e4m3 with its block scale in the same pass.  A sampler in ANOTHER process (split placement) opens the trainer
ranks' buffers through IPC handles (:func:`export_ipc` / :func:`open_ipc`) and runs the same kernel, pulling over
NVLink instead of receiving tensors through the host.

``sync_state_dict`` is the name-based fallback (different layouts, CPU, cross-process): it walks the
Hugging Face tensor names, validates that every expected name arrived and returns the count.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch

from ..ops import _lib

_FN: Dict[str, object] = {}


def _fns():
    if not _FN:
        c = ctypes
        vp, i, ll = c.c_void_p, c.c_int, c.c_longlong
        _FN["flat"] = _lib.declare("apb_sync_weights_flat", [vp, vp, i, i, i, i, vp, vp, i, vp, ll, vp])
        _FN["fp8"] = _lib.declare("apb_quant_fp8_block128", [vp, ll, i, i, vp, ll, vp, vp])
        _FN["table"] = _lib.declare("apb_sync_weights_table", [vp, i, ll, vp, i, i, vp, i, i, i, vp, vp, vp, i, vp])
        _FN["seg_bytes"] = _lib.declare("apb_sync_seg_bytes", [])
        _FN["ipc_export"] = _lib.declare("apb_ipc_export", [vp, vp, vp])
        _FN["ipc_open"] = _lib.declare("apb_ipc_open", [vp, ll, vp])
        _FN["ipc_close"] = _lib.declare("apb_ipc_close", [vp, ll])
    return _FN


@torch.no_grad()
def flatten_like(model, engine) -> torch.Tensor:
    """Re-points ``model``'s parameters into one flat buffer with the layout of ``engine`` (same units,
    offsets and padding) and returns that buffer."""
    flat = torch.zeros(engine.total, dtype=next(model.parameters()).dtype, device=next(model.parameters()).device)
    named = {}
    named["embed"] = model.embed
    if model.lm_head is not None:
        named["lm_head"] = model.lm_head
    named["final_norm"] = model.final_norm
    for i, blk in enumerate(model.blocks):
        for n, p in blk.named_parameters():
            named[f"blocks.{i}.{n}"] = p
    for name, (off, n, shape) in engine.param_slices.items():
        p = named[name]
        view = flat[off:off + n].view(shape)
        if p.data.numel() == n:
            view.copy_(p.data)
        p.data = view
    model._flat_params = flat
    return flat


@torch.no_grad()
def sync_flat(engine, dst_flat: torch.Tensor, stream=None) -> int:
    """One-kernel sync from the training engine's parameter buffer into ``dst_flat`` (same layout).
    Returns the number of bytes written."""
    if getattr(engine, "zero3", None) is not None:
        # stage 3: the gather of every rank's shards IS the sync -- each unit is pulled from the owners straight
        # into the sampler's buffer (same parameter-major layout), no intermediate full copy on the trainer
        if dst_flat.numel() != engine.total or dst_flat.dtype != engine.param_dtype:
            raise ValueError("destination buffer does not have the trainer's flat layout")
        engine.zero3.gather_all_into(dst_flat)
        return dst_flat.numel() * dst_flat.element_size()
    if not dst_flat.is_cuda:
        dst_flat.copy_(engine.param_buf.tensor.to(dst_flat.dtype))
        return dst_flat.numel() * dst_flat.element_size()
    if dst_flat.numel() != engine.total or dst_flat.dtype != torch.bfloat16:
        raise ValueError("destination buffer does not have the trainer's flat layout")
    n_units = len(engine.units)
    offs = (ctypes.c_longlong * n_units)(*[u.offset for u in engine.units])
    lens = (ctypes.c_longlong * n_units)(*[u.length for u in engine.units])
    flags = engine.flags
    W = engine.param_buf.world
    epoch = flags.next() if W > 1 else 0
    code = _fns()["flat"](engine.param_buf.ptr_table(), flags.ptr_table(), engine.param_buf.rank, W, epoch, 0,
                          offs, lens, n_units, _lib.ptr(dst_flat), engine.total, _lib.stream_ptr(stream))
    _lib.check(code, "apb_sync_weights_flat")
    return engine.total * 2


@torch.no_grad()
def quantize_fp8_block128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w [N, K]`` bf16 -> ``(q [N, K] float8_e4m3fn, scales [ceil(N/128), ceil(K/128)] fp32)`` with
    ``w ~= q * scale`` per 128 x 128 block."""
    N, K = w.shape
    if not w.is_cuda:
        wf = w.float()
        pad = torch.zeros(((N + 127) // 128 * 128, (K + 127) // 128 * 128))
        pad[:N, :K] = wf
        blocks = pad.view(pad.shape[0] // 128, 128, pad.shape[1] // 128, 128)
        amax = blocks.abs().amax(dim=(1, 3))
        scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
        q = (blocks / scale[:, None, :, None]).view_as(pad)[:N, :K].to(torch.float8_e4m3fn)
        return q, scale
    q = torch.empty((N, K), device=w.device, dtype=torch.float8_e4m3fn)
    scales = torch.empty(((N + 127) // 128, (K + 127) // 128), device=w.device, dtype=torch.float32)
    _lib.check(_fns()["fp8"](_lib.ptr(w), w.stride(0), N, K, _lib.ptr(q), q.stride(0), _lib.ptr(scales),
                             _lib.stream_ptr()), "apb_quant_fp8_block128")
    return q, scales


@torch.no_grad()
def sync_state_dict(named_tensors: Iterable[Tuple[str, torch.Tensor]], dst_model, expected_names=None) -> int:
    """Name-based sync: copies every ``(hf_name, tensor)`` into ``dst_model`` and checks the name set."""
    from ..models.hf_io import hf_param_names, load_hf_tensor
    expected = set(expected_names if expected_names is not None else hf_param_names(dst_model.cfg))
    seen = set()
    for name, t in named_tensors:
        load_hf_tensor(dst_model, name, t)
        seen.add(name)
    missing = expected - seen
    if missing:
        raise KeyError(f"weight sync is missing {len(missing)} tensors, e.g. {sorted(missing)[:3]}")
    return len(seen)


# ----------------------------------------------------------------------------- table-driven sync
class _SyncSeg(ctypes.Structure):
    """Mirror of ``apb::SyncSeg`` (``optim.cu``)."""
    _fields_ = [("src_elem", ctypes.c_longlong), ("piece_len", ctypes.c_longlong), ("shard_off", ctypes.c_longlong),
                ("dst_elem", ctypes.c_longlong), ("q_off", ctypes.c_longlong), ("scale_off", ctypes.c_longlong),
                ("tile_start", ctypes.c_longlong),
                ("src_ld", ctypes.c_int), ("row0", ctypes.c_int), ("col0", ctypes.c_int), ("rows", ctypes.c_int),
                ("cols", ctypes.c_int), ("dst_ld", ctypes.c_int), ("q_ld", ctypes.c_int), ("scale_ld", ctypes.c_int),
                ("fp8", ctypes.c_int), ("tiles_c", ctypes.c_int)]


FP8_MATRICES = ("wqkv", "wo", "wgu", "wdown")


def trainer_layout(engine) -> Dict[str, Any]:
    """What a sync plan needs to know about the trainer, as plain data (it travels to a sampler in another process):
    the flat offset and shape of every parameter and, under ZeRO-3, the piece length and shard offset of each."""
    out = {"total": int(engine.total), "world": int(engine.world), "dtype": str(engine.param_dtype),
           "params": {n: (int(o), int(k), tuple(int(x) for x in shp)) for n, (o, k, shp) in engine.param_slices.items()},
           "zero3": None}
    z = getattr(engine, "zero3", None)
    if z is not None:
        pieces = {}
        for ui, rows in enumerate(z.pieces):
            for name, _fo, pl, so in rows:
                pieces[name] = (int(pl), int(z.bf16_off[ui] + so))
        out["zero3"] = pieces
    return out


def _model_params(model) -> Dict[str, torch.nn.Parameter]:
    named = {"embed": model.embed, "final_norm": model.final_norm}
    if model.lm_head is not None:
        named["lm_head"] = model.lm_head
    for i, blk in enumerate(model.blocks):
        for n, p in blk.named_parameters():
            named[f"blocks.{i}.{n}"] = p
    return named


def _tp_slices(leaf: str, full_shape, cfg, tp_rank: int, tp: int) -> List[Tuple[int, int, int, int, int]]:
    """``[(dst_row0, src_row0, src_col0, rows, cols)]``: which rectangles of the full parameter make up this rank's
    tensor-parallel shard (Megatron split: q / k / v by heads, o and down by input columns, gate/up by rows)."""
    if len(full_shape) == 1:
        return [(0, 0, 0, 1, full_shape[0])]
    R, C = full_shape
    if tp == 1:
        return [(0, 0, 0, R, C)]
    if leaf == "wqkv":
        D = cfg.head_dim
        q, kv = cfg.num_heads * D, cfg.num_kv_heads * D
        ql, kl = q // tp, kv // tp
        return [(0, tp_rank * ql, 0, ql, C), (ql, q + tp_rank * kl, 0, kl, C), (ql + kl, q + kv + tp_rank * kl, 0, kl, C)]
    if leaf in ("wo", "wdown"):
        return [(0, 0, tp_rank * (C // tp), R, C // tp)]
    if leaf in ("wgu", "wgate"):
        return [(0, tp_rank * (R // tp), 0, R // tp, C)]
    return [(0, 0, 0, R, C)]


@dataclass
class SyncPlan:
    """Device table + destination buffers of one sampler rank.  ``dst_flat`` holds the sampler model's parameters
    (the model's tensors are views into it); ``fp8[(layer, name)] = (q [N, K] float8_e4m3fn, scales)`` when the
    projection matrices are also kept block-scaled."""
    segs: torch.Tensor
    n_seg: int
    total_tiles: int
    dst_flat: torch.Tensor
    q_buf: Optional[torch.Tensor]
    scale_buf: Optional[torch.Tensor]
    fp8: Dict[Tuple[int, str], Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)
    src_bytes: int = 0
    dst_bytes: int = 0
    layout_key: Any = None


@torch.no_grad()
def build_sync_plan(layout: Dict[str, Any], model, full_cfg=None, tp_rank: int = 0, tp: int = 1, fp8: bool = False,
                    keep_bf16: bool = True) -> SyncPlan:
    """Table for ``model`` (a sampler's decoder: full, or one tensor-parallel shard built from ``tp_config``) fed
    from a trainer with ``layout``.  Re-points the model's parameters into one flat bf16 buffer."""
    cfg = full_cfg if full_cfg is not None else model.cfg
    if cfg.is_moe:
        raise NotImplementedError("the table-driven weight sync covers dense decoders; mixture-of-experts models use "
                                  "the name-based hand-over")
    params = _model_params(model)
    dev = next(model.parameters()).device
    # shapes survive a sleep that dropped the weights (the tensors are then empty placeholders)
    kept = getattr(model, "_param_shapes", None) or {}
    shapes = {name: tuple(kept.get(name, p.shape)) for name, p in params.items()}
    model._param_shapes = shapes

    def numel(shape):
        n = 1
        for d in shape:
            n *= int(d)
        return n

    # ---- destination flat buffer (8-element aligned parameters)
    offs, cur = {}, 0
    for name in params:
        offs[name] = cur
        cur = (cur + numel(shapes[name]) + 7) // 8 * 8
    flat = torch.zeros(max(cur, 8), dtype=torch.bfloat16, device=dev)
    for name, p in params.items():
        view = flat[offs[name]:offs[name] + numel(shapes[name])].view(shapes[name])
        if p.data.numel() == view.numel():
            view.copy_(p.data)
        p.data = view
    model._flat_params = flat
    # ---- fp8 buffers
    q_total = s_total = 0
    fp8_place = {}
    if fp8:
        for name, p in params.items():
            leaf = name.split(".")[-1]
            if leaf in FP8_MATRICES and p.dim() == 2:
                N, K = p.shape
                fp8_place[name] = (q_total, s_total, N, K)
                q_total += (N * K + 15) // 16 * 16
                s_total += ((N + 127) // 128) * ((K + 127) // 128)
    q_buf = torch.zeros(max(q_total, 16), dtype=torch.uint8, device=dev) if fp8 else None
    scale_buf = torch.ones(max(s_total, 1), dtype=torch.float32, device=dev) if fp8 else None
    # ---- segments
    segs: List[_SyncSeg] = []
    tiles = 0
    src_bytes = dst_bytes = 0
    z3 = layout.get("zero3")
    for name, p in params.items():
        if name not in layout["params"]:
            raise KeyError(f"the trainer has no parameter {name!r}")
        src_off, _n, full_shape = layout["params"][name]
        leaf = name.split(".")[-1]
        src_ld = full_shape[-1] if len(full_shape) == 2 else full_shape[0]
        local_cols = p.shape[-1] if p.dim() == 2 else p.shape[0]
        place = fp8_place.get(name)
        rows_seen = 0
        for dst_row0, r0, c0, rows, cols in _tp_slices(leaf, full_shape, cfg, tp_rank, tp):
            if cols % 8 or c0 % 8 or src_ld % 8:
                raise ValueError(f"{name}: slices must be multiples of 8 elements wide")
            sg = _SyncSeg()
            sg.src_elem = src_off
            sg.piece_len, sg.shard_off = (z3[name] if z3 is not None else (0, 0))
            sg.src_ld, sg.row0, sg.col0, sg.rows, sg.cols = src_ld, r0, c0, rows, cols
            want_bf16 = keep_bf16 or place is None
            sg.dst_elem = offs[name] + dst_row0 * local_cols if want_bf16 else -1
            sg.dst_ld = local_cols
            sg.fp8 = 0
            if place is not None:
                if dst_row0 % 128:
                    raise ValueError(f"{name}: a shard boundary at row {dst_row0} cuts a 128-row fp8 block")
                q0, s0, N, K = place
                sg.fp8 = 1
                sg.q_off = q0 + dst_row0 * K
                sg.q_ld = K
                sg.scale_ld = (K + 127) // 128
                sg.scale_off = s0 + (dst_row0 // 128) * sg.scale_ld
            sg.tiles_c = (cols + 127) // 128
            sg.tile_start = tiles
            tiles += ((rows + 127) // 128) * sg.tiles_c
            segs.append(sg)
            rows_seen += rows
            src_bytes += rows * cols * 2
            dst_bytes += rows * cols * ((2 if want_bf16 else 0) + (1 if place is not None else 0))
        expect_rows = p.shape[0] if p.dim() == 2 else 1
        if rows_seen != expect_rows:
            raise ValueError(f"{name}: slices cover {rows_seen} rows, the sampler's tensor has {expect_rows}")
    n = len(segs)
    from ..utils import checked
    if checked.enabled():                       # host records: extents of every slice inside source and destination
        for i, sg in enumerate(segs):
            last_src = sg.src_elem + (sg.row0 + sg.rows - 1) * sg.src_ld + sg.col0 + sg.cols
            if sg.src_elem < 0 or last_src > layout["total"]:
                raise checked.TableError(f"sync segment {i}: source elements up to {last_src} of {layout['total']}")
        live = [sg for sg in segs if sg.dst_elem >= 0]
        checked.check_copy_table("sync plan", [0] * len(live), [sg.dst_elem for sg in live],
                                 [(sg.rows - 1) * sg.dst_ld + sg.cols for sg in live], 1 << 62, flat.numel())
    if _fns()["seg_bytes"]() != ctypes.sizeof(_SyncSeg):
        raise RuntimeError("sync table record layout differs between the library and its Python mirror")
    arr = (_SyncSeg * n)(*segs)
    host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
    seg_dev = host.to(dev)
    plan = SyncPlan(seg_dev, n, tiles, flat, q_buf, scale_buf, {}, src_bytes, dst_bytes,
                    (layout["total"], layout["world"], layout["zero3"] is not None, tp_rank, tp, fp8, keep_bf16))
    if fp8:
        f8 = torch.float8_e4m3fn
        for name, (q0, s0, N, K) in fp8_place.items():
            parts = name.split(".")
            li = int(parts[1])
            q = q_buf[q0:q0 + N * K].view(f8).view(N, K)
            sc = scale_buf[s0:s0 + ((N + 127) // 128) * ((K + 127) // 128)].view((N + 127) // 128, (K + 127) // 128)
            plan.fp8[(li, parts[-1])] = (q, sc)
    return plan


@torch.no_grad()
def run_sync_plan(plan: SyncPlan, src_ptrs: List[int], src_rank: int = 0, flags=None, rank: int = 0, world: int = 1,
                  max_ctas: int = 0, stream=None) -> int:
    """Launches the one kernel.  ``src_ptrs``: device addresses of the trainer ranks' parameter buffers as this
    process sees them (local / symmetric / opened IPC).  ``flags`` (:class:`EpochFlags`) + ``world`` > 1: the ranks
    that launch together first meet in an epoch barrier (every trainer shard is final).  Returns bytes written."""
    tbl = (ctypes.c_void_p * len(src_ptrs))(*[int(x) for x in src_ptrs])
    if flags is not None and world > 1:
        fl, epoch = flags.ptr_table(), flags.next()
    else:
        fl, epoch, world = None, 0, 1
    code = _fns()["table"](_lib.ptr(plan.segs), plan.n_seg, plan.total_tiles, tbl, len(src_ptrs), int(src_rank), fl,
                           int(rank), int(world), int(epoch), _lib.ptr(plan.dst_flat),
                           _lib.ptr(plan.q_buf) if plan.q_buf is not None else None,
                           _lib.ptr(plan.scale_buf) if plan.scale_buf is not None else None, int(max_ctas),
                           _lib.stream_ptr(stream))
    _lib.check(code, "apb_sync_weights_table")
    return plan.dst_bytes


def engine_source(engine) -> Tuple[List[int], int]:
    """``(addresses, src_rank)`` of a trainer engine's parameter storage in THIS process: the ZeRO-3 shard buffers of
    all ranks (peer mappings), or this rank's replicated flat buffer."""
    if getattr(engine, "zero3", None) is not None:
        return [int(x) for x in engine.zero3.shard_buf.peer_ptrs], int(engine.rank)
    return [int(engine.param_buf.tensor.data_ptr())], 0


def export_ipc(t: torch.Tensor) -> Tuple[bytes, int]:
    """Opaque handle of the allocation behind ``t`` plus the tensor's byte offset inside it; send both to the process
    that wants to read the tensor over NVLink (:func:`open_ipc`).  The tensor must stay alive while it is mapped."""
    buf = ctypes.create_string_buffer(64)
    off = ctypes.c_longlong(0)
    _lib.check(_fns()["ipc_export"](_lib.ptr(t), ctypes.cast(buf, ctypes.c_void_p),
                                    ctypes.cast(ctypes.pointer(off), ctypes.c_void_p)), "apb_ipc_export")
    return bytes(buf.raw), int(off.value)


def open_ipc(handle: bytes, offset: int) -> int:
    """Maps another process's allocation into this one and returns the device address of the exported tensor."""
    torch.cuda.current_stream()                       # a context on the current device
    _lib.stream_ptr()
    buf = ctypes.create_string_buffer(handle, 64)
    out = ctypes.c_void_p(0)
    _lib.check(_fns()["ipc_open"](ctypes.cast(buf, ctypes.c_void_p), int(offset),
                                  ctypes.cast(ctypes.pointer(out), ctypes.c_void_p)), "apb_ipc_open")
    return int(out.value)


def close_ipc(address: int, offset: int) -> None:
    _fns()["ipc_close"](ctypes.c_void_p(int(address)), int(offset))
