"""Trainer -> sampler weight synchronisation.

The reference has four routes (NCCL broadcast groups, CUDA-IPC bulk, CUDA-IPC streaming, CPU file:
arctic_platform/common/utils/weight_sync.py:47-187, common/ray_server.py:1099-1165), all of which first
all-gather every ZeRO-3 parameter one by one on the sender and then copy ~310 tensors one at a time.
Here the sampler keeps its parameters in ONE flat bf16 buffer with exactly the trainer's layout
(:func:`flatten_like`), so a sync is a single kernel (``sync_weights_flat_kernel`` in ``optim.cu``):
every 16-byte piece of the destination is read from the rank that owns it -- through the NVLink peer
mapping when the trainer state is ZeRO-sharded -- and written once.  Optional block-scaled fp8
(e4m3, 128 x 128 blocks) copies of the matrix weights are produced by ``quant_fp8_block128_kernel``.

``sync_state_dict`` is the name-based fallback (different layouts, CPU, cross-process): it walks the
Hugging Face tensor names, validates that every expected name arrived and returns the count.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Iterable, Optional, Tuple

import torch

from ..ops import _lib

_FN: Dict[str, object] = {}


def _fns():
    if not _FN:
        c = ctypes
        vp, i, ll = c.c_void_p, c.c_int, c.c_longlong
        _FN["flat"] = _lib.declare("apb_sync_weights_flat", [vp, vp, i, i, i, i, vp, vp, i, vp, ll, vp])
        _FN["fp8"] = _lib.declare("apb_quant_fp8_block128", [vp, ll, i, i, vp, ll, vp, vp])
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
