"""Padded ``[B, S]`` <-> packed ``[1, T]`` conversion for callers that want the packed tensors themselves
(position ids, ``cu_seqlens``) -- the engine's own path builds its layout in ``zorro_train/layout.py``.
Contract of arctic_platform/rl/processors/packing.py:32-107."""
from __future__ import annotations

from typing import Any, Dict

import torch


def pack_sequences(batch: Dict[str, torch.Tensor]) -> Dict[str, Any]:
    ids, mask = batch["input_ids"], batch["attention_mask"].bool()
    B, S = ids.shape
    lens = mask.sum(-1)
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = lens.cumsum(0)
    flat_idx = mask.reshape(-1).nonzero(as_tuple=False).squeeze(-1)
    out: Dict[str, Any] = {"input_ids": ids.reshape(-1)[flat_idx][None]}
    pos = (mask.long().cumsum(-1) - 1).clamp_min(0)
    out["position_ids"] = pos.reshape(-1)[flat_idx][None]
    out["cu_seqlens"] = cu
    out["max_seqlen"] = int(lens.max()) if B else 0
    for k, v in batch.items():
        if k in ("input_ids", "attention_mask", "position_ids"):
            continue
        if torch.is_tensor(v) and v.shape[:2] == (B, S):
            out[k] = v.reshape(B * S, *v.shape[2:])[flat_idx][None]
        else:
            out[k] = v
    out["_pack_meta"] = {"flat_idx": flat_idx, "shape": (B, S)}
    return out


def pad_packed_for_model(packed: Dict[str, Any], multiple: int = 256) -> Dict[str, Any]:
    """Pads the token axis to a multiple (extra tokens form one trailing dummy sequence) and adds the
    flash-attention style keyword names."""
    T = packed["input_ids"].shape[1]
    pad = (-T) % multiple
    out = dict(packed)
    if pad:
        for k in ("input_ids", "position_ids"):
            out[k] = torch.nn.functional.pad(packed[k], (0, pad))
        cu = packed["cu_seqlens"]
        out["cu_seqlens"] = torch.cat([cu, cu[-1:] + pad])
        out["max_seqlen"] = max(packed["max_seqlen"], pad)
    out["cu_seq_lens_q"] = out["cu_seq_lens_k"] = out["cu_seqlens"]
    out["max_length_q"] = out["max_length_k"] = out["max_seqlen"]
    return out


def unpack_sequences(values: torch.Tensor, pack_meta: Dict[str, Any], fill: float = 0.0) -> torch.Tensor:
    """``[1, T, ...]`` (or ``[T, ...]``) back to ``[B, S, ...]`` with ``fill`` at padded positions."""
    B, S = pack_meta["shape"]
    idx = pack_meta["flat_idx"]
    v = values[0] if values.dim() >= 2 and values.shape[0] == 1 else values
    v = v[: idx.numel()]
    out = v.new_full((B * S, *v.shape[1:]), fill)
    out[idx] = v
    return out.view(B, S, *v.shape[1:])
