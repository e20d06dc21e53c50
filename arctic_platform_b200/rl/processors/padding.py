"""Padded ``[B, S]`` grids <-> padding-free ``[1, T]`` rows, selected by a boolean attention mask.

The helpers a caller needs when it holds verl-style padded batches and wants to feed (or read back) the packed
form by hand; the pipeline itself packs through ``rl/zorro_train/layout.py``.  Names and argument order follow
arctic_platform/rl/processors/pipeline.py:96-203.  Every function is one boolean-mask gather or scatter: row-major
order of the mask IS the packed order, so no per-sequence loop is needed.  Unlike the reference, a size mismatch
between the packed values and the mask raises instead of being ignored.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

__all__ = ["compute_packing_info_for_batch", "padded_tensor_2d_dict_to_unpadded_tensor_1d_dict",
           "padded_tensor_2d_full_to_unpadded_tensor_1d_response", "padded_tensor_2d_to_unpadded_tensor_1d",
           "unpadded_tensor_1d_dict_to_padded_tensor_2d_dict", "unpadded_tensor_1d_response_dict_to_padded_tensor_2d_full_dict",
           "unpadded_tensor_1d_response_to_padded_tensor_2d_full", "unpadded_tensor_1d_to_padded_tensor_2d"]


def _bool(mask: torch.Tensor) -> torch.Tensor:
    return mask if mask.dtype == torch.bool else mask != 0


def _scatter(values: torch.Tensor, mask: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    flat = values.reshape(-1)
    want = int(mask.sum())
    if flat.numel() != want:
        raise ValueError(f"{flat.numel()} packed values for a mask that selects {want} positions")
    out[mask] = flat
    return out


def padded_tensor_2d_to_unpadded_tensor_1d(tensor_2d: torch.Tensor, attention_mask_2d_bool: torch.Tensor) -> torch.Tensor:
    """``[B, S]`` -> ``[1, T]``: the attended positions, row after row."""
    return tensor_2d[_bool(attention_mask_2d_bool)].unsqueeze(0)


def padded_tensor_2d_dict_to_unpadded_tensor_1d_dict(tensor_dict: Dict[str, Any], attention_mask_2d_bool: torch.Tensor
                                                     ) -> Dict[str, Any]:
    """Packs, in place, every tensor of the dict that has the mask's shape; everything else is left alone."""
    mask = _bool(attention_mask_2d_bool)
    for key, value in list(tensor_dict.items()):
        if torch.is_tensor(value) and value.shape == mask.shape:
            tensor_dict[key] = value[mask].unsqueeze(0)
    return tensor_dict


def unpadded_tensor_1d_to_padded_tensor_2d(tensor_1d: torch.Tensor, attention_mask_2d_bool: torch.Tensor, pad_value
                                           ) -> torch.Tensor:
    """``[1, T]`` (or ``[T]``) -> ``[B, S]`` with ``pad_value`` outside the mask."""
    mask = _bool(attention_mask_2d_bool)
    out = torch.full(mask.shape, pad_value, dtype=tensor_1d.dtype, device=tensor_1d.device)
    return _scatter(tensor_1d, mask.to(tensor_1d.device), out)


def unpadded_tensor_1d_dict_to_padded_tensor_2d_dict(tensor_dict: Dict[str, Any], attention_mask_2d_bool: torch.Tensor,
                                                     pad_value) -> Dict[str, Any]:
    for key, value in list(tensor_dict.items()):
        if torch.is_tensor(value):
            tensor_dict[key] = unpadded_tensor_1d_to_padded_tensor_2d(value, attention_mask_2d_bool, pad_value)
    return tensor_dict


def padded_tensor_2d_full_to_unpadded_tensor_1d_response(tensor_2d: torch.Tensor, attention_mask_2d_bool: torch.Tensor,
                                                         max_prompt_len: int) -> torch.Tensor:
    """The attended RESPONSE positions (columns from ``max_prompt_len`` on) of a ``[B, P + R]`` grid as ``[1, T_r]``."""
    mask = _bool(attention_mask_2d_bool)[:, max_prompt_len:]
    return tensor_2d[:, max_prompt_len:][mask].unsqueeze(0)


def unpadded_tensor_1d_response_to_padded_tensor_2d_full(tensor_1d: torch.Tensor, attention_mask_2d_bool: torch.Tensor,
                                                         max_prompt_len: int) -> torch.Tensor:
    """Packed response values back into a full ``[B, P + R]`` grid; prompt columns and padding are zero (the grid is
    a shape placeholder there)."""
    mask = _bool(attention_mask_2d_bool).to(tensor_1d.device)
    out = torch.zeros(mask.shape, dtype=tensor_1d.dtype, device=tensor_1d.device)
    _scatter(tensor_1d, mask[:, max_prompt_len:], out[:, max_prompt_len:])
    return out


def unpadded_tensor_1d_response_dict_to_padded_tensor_2d_full_dict(tensor_dict: Dict[str, Any],
                                                                   attention_mask_2d_bool: torch.Tensor,
                                                                   max_prompt_len: int) -> Dict[str, Any]:
    for key, value in list(tensor_dict.items()):
        if torch.is_tensor(value):
            tensor_dict[key] = unpadded_tensor_1d_response_to_padded_tensor_2d_full(value, attention_mask_2d_bool,
                                                                                    max_prompt_len)
    return tensor_dict


def compute_packing_info_for_batch(tensor_dict: Dict[str, Any]) -> Dict[str, Any]:
    """Adds what the packed-row consumers read: ``sequence_offsets`` (running END offset of every sequence in the
    packed row) and ``response_lens`` (attended tokens behind the ``prompts`` columns)."""
    mask = tensor_dict["attention_mask"]
    tensor_dict["sequence_offsets"] = mask.long().sum(dim=1).cumsum(dim=0)
    tensor_dict["response_lens"] = mask[:, tensor_dict["prompts"].shape[1]:].long().sum(dim=1)
    return tensor_dict
