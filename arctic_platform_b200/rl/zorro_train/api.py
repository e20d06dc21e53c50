"""``ZoRRoTrain``: the prompt-deduplication entry points under the reference's class and method names.

The reference exposes its algorithm as static methods of one class that pass a ``reconstruction_info`` dict around
(arctic_platform/rl/zorro_train/zorro_train.py:238-2470) and patches the model's attention to use it.  This build
keeps the layout in ``PackedBatch`` index tables (``layout.py``) and resolves the shared prefix inside the attention
kernel, so nothing is patched; this module is the same call surface for code written against the class:

    groups, prompts = ZoRRoTrain.find_prompt_groups(input_ids, response_length)
    ids, pos, info = ZoRRoTrain.create_deduplicated_batch(input_ids, position_ids, response_length, groups, prompts,
                                                          attention_mask=mask, use_unpad=True)
    hidden = model(ids, pos, ...)                           # [1, T_dedup, H]
    full = ZoRRoTrain.reconstruct_sequences(hidden, info)   # [1, sum_b (P_b + R_b), H]

``info`` is a ``ReconstructionInfo`` (a dict that is only ever updated in place) whose ``"packed"`` entry is the
``PackedBatch``; every method also accepts the ``PackedBatch`` itself.  Only the padding-free form is produced
(``use_unpad`` is accepted and ignored): a padded deduplicated batch has no use here.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple, Union

import numpy as np
import torch

from . import reconstruct as _rc
from .layout import PackedBatch, build_packed_batch, find_prompt_groups as _group_ids

__all__ = ["ReconstructionInfo", "ZoRRoTrain", "analyze_normal_batch_via_attention_mask", "reconstruct_sequence"]


class ReconstructionInfo(dict):
    """A dict whose identity persists: holders of a reference see ``update()`` (closures over it stay valid)."""


Info = Union[PackedBatch, Dict[str, Any]]


def _packed(info: Info) -> PackedBatch:
    if isinstance(info, PackedBatch):
        return info
    pb = info.get("packed") if isinstance(info, dict) else None
    if not isinstance(pb, PackedBatch):
        raise TypeError("expected the info returned by ZoRRoTrain.create_deduplicated_batch (or a PackedBatch)")
    return pb


def _rows(t: torch.Tensor) -> Tuple[torch.Tensor, bool]:
    """``[1, T, ...]`` -> ``[T, ...]`` (and whether the batch dim has to be put back)."""
    lead = t.dim() >= 2 and t.shape[0] == 1
    return (t[0], True) if lead else (t, False)


def _like(t: torch.Tensor, lead: bool) -> torch.Tensor:
    return t.unsqueeze(0) if lead else t


def analyze_normal_batch_via_attention_mask(input_ids: torch.Tensor, attention_mask: torch.Tensor,
                                            padded_response_len: int) -> Dict[str, Any]:
    """Token accounting of a padded ``[B, P + R]`` batch: valid prompt / response tokens per sample and what
    prompt de-duplication would save."""
    mask = attention_mask.bool()
    P = input_ids.shape[1] - int(padded_response_len)
    prompt_lens = mask[:, :P].sum(1)
    response_lens = mask[:, P:].sum(1)
    pb = build_packed_batch(input_ids, attention_mask, int(padded_response_len))
    return {"batch_size": int(input_ids.shape[0]), "prompt_lens": prompt_lens.tolist(), "response_lens": response_lens.tolist(),
            "total_tokens": int(mask.sum()), "padded_tokens": int(mask.numel()), "num_groups": pb.num_groups,
            "dedup_tokens": pb.total_tokens, "redundancy": pb.redundancy}


def reconstruct_sequence(dedup: torch.Tensor, info: Info) -> torch.Tensor:
    """Free-function spelling of :meth:`ZoRRoTrain.reconstruct_sequences`."""
    return ZoRRoTrain.reconstruct_sequences(dedup, info)


class ZoRRoTrain:
    """Prompt de-duplication: stateless, every method is static."""

    @staticmethod
    def find_prompt_groups(input_ids: torch.Tensor, response_length: int) -> Tuple[List[List[int]], torch.Tensor]:
        """-> (sample indices per distinct prompt, in order of first appearance; the distinct prompts ``[G, P]``)."""
        ids = _group_ids(input_ids, int(response_length))
        groups: List[List[int]] = [[] for _ in range(int(ids.max()) + 1 if len(ids) else 0)]
        for b, g in enumerate(ids.tolist()):
            groups[g].append(b)
        P = input_ids.shape[1] - int(response_length)
        first = torch.tensor([g[0] for g in groups], dtype=torch.long, device=input_ids.device)
        return groups, input_ids.index_select(0, first)[:, :P]

    @staticmethod
    def create_deduplicated_batch(input_ids: torch.Tensor, position_ids: Optional[torch.Tensor], response_length: int,
                                  prompt_groups: Optional[List[List[int]]] = None,
                                  unique_prompts: Optional[torch.Tensor] = None,
                                  attention_mask: Optional[torch.Tensor] = None, use_unpad: bool = True
                                  ) -> Tuple[torch.Tensor, torch.Tensor, ReconstructionInfo]:
        """-> ``(input ids [1, T], position ids [1, T], info)``: every distinct prompt once, followed by the responses
        that share it, padding removed.  Positions restart per prompt and continue from the prompt's end in every
        response.  ``position_ids`` of the input are not needed (they follow from the mask)."""
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        group_of = None
        if prompt_groups is not None:
            group_of = np.zeros(input_ids.shape[0], dtype=np.int32)
            for g, members in enumerate(prompt_groups):
                group_of[list(members)] = g
        pb = build_packed_batch(input_ids, attention_mask, int(response_length), dedup=True, group_of=group_of)
        info = ReconstructionInfo(packed=pb, batch_size=pb.batch_size, response_length=pb.response_length,
                                  num_groups=pb.num_groups, total_tokens=pb.total_tokens, full_tokens=pb.full_tokens,
                                  prompt_groups=prompt_groups, is_packed=True)
        dev = input_ids.device
        return pb.input_ids.to(dev).unsqueeze(0), pb.positions.to(dev).long().unsqueeze(0), info

    @staticmethod
    def unpad_deduplicated_batch(dedup_input_ids, dedup_position_ids, reconstruction_info: Info):
        """The batch is padding-free already: returned unchanged."""
        return dedup_input_ids, dedup_position_ids, reconstruction_info

    @staticmethod
    def reconstruct_sequences(dedup_hidden: torch.Tensor, reconstruction_info: Info) -> torch.Tensor:
        """``[1, T_dedup, ...]`` -> ``[1, sum_b (P_b + R_b), ...]``: every sample's prompt + response, original order."""
        rows, lead = _rows(dedup_hidden)
        return _like(_rc.reconstruct_sequences(rows, _packed(reconstruction_info))[0], lead)

    @staticmethod
    def deduplicate_sequences(full_hidden: torch.Tensor, reconstruction_info: Info, reduce: str = "sum") -> torch.Tensor:
        """Inverse of :meth:`reconstruct_sequences`; the copies of a shared prompt row are summed (gradients) or the
        first is kept (``reduce="first"``, activations)."""
        rows, lead = _rows(full_hidden)
        return _like(_rc.deduplicate_sequences(rows, _packed(reconstruction_info), reduce), lead)

    @staticmethod
    def reconstruct_input_ids(dedup_input_ids: torch.Tensor, reconstruction_info: Info) -> torch.Tensor:
        return ZoRRoTrain.reconstruct_sequences(dedup_input_ids, reconstruction_info)

    @staticmethod
    def reconstruct_position_ids(dedup_pos: torch.Tensor, reconstruction_info: Info) -> torch.Tensor:
        return ZoRRoTrain.reconstruct_sequences(dedup_pos, reconstruction_info)

    @staticmethod
    def get_reconstructed_shape(dedup_shape: tuple, reconstruction_info: Info) -> tuple:
        pb = _packed(reconstruction_info)
        shape = tuple(dedup_shape)
        axis = 1 if len(shape) >= 2 and shape[0] == 1 else 0
        return shape[:axis] + (int(pb.full_tokens),) + shape[axis + 1:]

    @staticmethod
    def extract_response_queries(query_states: torch.Tensor, reconstruction_info: Info) -> torch.Tensor:
        """The rows of the de-duplicated axis that belong to responses (their own positions)."""
        rows, lead = _rows(query_states)
        return _like(_rc.extract_responses(rows, _packed(reconstruction_info), offset=0), lead)

    @staticmethod
    def extract_unpadded_responses_from_deduped_packed_ids(dedup: torch.Tensor, reconstruction_info: Info,
                                                           predictors: bool = False) -> torch.Tensor:
        """Per-response-token rows, samples in original order, no padding.  ``predictors=True`` takes the rows whose
        hidden states PREDICT those tokens (one position earlier) -- what a log-prob computation reads."""
        rows, lead = _rows(dedup)
        return _like(_rc.extract_responses(rows, _packed(reconstruction_info), offset=-1 if predictors else 0), lead)

    @staticmethod
    def extract_padded_responses_from_deduped_packed_ids(dedup: torch.Tensor, reconstruction_info: Info,
                                                         predictors: bool = False, fill: float = 0.0) -> torch.Tensor:
        pb = _packed(reconstruction_info)
        rows, _ = _rows(dedup)
        return _rc.pad_responses(_rc.extract_responses(rows, pb, offset=-1 if predictors else 0), pb, fill)

    @staticmethod
    def pad_responses(packed_responses: torch.Tensor, reconstruction_info: Info, fill: float = 0.0) -> torch.Tensor:
        """Per-response-token values (original sample order) -> ``[B, R, ...]``."""
        rows, _ = _rows(packed_responses)
        return _rc.pad_responses(rows, _packed(reconstruction_info), fill)

    @staticmethod
    def responses_in_orig_sample_order(packed_responses: torch.Tensor, reconstruction_info: Info) -> List[torch.Tensor]:
        rows, _ = _rows(packed_responses)
        return _rc.responses_in_orig_sample_order(rows, _packed(reconstruction_info))

    @staticmethod
    def get_group_token_layout(reconstruction_info: Info) -> List[dict]:
        return _rc.get_group_token_layout(_packed(reconstruction_info))

    @staticmethod
    def split_deduplicated_hidden_by_group(dedup_hidden: torch.Tensor, reconstruction_info: Info) -> List[dict]:
        rows, _ = _rows(dedup_hidden)
        return _rc.split_deduplicated_hidden_by_group(rows, _packed(reconstruction_info))
