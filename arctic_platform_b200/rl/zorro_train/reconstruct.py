"""Tensor-level views of the ZoRRo layout for code that wants the tensors themselves.

The engine never materialises these (attention resolves the shared prefix in the kernel), but frameworks
and tests do: ``reconstruct_sequences`` expands a deduplicated ``[T_dedup, ...]`` tensor to the full packed
per-sample layout (prompt rows repeated per rollout), ``deduplicate_sequences`` is its inverse (sum or first),
``extract_responses`` pulls predictor rows (``offset=-1``) or label rows (``offset=0``) per rollout, and
``responses_in_orig_sample_order`` / ``pad_responses`` arrange per-rollout pieces as a padded grid.
Counterparts of arctic_platform/rl/zorro_train/zorro_train.py:724-2017 built on ``PackedBatch`` index tables
(one ``index_select`` each, no per-segment Python loops on the device tensors)."""
from __future__ import annotations

from typing import List, Tuple

import numpy as np
import torch

from .layout import PackedBatch


def _full_index(pb: PackedBatch) -> Tuple[torch.Tensor, np.ndarray]:
    """For every token of the NON-deduplicated packing (samples in original order, prompt then response) the
    row of the deduplicated axis it corresponds to, plus per-sample lengths."""
    segs = pb.layout.segs
    prompts = {int(s[0]): int(s[1]) for s in segs if s[3] == 0}                 # prompt start -> length
    resp = [(int(s[0]), int(s[1]), int(s[2]), int(s[3])) for s in segs if s[3] > 0 or s[0] not in prompts]
    # response segments carry (q_start, q_len, pre_start, pre_len); order them by original sample via out_index
    B, R = pb.batch_size, pb.response_length
    first_of_sample = {}
    pos = 0
    oi = pb.out_index.cpu().numpy()
    pred = pb.pred_index.cpu().numpy()
    labels_rows = {}
    k = 0
    idx_parts: List[np.ndarray] = []
    lens = np.zeros(B, dtype=np.int64)
    by_start = {r[0]: r for r in resp}
    # reconstruct each sample's response start from pred_index (second predictor row = response start)
    samples = {}
    i = 0
    while i < len(oi):
        b = int(oi[i] // R)
        j = i
        while j < len(oi) and oi[j] // R == b:
            j += 1
        n = j - i
        if n >= 2:
            rs = int(pred[i + 1])
        else:
            # single-token response: find the response segment whose prefix ends at pred row
            rs = next(r[0] for r in resp if r[1] == 1 and r[2] + r[3] - 1 == int(pred[i]) and r[0] not in samples.values())
        samples[b] = rs
        i = j
    for b in range(B):
        if b not in samples:
            continue
        q_start, q_len, p_start, p_len = by_start[samples[b]]
        idx_parts.append(np.concatenate([np.arange(p_start, p_start + p_len), np.arange(q_start, q_start + q_len)]))
        lens[b] = p_len + q_len
    idx = np.concatenate(idx_parts) if idx_parts else np.zeros(0, dtype=np.int64)
    return torch.from_numpy(idx.astype(np.int64)), lens


def reconstruct_sequences(dedup: torch.Tensor, pb: PackedBatch) -> Tuple[torch.Tensor, np.ndarray]:
    """``[T_dedup, ...]`` -> ``[sum_b (P_b + R_b), ...]`` packed per sample in original order; returns the tensor
    and the per-sample lengths."""
    idx, lens = _full_index(pb)
    return dedup.index_select(0, idx.to(dedup.device)), lens


def deduplicate_sequences(full: torch.Tensor, pb: PackedBatch, reduce: str = "sum") -> torch.Tensor:
    """Inverse of :func:`reconstruct_sequences`: rows that map to the same deduplicated row are summed
    (gradients) or the first one is taken (activations)."""
    idx, _ = _full_index(pb)
    idx = idx.to(full.device)
    out = full.new_zeros((pb.total_tokens, *full.shape[1:]))
    if reduce == "sum":
        return out.index_add_(0, idx, full)
    if reduce == "first":
        rev = torch.arange(idx.numel() - 1, -1, -1, device=full.device)
        out[idx[rev]] = full[rev]
        return out
    raise ValueError("reduce must be 'sum' or 'first'")


def extract_responses(dedup: torch.Tensor, pb: PackedBatch, offset: int = 0) -> torch.Tensor:
    """``offset=0``: each rollout's own response rows (the labels' positions); ``offset=-1``: the rows whose
    hidden states predict them (last prompt row, then the response rows but the last)."""
    if offset == -1:
        return dedup.index_select(0, pb.pred_index.to(dedup.device))
    if offset == 0:
        idx = pb.pred_index.clone()
        oi = pb.out_index
        R = pb.response_length
        first = torch.ones_like(oi, dtype=torch.bool)
        first[1:] = (oi[1:] // R) != (oi[:-1] // R)
        own = idx + 1
        # the first token of a response sits right after the previous response row, not after the prompt row:
        # recover it from the second predictor (which IS the first response row) when present
        nxt = torch.roll(idx, -1)
        has_next = ~torch.roll(first, -1)
        has_next[-1] = False
        own = torch.where(first & has_next, nxt, own)
        return dedup.index_select(0, own.to(dedup.device))
    raise ValueError("offset must be 0 or -1")


def pad_responses(values: torch.Tensor, pb: PackedBatch, fill: float = 0.0) -> torch.Tensor:
    """Per-token values in packed original-sample order -> ``[B, R, ...]`` grid."""
    B, R = pb.batch_size, pb.response_length
    out = values.new_full((B * R, *values.shape[1:]), fill)
    out[pb.out_index.to(values.device)] = values
    return out.view(B, R, *values.shape[1:])


def responses_in_orig_sample_order(values: torch.Tensor, pb: PackedBatch) -> List[torch.Tensor]:
    """Splits per-token values into one tensor per sample (original order; empty for samples without a response)."""
    counts = torch.bincount(torch.div(pb.out_index, pb.response_length, rounding_mode="floor"), minlength=pb.batch_size)
    return list(torch.split(values, counts.tolist()))


def get_group_token_layout(pb: PackedBatch) -> List[dict]:
    """Token layout of the deduplicated axis, group by group: ``{"group_idx", "sample_indices", "prompt_start",
    "prompt_tokens", "response_starts", "response_tokens"}``.  A group is one prompt segment followed by the
    response segments that attend to it; ``sample_indices`` are the original batch rows of those responses in the
    order they are laid out (arctic_platform/rl/zorro_train/zorro_train.py:2413-2436)."""
    segs = [tuple(int(v) for v in s[:4]) for s in pb.layout.segs.tolist()]
    members: dict = {}
    for b, g in enumerate(np.asarray(pb.group_of).tolist()):
        members.setdefault(int(g), []).append(b)
    out: List[dict] = []
    by_prompt_start: dict = {}
    for q_start, q_len, p_start, p_len in segs:
        if p_len == 0:                                   # a segment without a shared prefix opens a group
            by_prompt_start[q_start] = len(out)
            out.append({"group_idx": len(out), "sample_indices": [], "prompt_start": q_start, "prompt_tokens": q_len,
                        "response_starts": [], "response_tokens": []})
        else:
            g = out[by_prompt_start[p_start]]
            g["response_starts"].append(q_start)
            g["response_tokens"].append(q_len)
    for g in out:
        samples = members.get(g["group_idx"], [])
        # rows whose response is empty have no segment; the others appear in ascending batch order
        present = [b for b in samples if pb.sample_tokens[b] > g["prompt_tokens"]] if g["response_tokens"] else []
        g["sample_indices"] = present if len(present) == len(g["response_tokens"]) else samples[:len(g["response_tokens"])]
    return out


def split_deduplicated_hidden_by_group(dedup_hidden: torch.Tensor, pb: PackedBatch) -> List[dict]:
    """Per-group views of a ``[T_dedup, ...]`` tensor: ``{"group_idx", "sample_indices", "prompt_hidden",
    "response_hiddens"}`` -- what a recurrent (linear-attention) layer needs to run each prompt once and every
    response from the prompt's final state (arctic_platform/rl/zorro_train/zorro_train.py:2438-2464)."""
    if dedup_hidden.shape[0] != pb.total_tokens:
        raise ValueError(f"expected {pb.total_tokens} rows on the deduplicated axis, got {dedup_hidden.shape[0]}")
    groups, used = [], 0
    for g in get_group_token_layout(pb):
        ps, pl = g["prompt_start"], g["prompt_tokens"]
        resp = [dedup_hidden[s:s + n] for s, n in zip(g["response_starts"], g["response_tokens"])]
        groups.append({"group_idx": g["group_idx"], "sample_indices": g["sample_indices"],
                       "prompt_hidden": dedup_hidden[ps:ps + pl], "response_hiddens": resp})
        used += pl + sum(g["response_tokens"])
    if used != pb.total_tokens:
        raise AssertionError(f"group split covered {used} tokens, expected {pb.total_tokens}")
    return groups
