"""Token-set constraints on the action distribution (allow / deny lists per target position).

An environment may restrict which tokens are legal at some response positions (tool names, digits, a closed
answer set).  ``ActionMasks`` stores, in CSR form over the ``N`` prediction rows of a packed batch, a token list
per row and whether that list is the allowed set or a denied set; rows without an entry are unconstrained.

The masked log-probability and entropy are computed WITHOUT a masked ``[N, V]`` logits tensor: the fused lm-head
kernel gives the unmasked ``logprob`` and ``entropy`` per row, the logits of the (few) listed tokens come from a
gathered dot product, and the masked statistics follow exactly from

    S = sum_v e^z_v,  A = sum_v e^z_v z_v      (unmasked: lse = log S, entropy = lse - A/S)
    deny  list L:  S' = S - sum_L e^z,  A' = A - sum_L e^z z
    allow list L:  S' = sum_L e^z,      A' = sum_L e^z z

evaluated relative to ``lse`` so nothing overflows.  The reference applies ``-inf`` inside every vocabulary chunk
of its chunked lm-head (arctic_platform/model/implementations/qwen35/gpu/action_masks.py:14-262).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch


@dataclass
class ActionMasks:
    row_ptr: torch.Tensor    # [N+1] int64
    tokens: torch.Tensor     # [nnz] int64
    allow: torch.Tensor      # [N] bool: True = listed tokens are the only legal ones, False = listed tokens are illegal

    @property
    def num_rows(self) -> int:
        return self.row_ptr.numel() - 1

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_constraints(num_rows: int, constraints: Dict[int, Tuple[str, Iterable[int]]]) -> "ActionMasks":
        """``constraints[row] = ("allow" | "deny", token ids)``."""
        counts = torch.zeros(num_rows, dtype=torch.int64)
        allow = torch.zeros(num_rows, dtype=torch.bool)
        toks: List[int] = []
        for row in sorted(constraints):
            mode, ids = constraints[row]
            if mode not in ("allow", "deny"):
                raise ValueError(f"constraint mode must be 'allow' or 'deny', got {mode!r}")
            if not 0 <= row < num_rows:
                raise IndexError(f"constraint row {row} outside 0..{num_rows - 1}")
            ids = sorted(set(int(t) for t in ids))
            if mode == "allow" and not ids:
                raise ValueError(f"row {row}: an empty allow list leaves no legal token")
            counts[row] = len(ids)
            allow[row] = mode == "allow"
            toks.extend(ids)
        row_ptr = torch.zeros(num_rows + 1, dtype=torch.int64)
        row_ptr[1:] = counts.cumsum(0)
        return ActionMasks(row_ptr, torch.tensor(toks, dtype=torch.int64), allow)

    @staticmethod
    def from_grid(tokens: torch.Tensor, allow: torch.Tensor) -> "ActionMasks":
        """From the dense form a batch carries over the wire: ``tokens [N, K]`` int64 padded with ``-1`` and
        ``allow [N]`` with 1 = the listed tokens are the legal set, 0 = they are illegal, negative = no constraint
        on that row."""
        tokens = tokens.to("cpu", torch.int64)
        allow = allow.to("cpu", torch.int64)
        keep = (tokens >= 0) & (allow >= 0)[:, None]
        counts = keep.sum(1)
        if bool(((allow == 1) & (counts == 0)).any()):
            raise ValueError("an empty allow list leaves no legal token")
        row_ptr = torch.zeros(tokens.shape[0] + 1, dtype=torch.int64)
        row_ptr[1:] = counts.cumsum(0)
        srt = torch.where(keep, tokens, torch.full_like(tokens, torch.iinfo(torch.int64).max)).sort(1).values
        return ActionMasks(row_ptr, srt[srt != torch.iinfo(torch.int64).max], allow == 1)

    @staticmethod
    def pack(parts: Sequence["ActionMasks"]) -> "ActionMasks":
        """Concatenates the masks of several samples in the order their prediction rows are packed."""
        ptrs, off = [torch.zeros(1, dtype=torch.int64)], 0
        for p in parts:
            ptrs.append(p.row_ptr[1:] + off)
            off += int(p.row_ptr[-1])
        return ActionMasks(torch.cat(ptrs), torch.cat([p.tokens for p in parts]) if parts else torch.zeros(0, dtype=torch.int64),
                           torch.cat([p.allow for p in parts]) if parts else torch.zeros(0, dtype=torch.bool))

    def select(self, rows: torch.Tensor) -> "ActionMasks":
        """Masks of a subset of rows (index or boolean mask) -- the shard a sequence-parallel rank owns."""
        rows = rows.nonzero().squeeze(-1) if rows.dtype == torch.bool else rows
        rows = rows.to(self.row_ptr.device)
        lens = (self.row_ptr[1:] - self.row_ptr[:-1])[rows]
        ptr = torch.zeros(rows.numel() + 1, dtype=torch.int64, device=rows.device)
        ptr[1:] = lens.cumsum(0)
        idx = _expand(self.row_ptr[:-1][rows], lens)
        return ActionMasks(ptr, self.tokens[idx], self.allow[rows])

    def to(self, device) -> "ActionMasks":
        return ActionMasks(self.row_ptr.to(device), self.tokens.to(device), self.allow.to(device))

    # ------------------------------------------------------------------ queries
    def entry_rows(self) -> torch.Tensor:
        """Row of every CSR entry ``[nnz]``."""
        lens = self.row_ptr[1:] - self.row_ptr[:-1]
        return torch.repeat_interleave(torch.arange(self.num_rows, device=lens.device), lens)

    def dense_allowed(self, vocab: int) -> torch.Tensor:
        """``[N, V]`` bool -- tests and tiny vocabularies only."""
        N = self.num_rows
        listed = torch.zeros((N, vocab), dtype=torch.bool, device=self.tokens.device)
        listed[self.entry_rows(), self.tokens] = True
        has = (self.row_ptr[1:] - self.row_ptr[:-1]) > 0
        allowed = torch.where(self.allow[:, None], listed, ~listed)
        return torch.where(has[:, None] | self.allow[:, None], allowed, torch.ones_like(allowed))

    def is_allowed(self, tokens: torch.Tensor) -> torch.Tensor:
        """Whether ``tokens [N]`` (one per row) satisfy the constraints."""
        rows = self.entry_rows()
        hit = torch.zeros(self.num_rows, dtype=torch.bool, device=tokens.device)
        match = self.tokens.to(tokens.device) == tokens[rows.to(tokens.device)]
        hit.index_put_((rows.to(tokens.device)[match],), torch.ones(int(match.sum()), dtype=torch.bool, device=tokens.device))
        allow = self.allow.to(tokens.device)
        return torch.where(allow, hit, ~hit)

    def validate_sampled(self, tokens: torch.Tensor) -> None:
        ok = self.is_allowed(tokens)
        if not bool(ok.all()):
            bad = (~ok).nonzero().squeeze(-1)[:8].tolist()
            raise ValueError(f"sampled tokens violate the action masks at prediction rows {bad}")


def _expand(starts: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
    total = int(lens.sum())
    if total == 0:
        return torch.zeros(0, dtype=torch.int64, device=starts.device)
    seg = torch.repeat_interleave(torch.arange(lens.numel(), device=lens.device), lens)
    first = lens.cumsum(0) - lens
    return starts[seg] + torch.arange(total, device=lens.device) - first[seg]


def masked_logprobs(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, masks: Optional[ActionMasks],
                    inv_temperature=1.0, with_entropy: bool = True):
    """Log-probability of ``labels`` and entropy under the constrained distribution (differentiable).  A label that is
    itself illegal gets ``-inf``."""
    from ..ops.logprob import lm_head_logprobs
    lp, ent = lm_head_logprobs(hidden, weight, labels, inv_temperature, True)
    if masks is None or masks.tokens.numel() == 0:
        return lp, (ent if with_entropy else None)
    masks = masks.to(hidden.device)
    N = hidden.shape[0]
    rows = masks.entry_rows()
    it = inv_temperature[rows].float() if torch.is_tensor(inv_temperature) and inv_temperature.dim() > 0 \
        else float(inv_temperature)
    z = (hidden.index_select(0, rows).float() * weight.index_select(0, masks.tokens).float()).sum(-1) * it   # [nnz]
    it_lab = inv_temperature.float() if torch.is_tensor(inv_temperature) and inv_temperature.dim() > 0 \
        else float(inv_temperature)
    z_lab = (hidden.float() * weight.index_select(0, labels.long()).float()).sum(-1) * it_lab
    lse = z_lab - lp                                              # log S of the unmasked distribution
    f = torch.exp(z - lse[rows])                                  # e^z / S per listed token, in (0, 1]
    zero = torch.zeros(N, dtype=torch.float32, device=hidden.device)
    sum_f = zero.index_add(0, rows, f)
    sum_fz = zero.index_add(0, rows, f * z)
    has = (masks.row_ptr[1:] - masks.row_ptr[:-1]) > 0
    allow = masks.allow & has
    deny = (~masks.allow) & has
    a_over_s = lse - ent                                          # A / S
    s_ratio = torch.where(allow, sum_f, torch.where(deny, (1.0 - sum_f).clamp_min(1e-30), torch.ones_like(sum_f)))
    a_ratio = torch.where(allow, sum_fz, torch.where(deny, a_over_s - sum_fz, a_over_s))
    lse_m = lse + torch.log(s_ratio)
    lp_m = z_lab - lse_m
    legal = masks.is_allowed(labels.long())
    lp_m = torch.where(legal, lp_m, torch.full_like(lp_m, float("-inf")))
    ent_m = lse_m - a_ratio / s_ratio
    return lp_m, (ent_m if with_entropy else None)
