"""Token-budget micro-batching: first-fit-decreasing over sequence lengths (C++ runtime) with a minimum
number of groups and a divisor, and the split of a padded tensor dict into micro-batches whose count is
agreed across data-parallel ranks.  Contract of arctic_platform/rl/processors/microbatch.py:29-207."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ...ops import _lib

DEFAULT_MAX_TOKENS_PER_MB = 10240


@dataclass
class MicroBatchSpec:
    max_tokens_per_mb: int = DEFAULT_MAX_TOKENS_PER_MB
    n_mbs: int = 1                 # minimum number of micro-batches
    n_mbs_divisor: int = 1         # the count is rounded up to a multiple of this


@dataclass
class MicroBatchList:
    """What the split returns: the micro-batches with the bookkeeping to put per-row results back in input order.
    ``forward_indices[j]`` is the input row that sits at position ``j`` of the concatenated micro-batches,
    ``backward_indices`` its inverse (``concat(results)[backward_indices]`` is in input order), ``group_lens`` the
    token count of every micro-batch.  Unpacks as ``(mbs, groups)`` too."""
    data: dict
    mb_spec: MicroBatchSpec
    mbs: list
    group_lens: list
    forward_indices: Optional[list] = None
    backward_indices: Optional[list] = None
    groups: Optional[list] = None

    def __len__(self) -> int:
        return len(self.mbs)

    def __iter__(self):
        return iter((self.mbs, self.groups))

    def __getitem__(self, i):
        return (self.mbs, self.groups)[i]


def ffd_allocate(sizes, capacity: int, min_groups: int = 1, divisor: int = 1) -> List[List[int]]:
    """Groups of item indices; every group's total size is within ``capacity``.  Raises when an item alone
    exceeds the capacity.  Trailing empty groups appear when ``min_groups`` / ``divisor`` ask for more
    groups than the items fill."""
    arr = np.ascontiguousarray(np.asarray(sizes, dtype=np.int64))
    out = np.empty(max(len(arr), 1), dtype=np.int32)
    rt = _lib.rt_lib()
    n = rt.apb_rt_ffd_pack(arr.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)), len(arr), int(capacity),
                           int(min_groups), int(divisor), out.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)))
    if n < 0:
        raise ValueError(f"a sequence of {int(arr.max())} tokens exceeds max_tokens_per_mb={capacity}")
    groups: List[List[int]] = [[] for _ in range(n)]
    for i in range(len(arr)):
        groups[int(out[i])].append(i)
    return groups


def split_padded_tensor_dict_into_mb_list(batch: Dict[str, torch.Tensor], spec: MicroBatchSpec, group=None
                                          ) -> MicroBatchList:
    """Splits along dim 0 by token budget (``attention_mask`` row sums).  With a process group the number
    of micro-batches is raised to the maximum over ranks so every rank runs the same number of steps."""
    lens = batch["attention_mask"].sum(-1).tolist()
    groups = ffd_allocate(lens, spec.max_tokens_per_mb, spec.n_mbs, spec.n_mbs_divisor)
    if dist.is_initialized() and (group is not None or dist.get_world_size() > 1):
        counts = [None] * dist.get_world_size(group)
        dist.all_gather_object(counts, len(groups), group=group)
        want = max(counts)
        if want > len(groups):
            groups = ffd_allocate(lens, spec.max_tokens_per_mb, want, spec.n_mbs_divisor)
    groups = [g for g in groups if g] or [[]]
    mbs = []
    for g in groups:
        idx = torch.tensor(g, dtype=torch.long)
        mbs.append({k: (v[idx] if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == len(lens) else v)
                    for k, v in batch.items()})
    forward = [i for g in groups for i in g]
    backward = [0] * len(forward)
    for pos, row in enumerate(forward):
        backward[row] = pos
    return MicroBatchList(data=batch, mb_spec=spec, mbs=mbs, group_lens=[int(sum(lens[i] for i in g)) for g in groups],
                          forward_indices=forward, backward_indices=backward, groups=groups)
