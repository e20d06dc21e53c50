"""Degrees of parallelism of one training job and the process groups derived from them.

``ParallelDims(dp_replicate, dp_shard, cp, pp, ep)`` lays the ranks out row-major as
``[pp, dp_replicate, dp_shard, cp]`` (``dp_shard = -1`` means "whatever is left").  Derived groups:

* ``dp``          -- dp_replicate x dp_shard      (data loading, loss normalisation)
* ``dp_shard_cp`` -- dp_shard x cp                (parameter / optimizer sharding)
* ``dp_cp``       -- dp_replicate x dp_shard x cp (gradient reduction of dense params)
* ``cp`` / ``sp`` -- context (Ulysses sequence) parallel group
* ``ep``          -- expert parallel: consecutive ranks inside ``dp_shard_cp``
* ``hsdp``        -- (dp_replicate, dp_shard_cp) pair when ``dp_replicate > 1``

``rank_groups(name)`` is pure arithmetic (tested without a process group); ``build_groups()`` creates the
``torch.distributed`` groups (every rank creates every group, as ``new_group`` requires).
Counterpart of arctic_platform/model/implementations/qwen35/parallel_dims.py:33-249.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np


@dataclass
class ParallelDims:
    dp_replicate: int = 1
    dp_shard: int = -1
    cp: int = 1
    pp: int = 1
    ep: int = 1
    world_size: int = 1
    _groups: Dict[str, object] = field(default_factory=dict, repr=False)

    def __post_init__(self):
        for name in ("dp_replicate", "cp", "pp", "ep"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1")
        rest = self.dp_replicate * self.cp * self.pp
        if self.dp_shard == -1:
            if self.world_size % rest:
                raise ValueError(f"world size {self.world_size} is not divisible by dp_replicate*cp*pp = {rest}")
            self.dp_shard = self.world_size // rest
        if self.dp_shard < 1:
            raise ValueError("dp_shard must be >= 1 or -1")
        if self.dp_replicate * self.dp_shard * self.cp * self.pp != self.world_size:
            raise ValueError(f"dp_replicate({self.dp_replicate}) * dp_shard({self.dp_shard}) * cp({self.cp}) * "
                             f"pp({self.pp}) != world size {self.world_size}")
        if (self.dp_shard * self.cp) % self.ep:
            raise ValueError(f"ep({self.ep}) must divide dp_shard*cp = {self.dp_shard * self.cp}")

    # ---------------------------------------------------------------- derived numbers
    @property
    def dp_enabled(self) -> bool:
        return self.dp_replicate * self.dp_shard > 1

    @property
    def cp_enabled(self) -> bool:
        return self.cp > 1

    @property
    def ep_enabled(self) -> bool:
        return self.ep > 1

    @property
    def pp_enabled(self) -> bool:
        return self.pp > 1

    @property
    def dp_size(self) -> int:
        return self.dp_replicate * self.dp_shard

    @property
    def non_data_parallel_size(self) -> int:
        return self.cp * self.pp

    @property
    def seq_len_divisor(self) -> int:
        """Sequence lengths must divide by this (2 x cp keeps causal load balance possible)."""
        return 2 * self.cp

    @property
    def fsdp_gradient_divide_factor(self) -> int:
        """Dense and expert gradients are both divided by the size of the full dp x cp domain."""
        return self.dp_replicate * self.dp_shard * self.cp

    # ---------------------------------------------------------------- rank arithmetic
    def _grid(self) -> np.ndarray:
        return np.arange(self.world_size).reshape(self.pp, self.dp_replicate, self.dp_shard, self.cp)

    def rank_groups(self, name: str) -> List[List[int]]:
        g = self._grid()
        pp, dr, ds, cp = g.shape
        if name == "pp":
            return g.reshape(pp, -1).T.tolist()
        if name == "dp_replicate":
            return g.transpose(0, 2, 3, 1).reshape(-1, dr).tolist()
        if name == "dp_shard":
            return g.transpose(0, 1, 3, 2).reshape(-1, ds).tolist()
        if name in ("cp", "sp"):
            return g.reshape(-1, cp).tolist()
        if name == "dp":
            return g.transpose(0, 3, 1, 2).reshape(-1, dr * ds).tolist()
        if name == "dp_shard_cp":
            return g.reshape(pp * dr, ds * cp).tolist()
        if name == "dp_cp":
            return g.reshape(pp, dr * ds * cp).tolist()
        if name == "ep":
            return g.reshape(-1, self.ep).tolist()
        raise KeyError(name)

    def group_of(self, name: str, rank: int) -> List[int]:
        for grp in self.rank_groups(name):
            if rank in grp:
                return grp
        raise ValueError(f"rank {rank} not in any {name} group")

    def coords(self, rank: int) -> Dict[str, int]:
        pp, dr, ds, cp = np.unravel_index(rank, self._grid().shape)
        return {"pp": int(pp), "dp_replicate": int(dr), "dp_shard": int(ds), "cp": int(cp),
                "dp": int(dr * self.dp_shard + ds), "ep": int((ds * self.cp + cp) % self.ep)}

    # ---------------------------------------------------------------- process groups
    GROUP_NAMES = ("pp", "dp_replicate", "dp_shard", "cp", "dp", "dp_shard_cp", "dp_cp", "ep")

    def build_groups(self, backend: Optional[str] = None) -> "ParallelDims":
        import torch.distributed as dist
        rank = dist.get_rank()
        for name in self.GROUP_NAMES:
            for ranks in self.rank_groups(name):
                grp = dist.new_group(ranks, backend=backend) if len(ranks) > 1 else None
                if rank in ranks:
                    self._groups[name] = grp
        self._groups["sp"] = self._groups.get("cp")
        return self

    def group(self, name: str):
        """Process group of this rank for ``name`` (None for a singleton group)."""
        if name not in self._groups:
            raise KeyError(f"group '{name}' not built; call build_groups() first")
        return self._groups[name]

    @property
    def hsdp(self):
        return (self.group("dp_replicate"), self.group("dp_shard_cp")) if self.dp_replicate > 1 else None
