"""Placement of colocated jobs on GPUs.

Pure placement arithmetic (usable and tested without Ray) plus thin Ray glue when Ray is importable.
Training, sampling and log-prob workers of a colocated deployment share each GPU through fractional
claims (0.34 / 0.33 / 0.33); bundles are laid out node by node, a global bundle index maps to
``(node placement group, local index)`` and a tensor-parallel group never straddles nodes.
Contract of arctic_platform/common/utils/ray_pg.py:54-224 in the reference.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

COLOCATE_FRACTIONS = {"training": 0.34, "sampling": 0.33, "log_prob": 0.33}
BUNDLE = {"GPU": 1, "CPU": 4}


@dataclass
class ColocatePlacement:
    gpus_per_node: List[int]                 # bundles (GPUs) in each node's placement group
    placement_groups: List[Any] = field(default_factory=list)   # Ray handles when created through Ray

    @property
    def total(self) -> int:
        return sum(self.gpus_per_node)

    def locate(self, bundle_idx: int) -> Tuple[int, int]:
        """Global bundle index -> ``(node index, index inside that node's group)``."""
        if bundle_idx < 0 or bundle_idx >= self.total:
            raise IndexError(f"bundle {bundle_idx} outside 0..{self.total - 1}")
        for node, n in enumerate(self.gpus_per_node):
            if bundle_idx < n:
                return node, bundle_idx
            bundle_idx -= n
        raise AssertionError("unreachable")

    def tp_layout(self, num_replicas: int, tp: int, bundle_offset: int = 0) -> List[List[int]]:
        """Global bundle indices of every replica's TP ranks; each replica sits on ONE node."""
        out: List[List[int]] = []
        node_start = 0
        cursor = bundle_offset
        for n in self.gpus_per_node:
            node_end = node_start + n
            cursor = max(cursor, node_start)
            while len(out) < num_replicas and cursor + tp <= node_end:
                out.append(list(range(cursor, cursor + tp)))
                cursor += tp
            node_start = node_end
        if len(out) < num_replicas:
            raise ValueError(f"cannot place {num_replicas} replicas of TP={tp} on nodes with {self.gpus_per_node} GPUs "
                             f"(offset {bundle_offset}) without splitting a replica across nodes")
        return out


def plan_colocate_placement(num_gpus: int, gpus_per_node: int) -> ColocatePlacement:
    """Fills nodes one by one: full nodes first, the remainder on the last node."""
    if num_gpus <= 0 or gpus_per_node <= 0:
        raise ValueError("num_gpus and gpus_per_node must be positive")
    full, rem = divmod(num_gpus, gpus_per_node)
    return ColocatePlacement([gpus_per_node] * full + ([rem] if rem else []))


def gpu_fraction(job_type: str, colocate: bool) -> float:
    return COLOCATE_FRACTIONS[job_type] if colocate else 1.0


def detect_gpus_per_node(default: int = 8) -> int:
    try:
        import ray
        if ray.is_initialized():
            per = [int(n["Resources"].get("GPU", 0)) for n in ray.nodes() if n.get("Alive")]
            per = [p for p in per if p > 0]
            if per:
                return min(per)
    except Exception:
        pass
    try:
        import torch
        if torch.cuda.is_available():
            return torch.cuda.device_count()
    except Exception:
        pass
    return default


def create_colocate_placement(num_gpus: int, gpus_per_node: Optional[int] = None) -> ColocatePlacement:
    """With Ray: one STRICT_PACK placement group per node with ``{GPU: 1, CPU: 4}`` bundles.  Without Ray:
    the plan only."""
    plan = plan_colocate_placement(num_gpus, gpus_per_node or detect_gpus_per_node())
    try:
        import ray
        from ray.util.placement_group import placement_group
    except Exception:
        return plan
    if not ray.is_initialized():
        return plan
    for n in plan.gpus_per_node:
        pg = placement_group([dict(BUNDLE) for _ in range(n)], strategy="STRICT_PACK")
        ray.get(pg.ready())
        plan.placement_groups.append(pg)
    return plan


def pg_scheduling_options(plan: ColocatePlacement, bundle_idx: int, job_type: str, colocate: bool) -> Dict[str, Any]:
    """Actor options (``num_gpus`` fraction and, under Ray, the placement-group strategy) for one worker."""
    node, local = plan.locate(bundle_idx)
    opts: Dict[str, Any] = {"num_gpus": gpu_fraction(job_type, colocate), "num_cpus": 1}
    if plan.placement_groups:
        from ray.util.scheduling_strategies import PlacementGroupSchedulingStrategy
        opts["scheduling_strategy"] = PlacementGroupSchedulingStrategy(
            placement_group=plan.placement_groups[node], placement_group_bundle_index=local)
    return opts
