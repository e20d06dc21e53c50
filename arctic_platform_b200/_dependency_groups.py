"""Optional dependency groups: which importable modules each feature needs, and an error that names the
missing group instead of a bare ImportError (arctic_platform/_dependency_groups.py:81-91 in the reference)."""
from __future__ import annotations

import importlib.util
from typing import Dict, Iterable, List

GROUPS: Dict[str, List[str]] = {
    "core": ["torch", "numpy", "pydantic"],
    "http": ["fastapi", "uvicorn", "requests"],
    "ray": ["ray"],
    "hf": ["transformers", "safetensors"],
    "testing": ["pytest"],
    # the reference's group names: what a training-only server, the full RL stack, the verl glue and development need
    "sft": ["torch", "numpy", "pydantic", "fastapi", "uvicorn", "requests", "safetensors"],
    "rl": ["torch", "numpy", "pydantic", "fastapi", "uvicorn", "requests", "safetensors", "pyarrow"],
    "verl": ["torch", "numpy", "pydantic", "omegaconf"],
    "dev": ["torch", "numpy", "pydantic", "pytest"],
}


def missing_modules(group: str) -> List[str]:
    if group not in GROUPS:
        raise KeyError(f"unknown dependency group {group!r} (known: {sorted(GROUPS)})")
    return [m for m in GROUPS[group] if importlib.util.find_spec(m) is None]


def group_available(group: str) -> bool:
    return not missing_modules(group)


def require_any_dep_group(*groups: str, feature: str = "this feature") -> str:
    """Returns the first fully installed group; raises ImportError listing what each group lacks."""
    if not groups:
        raise ValueError("name at least one dependency group")
    problems = []
    for g in groups:
        miss = missing_modules(g)
        if not miss:
            return g
        problems.append(f"[{g}] missing {', '.join(miss)}")
    raise ImportError(f"{feature} needs one of the dependency groups {list(groups)}: " + "; ".join(problems))
