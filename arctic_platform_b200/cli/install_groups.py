"""Installs the optional dependency groups of ``pyproject.toml`` by name.

    python -m arctic_platform_b200.cli.install_groups http hf [--pyproject PATH] [--dry-run]

A group may list another group of this project as ``arctic-platform-b200[other]`` (any spelling of the project name
with ``-`` / ``_``); such references are followed, cycles included, and every requirement is installed once.
``--dry-run`` prints the ``pip`` command instead of running it (there is no package index on an air-gapped machine).
Counterpart of scripts/install_deps.py in the reference."""
from __future__ import annotations

import argparse
import re
import subprocess
import sys
import tomllib
from pathlib import Path
from typing import Dict, Iterable, List

_SELF_REF = re.compile(r"^\s*([A-Za-z0-9_.\-]+)\s*\[([^\]]+)\]\s*$")


def load_groups(pyproject: Path) -> Dict[str, List[str]]:
    with open(pyproject, "rb") as f:
        doc = tomllib.load(f)
    project = doc.get("project", {})
    groups = {k: list(v) for k, v in project.get("optional-dependencies", {}).items()}
    groups["__project__"] = [project.get("name", "")]
    return groups


def _same_project(a: str, b: str) -> bool:
    norm = lambda s: re.sub(r"[-_.]+", "-", s).lower()
    return norm(a) == norm(b)


def resolve(names: Iterable[str], groups: Dict[str, List[str]]) -> List[str]:
    """Requirements of the named groups, references to this project's own groups expanded, sorted, no duplicates."""
    project = (groups.get("__project__") or [""])[0]
    known = sorted(k for k in groups if k != "__project__")
    out, seen, todo = set(), set(), list(names)
    while todo:
        g = todo.pop()
        if g in seen:
            continue
        if g not in groups or g == "__project__":
            raise ValueError(f"no optional dependency group {g!r}; groups: {', '.join(known)}")
        seen.add(g)
        for req in groups[g]:
            m = _SELF_REF.match(req)
            if m and project and _same_project(m.group(1), project):
                todo.extend(x.strip() for x in m.group(2).split(","))
            else:
                out.add(req.strip())
    return sorted(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("groups", nargs="+")
    ap.add_argument("--pyproject", type=Path, default=Path(__file__).resolve().parents[2] / "pyproject.toml")
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    reqs = resolve(args.groups, load_groups(args.pyproject))
    if not reqs:
        print("nothing to install")
        return 0
    cmd = [sys.executable, "-m", "pip", "install", *reqs]
    if args.dry_run:
        print(" ".join(cmd))
        return 0
    return subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
