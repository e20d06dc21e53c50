"""Builds the wheel of a tagged commit and (optionally) uploads it.

    python -m arctic_platform_b200.cli.release [--upload] [--dry-run]

Refuses to run unless the working tree is clean and HEAD carries a tag equal to ``v<version>`` of ``pyproject.toml``
-- the checks scripts/release.sh of the reference makes before ``python -m build`` and ``twine upload``.  The CUDA
library is compiled in-tree first so that the wheel carries ``_C/*.so``.  ``--dry-run`` prints the commands."""
from __future__ import annotations

import argparse
import subprocess
import sys
import tomllib
from pathlib import Path
from typing import List

ROOT = Path(__file__).resolve().parents[2]


def project_version(pyproject: Path = ROOT / "pyproject.toml") -> str:
    with open(pyproject, "rb") as f:
        return tomllib.load(f)["project"]["version"]


def release_commands(upload: bool) -> List[List[str]]:
    cmds = [[sys.executable, "-c", "import __graft_entry__ as g; g.build()"],
            [sys.executable, "-m", "build", "--wheel", "--no-isolation"]]
    if upload:
        cmds.append([sys.executable, "-m", "twine", "upload", "dist/*"])
    return cmds


def check_tree(version: str, run=subprocess.run) -> str:
    """'' when releasable, else the reason."""
    dirty = run(["git", "status", "--porcelain"], cwd=ROOT, capture_output=True, text=True).stdout.strip()
    if dirty:
        return "the working tree has uncommitted changes"
    tags = run(["git", "tag", "--points-at", "HEAD"], cwd=ROOT, capture_output=True, text=True).stdout.split()
    if f"v{version}" not in tags:
        return f"HEAD is not tagged v{version} (tags here: {tags or 'none'})"
    return ""


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--upload", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    version = project_version()
    why = check_tree(version)
    if why and not args.dry_run:
        print(f"not releasing {version}: {why}", file=sys.stderr)
        return 1
    for cmd in release_commands(args.upload):
        print(" ".join(cmd))
        if not args.dry_run:
            rc = subprocess.call(cmd, cwd=ROOT)
            if rc:
                return rc
    return 0


if __name__ == "__main__":
    sys.exit(main())
