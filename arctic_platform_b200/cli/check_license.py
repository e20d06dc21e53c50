"""Fails (exit 1) when a tracked source file lacks the SPDX license line.

    python -m arctic_platform_b200.cli.check_license [--fix] [paths...]

Checks ``*.py``, ``*.cu``, ``*.cuh``, ``*.cpp``, ``*.h``, ``*.sh`` under the given paths (default: the package
directory).  ``--fix`` prepends the line with the right comment prefix.  Counterpart of scripts/check_license.py in
the reference."""
from __future__ import annotations

import argparse
import sys
from pathlib import Path
from typing import List

SPDX = "SPDX-License-Identifier: Apache-2.0"
PREFIX = {".py": "# ", ".sh": "# ", ".cu": "// ", ".cuh": "// ", ".cpp": "// ", ".h": "// "}


def missing(paths: List[Path]) -> List[Path]:
    bad = []
    for root in paths:
        files = [root] if root.is_file() else [p for p in root.rglob("*") if p.suffix in PREFIX and "_C" not in p.parts]
        for f in files:
            head = f.read_text(errors="ignore")[:2048]
            if SPDX not in head and head.strip():
                bad.append(f)
    return bad


def fix(path: Path) -> None:
    text = path.read_text()
    line = PREFIX[path.suffix] + SPDX + "\n"
    if text.startswith("#!"):
        first, rest = text.split("\n", 1)
        path.write_text(first + "\n" + line + rest)
    else:
        path.write_text(line + text)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("paths", nargs="*", default=[str(Path(__file__).resolve().parents[1])])
    ap.add_argument("--fix", action="store_true")
    a = ap.parse_args(argv)
    bad = missing([Path(p) for p in a.paths])
    for f in bad:
        if a.fix:
            fix(f)
        else:
            print(f"missing license line: {f}")
    return 0 if (a.fix or not bad) else 1


if __name__ == "__main__":
    sys.exit(main())
