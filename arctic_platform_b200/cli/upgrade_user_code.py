"""Rewrites user trainer classes from the old class-attribute style to annotations.

    python -m arctic_platform_b200.cli.upgrade_user_code my_trainer.py [--check]

Older user code declared the pluggable parts of a trainer as assignments -- ``config_type = MyConfig``,
``data_factory_type = [A, B]`` -- where current code writes annotations: ``config: MyConfig``,
``data_factory: Union[A, B]``.  The tool rewrites the seven known attributes (``config``, ``data_factory``,
``model_factory``, ``checkpoint_engine``, ``optimizer_factory``, ``scheduler_factory``, ``tokenizer_factory``),
keeps indentation and everything else, and adds ``from typing import Union`` when a list became a union and the
import is missing.  ``--check`` only reports (exit 1 when the file would change).  Counterpart of
scripts/upgrade_user_code.py in the reference."""
from __future__ import annotations

import argparse
import re
import sys
from pathlib import Path
from typing import Tuple

ATTRIBUTES = ("config", "data_factory", "model_factory", "checkpoint_engine", "optimizer_factory",
              "scheduler_factory", "tokenizer_factory")
_NAME = r"[A-Za-z_][A-Za-z0-9_.]*"


def upgrade_source(text: str) -> Tuple[str, bool]:
    """Returns ``(new text, whether a Union was introduced)``."""
    used_union = False
    for attr in ATTRIBUTES:
        single = re.compile(rf"^(\s*){attr}_type\s*=\s*({_NAME})\s*$", re.M)
        text = single.sub(lambda m: f"{m.group(1)}{attr}: {m.group(2)}", text)
        many = re.compile(rf"^(\s*){attr}_type\s*=\s*\[\s*((?:{_NAME}\s*,\s*)*{_NAME})\s*,?\s*\]\s*$", re.M)

        def to_union(m):
            nonlocal used_union
            names = [n.strip() for n in m.group(2).split(",") if n.strip()]
            if len(names) == 1:
                return f"{m.group(1)}{attr}: {names[0]}"
            used_union = True
            return f"{m.group(1)}{attr}: Union[{', '.join(names)}]"

        text = many.sub(to_union, text)
    if used_union and not re.search(r"^\s*from typing import [^\n]*\bUnion\b", text, re.M) \
            and not re.search(r"^\s*import typing\b", text, re.M):
        lines = text.split("\n")
        at = 0
        # after a module docstring / __future__ imports / leading comments
        while at < len(lines) and (lines[at].startswith("#") or lines[at].startswith("from __future__")
                                   or not lines[at].strip()):
            at += 1
        lines.insert(at, "from typing import Union")
        text = "\n".join(lines)
    return text, used_union


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("file", type=Path)
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args(argv)
    if not args.file.is_file():
        print(f"{args.file}: no such file", file=sys.stderr)
        return 2
    old = args.file.read_text()
    new, _ = upgrade_source(old)
    if new == old:
        return 0
    if args.check:
        print(f"{args.file}: would be rewritten")
        return 1
    args.file.write_text(new)
    return 0


if __name__ == "__main__":
    sys.exit(main())
