"""Pre-fetches what a training recipe needs onto a node: its datasets or its model.

    python -m arctic_platform_b200.cli.fetch_assets --config recipe.yaml --what data  [--tmp-path /scratch/tmp]
    python -m arctic_platform_b200.cli.fetch_assets --config recipe.yaml --what model

The YAML is a training configuration with ``data.sources`` (each entry a dataset name / path, or a mapping
``{name_or_path, split, kwargs}``) and ``model.name_or_path``.  ``data`` loads every source once through
``datasets.load_dataset`` so that it lands in the local cache (temporary files go under ``--tmp-path``); ``model``
pulls the weights and the tokenizer through ``transformers``.  Run it on a machine with network access before a job
starts on nodes without one.  Counterpart of scripts/download_data.py in the reference."""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple


def data_sources(config: Dict[str, Any]) -> List[Tuple[str, Optional[str], Dict[str, Any]]]:
    """``(name_or_path, split, kwargs)`` of every entry of ``data.sources``."""
    out = []
    for src in (config.get("data") or {}).get("sources") or []:
        if isinstance(src, dict):
            if "name_or_path" not in src:
                raise ValueError(f"data source without name_or_path: {src}")
            out.append((str(src["name_or_path"]), src.get("split"), dict(src.get("kwargs") or {})))
        else:
            out.append((str(src), None, {}))
    return out


def fetch_data(config: Dict[str, Any], load: Optional[Callable[..., Any]] = None) -> int:
    if load is None:
        from datasets import load_dataset as load
    n = 0
    for name, split, kwargs in data_sources(config):
        print(f"dataset {name} split={split} {kwargs if kwargs else ''}".rstrip())
        load(path=name, split=split, **kwargs)
        n += 1
    return n


def fetch_model(config: Dict[str, Any], load_model: Optional[Callable[[str], Any]] = None,
                load_tokenizer: Optional[Callable[[str], Any]] = None) -> str:
    name = ((config.get("model") or {}).get("name_or_path") or "").strip()
    if not name:
        raise ValueError("the configuration names no model (model.name_or_path)")
    if load_model is None or load_tokenizer is None:
        from transformers import AutoModelForCausalLM, AutoTokenizer
        load_model = load_model or AutoModelForCausalLM.from_pretrained
        load_tokenizer = load_tokenizer or AutoTokenizer.from_pretrained
    print(f"model {name}")
    load_model(name)
    load_tokenizer(name)
    return name


def main(argv=None) -> int:
    import yaml
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("-c", "--config", type=Path, required=True)
    ap.add_argument("-w", "--what", choices=["data", "model"], required=True)
    ap.add_argument("-t", "--tmp-path", type=Path, default=Path(tempfile.gettempdir()))
    args = ap.parse_args(argv)
    config = yaml.safe_load(args.config.read_text()) or {}
    if args.what == "data":
        os.makedirs(args.tmp_path, exist_ok=True)
        tempfile.tempdir = str(args.tmp_path)
        fetch_data(config)
    else:
        fetch_model(config)
    return 0


if __name__ == "__main__":
    sys.exit(main())
