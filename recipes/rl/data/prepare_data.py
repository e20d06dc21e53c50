"""Fetches the recipe datasets and writes them in the row format verl and the SkyRL-style loop read.

    python -m recipes.rl.data.prepare_data gsm8k            --output-dir ~/data/gsm8k
    python -m recipes.rl.data.prepare_data long_context_qa  --output-dir ~/data/long-context [--test-ratio 0.05]

Every output row has ``data_source``, ``prompt`` (chat messages), ``ability``, ``reward_model = {style: rule,
ground_truth}`` and ``extra_info``; files are ``train.parquet`` / ``test.parquet`` (pandas + pyarrow).  Needs network
access and the ``datasets`` package for the download itself; everything after the download is plain Python (the
loaders can be replaced, which is how the tests run it).  BIRD / Spider come as local files with SQLite databases
and are converted by ``recipes/rl/verl/txt2sql/preprocess_bird.py``.  Counterparts of the per-recipe
``download_data.py`` scripts of the reference (recipes/rl/verl/simple, recipes/rl/verl/long_context_qa,
recipes/rl/skyrl/*).
"""
from __future__ import annotations

import argparse
import os
import random
import re
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

GSM8K_SOURCE = "openai/gsm8k"
GSM8K_SUFFIX = 'Let\'s think step by step and output the final answer after "####".'

LOONGRL_REPO = "OldKingMeister/LoongRL-Train-Data"
LOONGRL_TASKS = {
    "hotpotqa": ("hotpotqa_qwen_0_2500", "hotpotqa_distractor_2500_5000"),
    "musique": ("musique_qwen_0_2500", "musique_distractor_2500_5000"),
    "2wikimqa": ("2wikipedia_qwen_0_2500", "2wikipedia_distractor_2500_5000"),
}
BOXED_SYSTEM_PROMPT = ("A conversation between User and Assistant. The User asks a question, and the Assistant solves it. "
                       "The Assistant first thinks about the reasoning process in the mind and then provides the User with "
                       "the answer. The reasoning process is enclosed within <think> </think> and answer is enclosed within "
                       "\\boxed{} tags, respectively, i.e., <think> reasoning process here </think> \\boxed{answer here}.")
ROW_KEYS = ("data_source", "prompt", "ability", "reward_model", "extra_info")


def gsm8k_final_answer(solution: str) -> str:
    """The number after ``####`` in a GSM8K solution, thousands separators removed."""
    m = re.search(r"####\s*(-?[0-9][0-9.,]*)", solution)
    if m is None:
        raise ValueError(f"no '#### <answer>' in {solution[:80]!r}")
    return m.group(1).replace(",", "").rstrip(".")


def gsm8k_row(example: Dict[str, Any], index: int, split: str) -> Dict[str, Any]:
    q, a = example["question"], example["answer"]
    return {"data_source": GSM8K_SOURCE, "prompt": [{"role": "user", "content": f"{q} {GSM8K_SUFFIX}"}],
            "ability": "math", "reward_model": {"style": "rule", "ground_truth": gsm8k_final_answer(a)},
            "extra_info": {"split": split, "index": index, "question": q, "answer": a}}


def long_context_row(example: Dict[str, Any]) -> Dict[str, Any]:
    """Keeps the five standard keys and puts the boxed-answer system prompt in front of the conversation."""
    row = {k: example[k] for k in ROW_KEYS if k in example}
    msgs = [dict(m) for m in row.get("prompt", [])]
    if not msgs or msgs[0].get("role") != "system":
        msgs.insert(0, {"role": "system", "content": BOXED_SYSTEM_PROMPT})
    row["prompt"] = msgs
    return row


def split_rows(rows: List[Dict[str, Any]], test_ratio: float, seed: int) -> Tuple[List[dict], List[dict]]:
    order = list(range(len(rows)))
    random.Random(seed).shuffle(order)
    n_test = int(round(len(rows) * test_ratio))
    test = [rows[i] for i in order[:n_test]]
    train = [rows[i] for i in order[n_test:]]
    return train, test


def write_parquet(rows: List[Dict[str, Any]], path: str) -> str:
    import pandas as pd
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    pd.DataFrame(rows, columns=[k for k in ROW_KEYS if any(k in r for r in rows)] or list(ROW_KEYS)).to_parquet(path)
    return path


def _hf_loader() -> Callable[..., Iterable[Dict[str, Any]]]:
    from datasets import load_dataset
    return lambda repo, name, split: load_dataset(repo, name, split=split)


def prepare_gsm8k(output_dir: str, load: Optional[Callable] = None) -> Dict[str, int]:
    load = load or _hf_loader()
    out = {}
    for split in ("train", "test"):
        rows = [gsm8k_row(ex, i, split) for i, ex in enumerate(load(GSM8K_SOURCE, "main", split))]
        write_parquet(rows, os.path.join(os.path.expanduser(output_dir), f"{split}.parquet"))
        out[split] = len(rows)
    return out


def prepare_long_context_qa(output_dir: str, test_ratio: float = 0.05, seed: int = 42,
                            load: Optional[Callable] = None) -> Dict[str, Dict[str, int]]:
    """One directory per task (both subsets merged, then split) plus ``merged/`` over all tasks."""
    load = load or _hf_loader()
    root = os.path.expanduser(output_dir)
    all_train: List[dict] = []
    all_test: List[dict] = []
    out: Dict[str, Dict[str, int]] = {}
    for task, subsets in LOONGRL_TASKS.items():
        rows = [long_context_row(ex) for name in subsets for ex in load(LOONGRL_REPO, name, "train")]
        train, test = split_rows(rows, test_ratio, seed)
        write_parquet(train, os.path.join(root, task, "train.parquet"))
        write_parquet(test, os.path.join(root, task, "test.parquet"))
        out[task] = {"train": len(train), "test": len(test)}
        all_train += train
        all_test += test
    write_parquet(all_train, os.path.join(root, "merged", "train.parquet"))
    write_parquet(all_test, os.path.join(root, "merged", "test.parquet"))
    out["merged"] = {"train": len(all_train), "test": len(all_test)}
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("dataset", choices=["gsm8k", "long_context_qa"])
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--test-ratio", type=float, default=0.05)
    ap.add_argument("--seed", type=int, default=42)
    args = ap.parse_args(argv)
    res = prepare_gsm8k(args.output_dir) if args.dataset == "gsm8k" else \
        prepare_long_context_qa(args.output_dir, args.test_ratio, args.seed)
    print(res)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
