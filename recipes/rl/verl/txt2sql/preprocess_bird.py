"""Text-to-SQL training data -> verl-format parquet.

Input: a BIRD- or Spider-style question file (a JSON list of ``{"db_id", "question", "evidence"?, "SQL" | "query",
"difficulty"?}``) and the directory of SQLite databases (``<db_root>/<db_id>/<db_id>.sqlite``).  For every question
the prompt holds the database schema as ``CREATE TABLE`` statements -- read from the database itself, with a few
sample values per column and the foreign keys spelled out -- plus the question (and the evidence hint when there is
one); the gold SQL is the reward's ground truth.  Rows whose prompt is longer than ``--max-prompt-chars`` are
dropped and counted.

Output rows (one per question)::

    {"data_source": "bird", "prompt": [{"role": "system", ...}, {"role": "user", ...}], "ability": "text2sql",
     "reward_model": {"style": "rule", "ground_truth": <gold sql>},
     "extra_info": {"db_id", "db_path", "question", "difficulty", "index", "split"}}

Same role as recipes/rl/verl/txt2sql/preprocess_bird.py of the reference (which also merges two more corpora)."""
from __future__ import annotations

import argparse
import json
import os
import re
import sqlite3
from collections import Counter
from typing import Dict, List, Optional

SYSTEM_PROMPT = ("You are a data analyst who writes {engine} SQL. Think step by step inside <think> ... </think>, then "
                 "give the final query inside a ```sql ... ``` block.")


def _short(v, max_len: int = 60) -> str:
    s = " ".join(str(v).split())
    return s if len(s) <= max_len else s[:max_len - 3] + "..."


def foreign_keys(conn: sqlite3.Connection, table: str) -> List[str]:
    out = []
    for row in conn.execute(f'PRAGMA foreign_key_list("{table}")'):
        _id, _seq, ref_table, col, ref_col = row[0], row[1], row[2], row[3], row[4]
        out.append(f"{table}.{col} -> {ref_table}.{ref_col or col}")
    return out


def schema_ddl(db_path: str, samples_per_column: int = 3, max_tables: Optional[int] = None) -> str:
    """``CREATE TABLE`` statements of every user table, each followed by comment lines with example values per
    column and the foreign keys.  Read-only connection; nothing is executed but catalogue queries and ``LIMIT``ed
    selects."""
    conn = sqlite3.connect(f"file:{db_path}?mode=ro", uri=True)
    try:
        tables = conn.execute("SELECT name, sql FROM sqlite_master WHERE type='table' AND name NOT LIKE 'sqlite_%' "
                              "ORDER BY name").fetchall()
        parts = []
        for name, sql in tables[:max_tables]:
            block = [re.sub(r"[ \t]+", " ", (sql or f"CREATE TABLE {name} ()").strip()) + ";"]
            if samples_per_column > 0:
                cols = [r[1] for r in conn.execute(f'PRAGMA table_info("{name}")')]
                for c in cols:
                    try:
                        vals = [r[0] for r in conn.execute(
                            f'SELECT DISTINCT "{c}" FROM "{name}" WHERE "{c}" IS NOT NULL LIMIT {int(samples_per_column)}')]
                    except sqlite3.Error:
                        vals = []
                    if vals:
                        block.append(f"-- {name}.{c} examples: " + ", ".join(_short(v) for v in vals))
            fks = foreign_keys(conn, name)
            if fks:
                block.append("-- foreign keys: " + "; ".join(fks))
            parts.append("\n".join(block))
        return "\n\n".join(parts)
    finally:
        conn.close()


def build_messages(ddl: str, question: str, evidence: str = "", engine: str = "SQLite") -> List[Dict[str, str]]:
    user = f"Database schema:\n{ddl}\n\nQuestion: {question.strip()}"
    if evidence and evidence.strip():
        user += f"\nHint: {evidence.strip()}"
    return [{"role": "system", "content": SYSTEM_PROMPT.format(engine=engine)}, {"role": "user", "content": user}]


def process(questions_file: str, db_root: str, data_source: str = "bird", split: str = "train",
            samples_per_column: int = 3, max_prompt_chars: Optional[int] = None) -> List[dict]:
    with open(questions_file, encoding="utf-8") as f:
        items = json.load(f)
    cache: Dict[str, str] = {}
    rows, dropped = [], Counter()
    for i, it in enumerate(items):
        db_id = it["db_id"]
        db_path = os.path.join(db_root, db_id, f"{db_id}.sqlite")
        if not os.path.isfile(db_path):
            dropped["missing_db"] += 1
            continue
        if db_id not in cache:
            cache[db_id] = schema_ddl(db_path, samples_per_column)
        gold = (it.get("SQL") or it.get("query") or "").strip()
        if not gold:
            dropped["missing_sql"] += 1
            continue
        msgs = build_messages(cache[db_id], it["question"], it.get("evidence", ""))
        if max_prompt_chars and sum(len(m["content"]) for m in msgs) > max_prompt_chars:
            dropped["too_long"] += 1
            continue
        rows.append({"data_source": data_source, "prompt": msgs, "ability": "text2sql",
                     "reward_model": {"style": "rule", "ground_truth": gold},
                     "extra_info": {"db_id": db_id, "db_path": db_path, "question": it["question"],
                                    "difficulty": it.get("difficulty", "unknown"), "index": i, "split": split}})
    process.last_dropped = dict(dropped)
    return rows


def write_parquet(rows: List[dict], path: str) -> None:
    import pyarrow as pa
    import pyarrow.parquet as pq
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    pq.write_table(pa.Table.from_pylist(rows), path)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--train-questions")
    ap.add_argument("--train-db-root")
    ap.add_argument("--val-questions")
    ap.add_argument("--val-db-root")
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--data-source", default="bird")
    ap.add_argument("--samples-per-column", type=int, default=3)
    ap.add_argument("--max-prompt-chars", type=int, default=None)
    args = ap.parse_args(argv)
    for split, qf, root in (("train", args.train_questions, args.train_db_root), ("val", args.val_questions, args.val_db_root)):
        if not qf:
            continue
        rows = process(qf, root, args.data_source, split, args.samples_per_column, args.max_prompt_chars)
        out = os.path.join(args.output_dir, f"{split}.parquet")
        write_parquet(rows, out)
        print(f"{split}: {len(rows)} rows -> {out}; dropped {process.last_dropped}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
