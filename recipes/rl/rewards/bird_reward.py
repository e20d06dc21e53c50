"""Text-to-SQL (BIRD) reward: execution match of the predicted query against the gold query on the sample's SQLite
database.  The SQL is taken from the last ```sql fenced block (or ``<sql>`` tag) of the completion.  Scores:
1.0 result sets equal (order-insensitive), ``format_score`` when SQL was found and ran but differs, 0 otherwise.
Queries run read-only with a time limit (a progress handler aborts long scans).  Counterpart of
recipes/rl/verl/txt2sql/bird_reward.py in the reference."""
from __future__ import annotations

import re
import sqlite3
import time
from typing import List, Optional, Tuple

_FENCE = re.compile(r"```(?:sql|sqlite)?\s*(.*?)```", re.S | re.I)
_TAG = re.compile(r"<sql>(.*?)</sql>", re.S | re.I)


def extract_sql(text: str) -> Optional[str]:
    for pat in (_FENCE, _TAG):
        m = pat.findall(text)
        if m:
            sql = m[-1].strip().rstrip(";").strip()
            if sql:
                return sql
    return None


def run_query(db_path: str, sql: str, timeout_s: float = 10.0) -> Tuple[bool, List[tuple]]:
    t0 = time.monotonic()
    con = sqlite3.connect(f"file:{db_path}?mode=ro", uri=True) if db_path != ":memory:" else sqlite3.connect(db_path)
    try:
        con.set_progress_handler(lambda: 1 if time.monotonic() - t0 > timeout_s else 0, 10000)
        return True, con.execute(sql).fetchall()
    except Exception:
        return False, []
    finally:
        con.close()


def bird_reward(completion: str, gold_sql: str, db_path: str, format_score: float = 0.1, timeout_s: float = 10.0,
                connection: Optional[sqlite3.Connection] = None) -> float:
    sql = extract_sql(completion)
    if sql is None:
        return 0.0
    if connection is not None:                                    # tests / in-memory databases
        try:
            got, want = connection.execute(sql).fetchall(), connection.execute(gold_sql).fetchall()
        except Exception:
            return 0.0
    else:
        ok, got = run_query(db_path, sql, timeout_s)
        ok2, want = run_query(db_path, gold_sql, timeout_s)
        if not ok or not ok2:
            return 0.0
    same = sorted(map(repr, got)) == sorted(map(repr, want))
    return 1.0 if same else format_score
