"""Recipe pieces that run offline: BIRD preprocessing against a real SQLite file, the single-turn environments, and
the dataset-driven GRPO loop on the tiny preset."""
import json
import sqlite3

import pytest
import torch


def _make_db(root, db_id="shop"):
    d = root / db_id
    d.mkdir(parents=True)
    path = d / f"{db_id}.sqlite"
    conn = sqlite3.connect(path)
    conn.executescript("""
        CREATE TABLE customers (id INTEGER PRIMARY KEY, name TEXT, city TEXT);
        CREATE TABLE orders (id INTEGER PRIMARY KEY, customer_id INTEGER, total REAL,
                             FOREIGN KEY (customer_id) REFERENCES customers(id));
        INSERT INTO customers VALUES (1, 'Ann', 'Oslo'), (2, 'Bob', 'Rome'), (3, 'Cy', 'Oslo');
        INSERT INTO orders VALUES (1, 1, 10.0), (2, 1, 5.5), (3, 2, 7.0);
    """)
    conn.commit()
    conn.close()
    return path


def test_preprocess_bird_writes_verl_rows(tmp_path):
    from recipes.rl.verl.txt2sql import preprocess_bird as pb
    db = _make_db(tmp_path / "dbs")
    ddl = pb.schema_ddl(str(db))
    assert "CREATE TABLE customers" in ddl and "-- customers.city examples: Oslo, Rome" in ddl
    assert "-- foreign keys: orders.customer_id -> customers.id" in ddl
    qs = [{"db_id": "shop", "question": "How many customers live in Oslo?", "evidence": "city = 'Oslo'",
           "SQL": "SELECT COUNT(*) FROM customers WHERE city = 'Oslo'", "difficulty": "simple"},
          {"db_id": "shop", "question": "Total per customer?", "query": "SELECT customer_id, SUM(total) FROM orders GROUP BY 1"},
          {"db_id": "missing", "question": "?", "SQL": "SELECT 1"},
          {"db_id": "shop", "question": "no gold"}]
    qf = tmp_path / "train.json"
    qf.write_text(json.dumps(qs))
    assert pb.main(["--train-questions", str(qf), "--train-db-root", str(tmp_path / "dbs"), "--output-dir", str(tmp_path / "out")]) == 0
    assert pb.process.last_dropped == {"missing_db": 1, "missing_sql": 1}
    import pyarrow.parquet as pq
    rows = pq.read_table(tmp_path / "out" / "train.parquet").to_pylist()
    assert len(rows) == 2 and rows[0]["data_source"] == "bird" and rows[0]["prompt"][0]["role"] == "system"
    assert "Hint: city = 'Oslo'" in rows[0]["prompt"][1]["content"] and "Hint" not in rows[1]["prompt"][1]["content"]
    assert rows[0]["reward_model"] == {"style": "rule", "ground_truth": qs[0]["SQL"]}
    assert rows[1]["extra_info"]["db_path"].endswith("shop.sqlite") and rows[1]["extra_info"]["index"] == 1
    short = pb.process(str(qf), str(tmp_path / "dbs"), max_prompt_chars=50)
    assert short == [] and pb.process.last_dropped["too_long"] == 2


def test_single_turn_environments(tmp_path):
    from recipes.rl.skyrl import envs
    db = _make_db(tmp_path / "dbs")
    bird = envs.make("bird_sql_arctic", {"reward_model": {"ground_truth": "SELECT COUNT(*) FROM customers WHERE city='Oslo'"},
                                         "extra_info": {"db_path": str(db)}})
    good = bird.step("<think>count</think>\n```sql\nSELECT COUNT(id) FROM customers WHERE city = 'Oslo'\n```")
    bad = bird.step("```sql\nSELECT COUNT(*) FROM customers\n```")
    assert good.done and good.observations == [] and good.reward > bad.reward >= 0
    with pytest.raises(ValueError):
        envs.make("bird_sql_arctic", {"reward_spec": {"ground_truth": "SELECT 1"}}).step("```sql\nSELECT 1\n```")
    gsm = envs.make("gsm8k_arctic", {"reward_spec": {"ground_truth": "72"}})
    assert gsm.step("so the answer is #### 72").reward > gsm.step("#### 71").reward
    qa = envs.make("long_context_qa", {"reward_model": {"ground_truth": ["Marie Curie", "Curie"]}, "data_source": "loong"})
    assert qa.data_source == "loong" and qa.step(r"<think>..</think> \boxed{Marie Curie}").reward == 1.0
    assert qa.step("no box here").reward == 0.0
    with pytest.raises(ValueError):
        envs.make("long_context_qa", {"extra_info": {}})
    with pytest.raises(KeyError):
        envs.make("nope", {})
    assert envs.register_envs() == [] or envs.HAVE_SKYRL_GYM


def test_dataset_loop_runs_on_the_tiny_preset(tmp_path):
    from recipes.rl.skyrl import run_loop
    rows = [{"prompt": [{"role": "user", "content": f"What is {a}+{a}?"}], "reward_model": {"ground_truth": str(2 * a)}}
            for a in range(1, 7)]
    data = tmp_path / "p.jsonl"
    data.write_text("\n".join(json.dumps(r) for r in rows))
    assert run_loop.read_rows(str(data)) == rows
    import pyarrow as pa
    import pyarrow.parquet as pq
    pq.write_table(pa.Table.from_pylist(rows), tmp_path / "p.parquet")
    assert run_loop.read_rows(str(tmp_path / "p.parquet")) == rows
    assert [len(b) for b in run_loop.batches(rows, 2, 1)] == [2, 2, 2]
    assert [b[0]["reward_model"]["ground_truth"] for b in run_loop.batches(rows, 1, 1, rank=1, world=2)] == ["4", "8", "12"]
    adv = run_loop.grpo_advantages(torch.tensor([1.0, 0.0, 1.0, 1.0]), 2)
    assert adv[0] > 0 > adv[1] and adv[2] == adv[3] == 0
    codec = run_loop.ByteCodec(512)
    assert codec.decode(codec.encode("a+b=3")) == "a+b=3"
    args = run_loop.build_parser().parse_args(["--data", str(data), "--env", "gsm8k_arctic", "--model", "qwen3-tiny",
                                               "--batch-prompts", "2", "--n", "2", "--max-tokens", "4", "--max-steps", "2",
                                               "--max-prompt-tokens", "64", "--zero-stage", "1", "--lr", "1e-4"])
    logs = []
    hist = run_loop.run(args, log=logs.append)
    assert len(hist) == 2 and len(logs) == 2 and all(h["grad_norm"] >= 0 for h in hist)
    assert json.loads(logs[0])["step"] == 0


def test_entrypoint_runs_in_process_and_reattaches(tmp_path, capsys):
    from arctic_platform_b200.common.ray_server import create_arctic_rl_ray_server_state
    from recipes.rl.skyrl import entrypoint
    rows = [{"prompt": [{"role": "user", "content": f"What is {a}+{a}?"}], "reward_model": {"ground_truth": str(2 * a)}}
            for a in range(1, 5)]
    data = tmp_path / "p.jsonl"
    data.write_text("\n".join(json.dumps(r) for r in rows))
    argv = ["--data", str(data), "--env", "gsm8k_arctic", "--model", "qwen3-tiny", "--batch-prompts", "2", "--n", "2",
            "--max-tokens", "4", "--max-steps", "1", "--max-prompt-tokens", "64", "--zero-stage", "1", "--log-prob-gpus", "0",
            "--kl-loss-coef", "0"]
    assert entrypoint.main(argv) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["step"] == 0
    # a server state handed in by the caller hosts the engines; the loop leaves them to their owner
    state = create_arctic_rl_ray_server_state(colocate=True)
    hist = entrypoint.skyrl_entrypoint(argv, server_state=state)
    assert len(hist) == 1 and len(state.get_jobs()) == 2
    state.destroy()
    assert entrypoint.main(["--as-ray-task"] + argv) == 2                    # no Ray on this machine: says so, no traceback
    import recipes.rl.skyrl.sitecustomize  # noqa: F401  (importable, and harmless without skyrl_gym)
