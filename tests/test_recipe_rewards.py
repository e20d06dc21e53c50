import sqlite3

from recipes.rl.rewards import bird_reward, extract_answer, extract_sql, f1_score, gsm8k_reward, long_context_qa_reward


def test_gsm8k_reward():
    assert extract_answer("so 3+4=7\n#### 7") == "7" and extract_answer("\\boxed{1,234.50}") == "1234.5"
    assert extract_answer("no marker 12") is None and extract_answer("no marker 12", "flexible") == "12"
    assert gsm8k_reward("The answer is $18.", "... #### 18") == 1.0
    assert gsm8k_reward("#### 17", "#### 18", format_score=0.1) == 0.1 and gsm8k_reward("eighteen", "#### 18") == 0.0


def test_bird_reward_execution_match():
    con = sqlite3.connect(":memory:")
    con.executescript("create table t(a int, b text); insert into t values (1,'x'),(2,'y'),(3,'x');")
    gold = "select a from t where b='x' order by a"
    assert extract_sql("think...\n```sql\nSELECT 1;\n```") == "SELECT 1"
    assert bird_reward("```sql\nselect a from t where b = 'x' order by a desc\n```", gold, "", connection=con) == 1.0
    assert bird_reward("<sql>select a from t</sql>", gold, "", connection=con) == 0.1
    assert bird_reward("```sql\nselect nope from t\n```", gold, "", connection=con) == 0.0
    assert bird_reward("no sql here", gold, "", connection=con) == 0.0


def test_long_context_qa_reward():
    assert long_context_qa_reward("... \\boxed{The Eiffel Tower}", ["Eiffel Tower"]) == 1.0
    assert 0.0 < long_context_qa_reward("Answer: tower in Paris", ["Eiffel Tower"]) < 1.0
    assert long_context_qa_reward("Answer: tower in Paris", ["Eiffel Tower"], em_only=True) == 0.0
    assert long_context_qa_reward("nothing", ["x"]) == 0.0 and abs(f1_score("x b c", "b c d") - 2 / 3) < 1e-9
