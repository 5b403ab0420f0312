"""Text environments and tools (offline: SQLite in memory, local corpus, subprocess python)."""
from skyrl_isoexec_b200 import gym
from skyrl_isoexec_b200.gym.envs import aime


def test_registered_environments():
    assert {"aime", "gsm8k", "lcb", "rlm", "search", "searchcode", "sql", "multiply", "even_tokens"} <= set(gym.registered_envs())


def test_aime_scoring():
    assert aime.compute_score("so the result is \\boxed{042}", "42") == 1.0
    assert aime.compute_score("... \\boxed{\\frac{1}{2}} then \\boxed{7}.", 7) == 1.0
    assert aime.compute_score("Answer: 1,234", "1234") == 1.0 and aime.compute_score("no answer", "3") == 0.0
    env = gym.make("aime", {}, {"reward_spec": {"ground_truth": "113"}})
    assert env.step("thus \\boxed{113}")["reward"] == 1.0 and env.step("\\boxed{114}")["reward"] == 0.0


def test_sql_env_multi_turn():
    schema = "create table t (id integer, name text, score real); insert into t values (1,'a',2.5),(2,'b',4.0),(3,'c',1.0);"
    ex = {"reward_spec": {"ground_truth": "select name from t where score > 2 order by name"}, "schema_sql": schema, "max_turns": 3}
    env = gym.make("sql", {}, ex)
    o = env.step("let me look <sql>select * from t</sql>")
    assert not o["done"] and "2.5" in o["observations"][0]["content"]
    o = env.step("<sql>selec nonsense</sql>")
    assert not o["done"] and "error" in o["observations"][0]["content"]
    o = env.step("<solution>select name from t where score >= 2.5</solution>")
    assert o["done"] and o["reward"] == 1.0
    env2 = gym.make("sql", {}, ex)
    assert env2.step("<solution>select name from t</solution>")["reward"] == 0.0
    env3 = gym.make("sql", {}, dict(ex, max_turns=1))
    assert env3.step("thinking...")["done"]


def test_search_env_and_bm25():
    corpus = ["The capital of France is Paris.", "Berlin is the capital of Germany.", "Bananas are rich in potassium."]
    env = gym.make("search", {"topk": 2}, {"reward_spec": {"ground_truth": ["Paris"]}, "corpus": corpus})
    o = env.step("<search>capital of France</search>")
    assert not o["done"] and o["observations"][0]["content"].startswith("<observation>Doc 1: The capital of France")
    assert env.step("<answer>the Paris.</answer>")["reward"] == 1.0
    env = gym.make("search", {}, {"reward_spec": {"ground_truth": "Paris"}, "corpus": corpus, "max_turns": 2})
    env.step("<search>zzz</search>")
    assert env.step("<search>qqq</search>")["done"]


def test_code_envs_run_tests_in_a_subprocess():
    tests = [{"input": "3 4\n", "output": "7"}, {"input": "10 -2\n", "output": "8"}]
    good = "```python\na, b = map(int, input().split())\nprint(a + b)\n```"
    bad = "```python\nprint(0)\n```"
    env = gym.make("lcb", {"timeout_s": 10}, {"reward_spec": {"ground_truth": tests}})
    assert env.step(good)["reward"] == 1.0 and env.step(bad)["reward"] == 0.0 and env.step("no code")["reward"] == 0.0
    loop = "```python\nwhile True: pass\n```"
    assert gym.make("lcb", {"timeout_s": 0.5}, {"reward_spec": {"ground_truth": tests}}).step(loop)["reward"] == 0.0
    sc = gym.make("searchcode", {}, {"reward_spec": {"ground_truth": "x", "tests": [{"assert": "assert add(2, 3) == 5"}]},
                                    "corpus": ["def add(a, b): return a + b  # adds two numbers"]})
    o = sc.step("<search>add two numbers</search>")
    assert "def add" in o["observations"][0]["content"]
    assert sc.step("```python\ndef add(a, b):\n    return a + b\n```")["reward"] == 1.0


def test_rlm_env_repl_over_a_long_context():
    lines = [f"row {i}: filler" for i in range(2000)]
    lines[1234] = "row 1234: the invoice total is 987.50 EUR"
    ctx = "\n".join(lines)
    mk = lambda **kw: gym.make("rlm", {}, {"context": ctx, "reward_spec": {"ground_truth": "987.50"}, "max_turns": 5, **kw})
    env = mk()
    prompt, info = env.init([{"role": "user", "content": "What is the invoice total?"}])
    assert prompt[0]["role"] == "system" and "length" in prompt[0]["content"] and info["context_len"] == len(ctx)
    assert ctx[:50] not in prompt[0]["content"]                       # the context itself is NOT in the prompt
    r = env.step("Let me look.\n```repl\nhits = [l for l in context.splitlines() if 'invoice' in l]\nprint(hits)\n```")
    assert not r["done"] and "987.50 EUR" in r["observations"][0]["content"]
    r = env.step("```repl\nprint(1/0)\n```")                          # an error is shown and not kept
    assert not r["done"] and "ZeroDivisionError" in r["observations"][0]["content"]
    r = env.step("```repl\ntotal = hits[0].split('is ')[1].split()[0]\nprint(SHOW_VARS())\n```")    # hits persists
    assert "'hits'" in r["observations"][0]["content"] and "'total'" in r["observations"][0]["content"]
    r = env.step("FINAL_VAR(total)")
    assert r["done"] and r["reward"] == 1.0 and r["metadata"]["how"] == "FINAL_VAR"
    assert env.get_metrics() == {"rlm/turns": 4, "rlm/blocks_run": 3, "rlm/block_errors": 1}
    # direct answers, wrong answers, the turn limit, a variable that does not exist
    assert mk().step("FINAL(987.50)")["reward"] == 1.0 and mk().step("FINAL(12)")["reward"] == 0.0
    assert mk(reward_spec={"ground_truth": "987.50", "match": "contains"}).step("FINAL(it is 987.50 EUR)")["reward"] == 1.0
    e = mk(max_turns=2)
    assert "FINAL_VAR failed" in e.step("FINAL_VAR(nope)")["observations"][0]["content"]
    out = e.step("no code here")
    assert out["done"] and out["reward"] == 0.0 and out["metadata"]["how"] == "turn limit"


def test_llm_judge_env_parses_scores_retries_and_counts_broken_replies():
    import http.server
    import json
    import threading

    import pytest

    from skyrl_isoexec_b200 import gym
    from skyrl_isoexec_b200.gym.envs.llm_judge import parse_judge_reply

    assert parse_judge_reply("thinking...\n### Final Score: 1") == 1.0 and parse_judge_reply("### Final Score: 0.0\n") == 0.0
    assert parse_judge_reply("1") == 1.0 and parse_judge_reply("maybe") is None
    assert parse_judge_reply("### Final Score: 0\nsecond thoughts\n### Final Score: 1") == 1.0      # the last verdict counts
    ex = {"reward_spec": {"ground_truth": "#### 42"}}
    with pytest.raises(ValueError):
        gym.make("llm_judge", {}, ex)
    with pytest.raises(ValueError):
        gym.make("llm_judge", {"judge_fn": lambda m: "1"}, {})
    seen = []

    def judge(messages):
        seen.append(messages[0]["content"])
        return "The numbers agree.\n### Final Score: 1" if "#### 42" in messages[0]["content"].split("PREDICTED SOLUTION:")[1] else "### Final Score: 0"

    env = gym.make("llm_judge", {"judge_fn": judge}, ex)
    out = env.step("so the answer is\n#### 42")
    assert out["reward"] == 1.0 and out["done"] and "GOLD SOLUTION:\n#### 42" in seen[0]
    assert gym.make("llm_judge", {"judge_fn": judge}, ex).step("#### 41")["reward"] == 0.0
    bad = gym.make("llm_judge", {"judge_fn": lambda m: "no idea"}, ex)
    assert bad.step("x")["reward"] == 0.0 and bad.get_metrics()["judge_unparsed"] == 1
    calls = []

    def flaky(messages):
        calls.append(1)
        if len(calls) < 3:
            raise ConnectionError("judge down")
        return "1"

    fl = gym.make("llm_judge", {"judge_fn": flaky, "retries": 2}, ex)
    assert fl.step("x")["reward"] == 1.0 and fl.get_metrics() == {"judge_calls": 3, "judge_unparsed": 0, "judge_errors": 2}

    class H(http.server.BaseHTTPRequestHandler):          # an OpenAI-compatible grader endpoint
        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            ok = self.path == "/v1/chat/completions" and body["messages"][0]["role"] == "user" and body["temperature"] == 0.0
            data = json.dumps({"choices": [{"message": {"role": "assistant", "content": f"### Final Score: {int(ok)}"}}]}).encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def log_message(self, *a):
            pass

    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        env = gym.make("llm_judge", {"base_url": f"http://127.0.0.1:{srv.server_address[1]}"}, ex)
        assert env.step("#### 42")["reward"] == 1.0
    finally:
        srv.shutdown()
