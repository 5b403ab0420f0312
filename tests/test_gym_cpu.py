"""Text environments and tools (offline: SQLite in memory, local corpus, subprocess python)."""
from skyrl_isoexec_b200 import gym
from skyrl_isoexec_b200.gym.envs import aime


def test_registered_environments():
    assert {"aime", "gsm8k", "gsm8k_multi_turn", "lcb", "rlm", "search", "searchcode", "sql", "multiply", "even_tokens", "visual_count"} \
        <= set(gym.registered_envs())


def test_aime_scoring():
    assert aime.compute_score("so the result is \\boxed{042}", "42") == 1.0
    assert aime.compute_score("... \\boxed{\\frac{1}{2}} then \\boxed{7}.", 7) == 1.0
    assert aime.compute_score("Answer: 1,234", "1234") == 1.0 and aime.compute_score("no answer", "3") == 0.0
    # the Minerva normalisation: units, wrappers, shorthand fractions and roots, what stands left of '=', signs and zeros
    for text, gold in (("Answer: $x = 5$ dollars", "5"), ("Answer: \\frac12", "\\frac{1}{2}"), ("Answer: \\text{12 cm}", "12"),
                       ("\\boxed{3.0}", "3"), ("\\boxed{90^\\circ}", "90"), ("Answer: \\sqrt2", "\\sqrt{2}"), ("\\boxed{-007}", "-7"),
                       ("Answer: 10\\%", "10"), ("\\boxed{\\textbf{(B)}}", "(B)")):
        assert aime.compute_score(text, gold) == 1.0, text
    assert aime.compute_score("\\boxed{12}", "13") == 0.0 and aime.compute_score("\\boxed{12}", "13", wrong_reward=-1.0) == -1.0
    # modes: an Answer line near the end only; a boxed string compared as it stands
    assert aime.score_info("x" * 400 + "Answer: 5", "5", "minerva")["acc"] and not aime.score_info("Answer: 5" + "x" * 400, "5", "minerva")["acc"]
    assert not aime.score_info("\\boxed{05}", "5", "strict_box")["acc"] and aime.score_info("\\boxed{5}", "5", "strict_box")["acc"]
    env = gym.make("aime", {}, {"reward_spec": {"ground_truth": "113"}})
    out = env.step("thus \\boxed{113}")
    assert out["reward"] == 1.0 and out["metadata"] == {"acc": True, "pred": "113"} and env.get_metrics() == {"acc": 1.0}
    assert env.step("\\boxed{114}")["reward"] == -1.0                                  # the reference's value for a wrong answer
    assert gym.make("aime", {"wrong_reward": 0.0}, {"reward_model": {"ground_truth": "113"}}).step("\\boxed{114}")["reward"] == 0.0


def test_gsm8k_multi_turn_rewards_every_turn():
    mk = lambda **kw: gym.make("gsm8k_multi_turn", {}, {"reward_spec": {"ground_truth": "72"}, **kw})
    env = mk(max_turns=3)
    o = env.step("I think #### 70")
    assert not o["done"] and abs(o["reward"] - 0.2 / 3) < 1e-9 and "tentative numeric answer" in o["observations"][0]["content"]
    o = env.step("no number here")
    assert not o["done"] and o["reward"] == 0.0 and "only the final numeric answer" in o["observations"][0]["content"]
    o = env.step("#### 72")
    assert o["done"] and o["reward"] == 1.0 and env.get_metrics() == {"steps": 3, "solved": 1.0}
    env = mk(extra_info={"max_turns": 2})
    assert env.step("#### 72")["done"] and env.max_turns == 2
    e = mk(max_turns=1)
    assert e.step("#### 1")["done"]
    agg = type(e).aggregate_metrics([{"steps": 1, "solved": 0.0}, {"steps": 3, "solved": 1.0}])
    assert agg == {"avg_steps": 2.0, "solved": 0.5}


def test_sql_env_format_rules_result_sets_and_probe_isolation(tmp_path):
    from skyrl_isoexec_b200.gym.envs import sql as S

    schema = "create table t (id integer, name text, score real); insert into t values (1,'a',2.5),(2,'b',4.0),(3,'c',1.0);"
    ex = {"reward_spec": {"ground_truth": "select name from t where score > 2 order by name"}, "schema_sql": schema, "max_turns": 4}
    env = gym.make("sql", {}, ex)
    o = env.step("<think>let me look</think><sql>select * from t</sql>")
    text = o["observations"][0]["content"]
    assert not o["done"] and "2.5" in text and text.strip().startswith("<observation>") and "You have 3 turns left" in text
    o = env.step("<think>hm</think><sql>selec nonsense</sql>")
    assert not o["done"] and "Error executing SQL" in o["observations"][0]["content"]
    o = env.step("<think>try to break it</think><sql>delete from t</sql>")            # a probe is rolled back
    assert not o["done"]
    o = env.step("<think>now</think><solution>select name from t where score >= 2.5</solution>")
    assert o["done"] and o["reward"] == 1.0 and env.get_metrics() == {"turns": 4, "queries": 3, "query_errors": 1}
    env.close()
    # rows are compared as a set: order and duplicates do not matter, other rows do
    mk = lambda **kw: gym.make("sql", {}, dict(ex, **kw))
    assert mk().step("<think>x</think><solution>select name from t where score > 2 order by name desc</solution>")["reward"] == 1.0
    assert mk().step("<think>x</think><solution>select name from t</solution>")["reward"] == 0.0
    assert mk().step("<think>x</think><solution>select nonsense</solution>")["reward"] == 0.0
    # format: no <think>, two solutions, a tool tag inside the solution, an observation not followed by <think>: -1
    assert mk().step("<solution>select name from t where score > 2</solution>")["reward"] == -1.0
    assert mk().step("<think>x</think><solution>a</solution><solution>b</solution>")["reward"] == -1.0
    assert mk().step("<think>x</think><solution><sql>select 1</sql></solution>")["reward"] == -1.0
    e = mk()
    e.step("<think>a</think><sql>select 1</sql>")
    assert e.step("no thinking <solution>select name from t where score > 2</solution>")["reward"] == -1.0
    e = mk(max_turns=1)
    out = e.step("<think>thinking...</think>")                                        # the turns ran out without a commit
    assert out["done"] and out["reward"] == -1.0
    assert "invalid" in mk().step("<think>x</think> no tag")["observations"][0]["content"]
    # a long result is cut to 50 rows; a runaway query is interrupted
    big = "create table n (i integer, pad text); " + "".join(f"insert into n values ({i}, '{'x' * 40}');" for i in range(400))
    e = gym.make("sql", {"query_timeout_s": 0.3}, {"reward_spec": {"ground_truth": "select 1"}, "schema_sql": big})
    assert "Truncated to 50 lines" in e.step("<think>a</think><sql>select * from n</sql>")["observations"][0]["content"]
    slow = "with recursive c(x) as (select 1 union all select x + 1 from c) select count(*) from c"
    assert "SQL Timeout" in e.step(f"<think>a</think><sql>{slow}</sql>")["observations"][0]["content"]
    e.close()
    # a database on disk in the layout of a released data set
    import sqlite3

    d = tmp_path / "spider" / "database" / "shop"
    d.mkdir(parents=True)
    conn = sqlite3.connect(d / "shop.sqlite")
    conn.executescript(schema)
    conn.commit()
    conn.close()
    e = gym.make("sql", {"db_path": str(tmp_path)}, {"reward_spec": {"ground_truth": "select count(*) from t"}, "db_id": "shop", "data": "spider"})
    assert e.step("<think>x</think><solution>select 3</solution>")["reward"] == 1.0
    import pytest

    with pytest.raises(FileNotFoundError):
        gym.make("sql", {"db_path": str(tmp_path)}, {"reward_spec": {"ground_truth": "select 1"}, "db_id": "nope", "data": "spider"})
    with pytest.raises(NotImplementedError):
        gym.make("sql", {"db_path": str(tmp_path)}, {"reward_spec": {"ground_truth": "select 1"}, "db_id": "shop", "data": "other"})
    assert S.check_format("<think>a</think><solution> select 1 </solution>") == (True, "select 1")


def test_search_env_scores_the_transcript_and_bm25_answers_locally():
    from skyrl_isoexec_b200.gym.envs import search as Q

    corpus = ["The capital of France is Paris.", "Berlin is the capital of Germany.", "Bananas are rich in potassium."]
    env = gym.make("search", {"topk": 2}, {"reward_spec": {"ground_truth": {"target": ["Paris"]}}, "corpus": corpus, "max_turns": 3})
    o = env.step("<search>capital of France</search>")
    assert not o["done"] and o["observations"][0]["content"].startswith("\n<information>Doc 1: The capital of France")
    assert o["metadata"]["status"] == "success" and o["metadata"]["tool_input"] == "capital of France"
    assert env.step("<answer>the Paris.</answer>")["reward"] == 1.0 and env.get_metrics()["searches"] == 1
    env = gym.make("search", {}, {"reward_spec": {"ground_truth": "Paris"}, "corpus": corpus, "max_turns": 2})
    assert "No search results" in env.step("<search>zzz</search>")["observations"][0]["content"]
    out = env.step("<search>qqq</search>")
    assert out["done"] and out["reward"] == 0.0
    # the LAST answer of the transcript counts; substring matching and a format score are options
    assert Q.compute_score("<answer>Rome</answer> no wait <answer>Paris</answer>", {"target": ["Paris"]}) == 1.0
    assert Q.compute_score("<answer>Paris</answer> no wait <answer>Rome</answer>", {"target": ["Paris"]}) == 0.0
    assert Q.compute_score("<answer>it is Paris, France</answer>", {"target": ["Paris"]}) == 0.0
    assert Q.compute_score("<answer>it is Paris, France</answer>", {"target": ["Paris"]}, match="substring") == 1.0
    assert Q.compute_score("<answer>Rome</answer>", ["Paris"], format_score=0.1) == 0.1 and Q.compute_score("none", ["Paris"], format_score=0.1) == 0.0
    assert Q.normalize_answer("  The  Eiffel-Tower! ") == "eiffeltower"
    # a turn without any tag gets no observation and the episode goes on
    env = gym.make("search", {}, {"reward_spec": {"ground_truth": "Paris"}, "corpus": corpus, "max_turns": 3})
    o = env.step("just thinking")
    assert not o["done"] and o["observations"] == []


def test_search_env_over_http_retries_server_errors_and_reports_failures():
    from skyrl_isoexec_b200.gym.retrieval_server import RetrievalServer

    corpus = ["The capital of France is Paris.", "Berlin is the capital of Germany.", "Bananas are rich in potassium."]
    srv = RetrievalServer(corpus).start()
    try:
        cfg = {"search_url": srv.url, "topk": 2, "retry_delay_s": 0.01, "max_retries": 4, "timeout": 5}
        env = gym.make("search", cfg, {"reward_spec": {"ground_truth": {"target": ["Berlin"]}}, "max_turns": 4})
        srv.fail_next = 2                                                      # two 503s, then the answer
        o = env.step("<search>capital of Germany</search>")
        assert "Doc 1: Berlin is the capital" in o["observations"][0]["content"] and env.tool.attempts == 3
        assert o["metadata"]["total_results"] == 2
        srv.fail_next = 10                                                     # more failures than retries: the model is told, nothing raises
        o = env.step("<search>capital of France</search>")
        assert "Search error: server error (503) after 4 attempts" in o["observations"][0]["content"]
        srv.fail_next = 0
        assert env.step("<answer>Berlin</answer>")["reward"] == 1.0
        assert env.get_metrics() == {"turns": 3, "searches": 2, "failed_searches": 1}
        # several queries in one request
        import json
        import urllib.request

        req = urllib.request.Request(srv.url, data=json.dumps({"query": ["bananas", "paris"], "topk": 1, "return_scores": False}).encode())
        res = json.loads(urllib.request.urlopen(req, timeout=5).read())["result"]
        assert len(res) == 2 and "Bananas" in res[0][0]["document"]["contents"] and "score" not in res[0][0]
    finally:
        srv.shutdown()
    dead = gym.make("search", {"search_url": srv.url, "retry_delay_s": 0.0, "max_retries": 2, "timeout": 1},
                    {"reward_spec": {"ground_truth": "x"}, "max_turns": 3})
    assert "Search error: connection error" in dead.step("<search>q</search>")["observations"][0]["content"]


def test_code_grader_stdin_functional_limits_and_guards():
    from skyrl_isoexec_b200.gym.envs import lcb as L

    tests = [{"input": "3 4\n", "output": "7"}, {"input": "10 -2\n", "output": "8"}]
    good = "```python\na, b = map(int, input().split())\nprint(a + b)\n```"
    env = gym.make("lcb", {"timeout_s": 10}, {"reward_spec": {"ground_truth": tests}})
    assert env.step(good)["reward"] == 1.0 and env.step("```python\nprint(0)\n```")["reward"] == 0.0
    out = env.step("no code")
    assert out["reward"] == 0.0 and not out["metadata"]["has_code"]
    loop = "```python\nwhile True: pass\n```"
    e = gym.make("lcb", {"timeout_s": 1}, {"reward_spec": {"ground_truth": json_text(tests)}})      # tests may come as JSON text
    out = e.step(loop)
    assert out["reward"] == 0.0 and out["metadata"]["error_message"] == "Time Limit Exceeded" and e.get_metrics()["timed_out"] == 1.0
    # numbers are compared as numbers, lines after stripping
    num = [{"input": "", "output": "1\n0.5\n"}]
    assert L.compute_score("```python\nprint('1.0  ')\nprint(0.50)\n```", num)[1] == 1.0
    assert L.compute_score("```python\nprint(1)\n```", num)[1] == 0.0
    # call-based tests: a method of Solution or a plain function; a tuple counts as a list; the packed form with fn_name
    fn = [{"input": "[1,2,3]\n2", "output": "[3, 4, 5]", "testtype": "functional", "metadata": {"func_name": "addk"}}]
    assert L.compute_score("```python\nclass Solution:\n    def addk(self, a, k):\n        return tuple(x + k for x in a)\n```", fn)[1] == 1.0
    assert L.compute_score("```py\ndef addk(a, k):\n    return [x + k for x in a]\n```", fn)[1] == 1.0
    assert L.compute_score("```python\nclass Solution:\n    def addk(self, a, k):\n        return a\n```", fn)[2]["error_message"] == "Wrong Answer"
    packed = {"inputs": ["[1]\n1"], "outputs": ["[2]"], "fn_name": "addk"}
    assert L.compute_score("```python\ndef addk(a, k):\n    return [x + k for x in a]\n```", packed)[1] == 1.0
    assert L.compute_score("```python\ndef other():\n    pass\n```", fn)[2]["error_message"] == "Runtime Error"
    # the sandbox: destructive calls are disabled, memory is capped, exit() does not pass a test, syntax errors are reported
    assert L.compute_score("```python\nimport os\nos.system('echo hi')\nprint(7)\n```", tests)[1] == 0.0
    assert "MemoryError" in L.compute_score("```python\nx = [0] * (10 ** 10)\n```", tests)[2]["error"]
    assert L.compute_score("```python\nimport sys\nsys.exit(0)\n```", tests)[2]["error_message"] == "Wrong Answer"
    assert L.compute_score("```python\ndef f(:\n```", tests)[2]["error_message"] == "Compilation Error"
    # the first failure stops the run: one verdict per test reached
    res, meta = L.grade("a, b = map(int, input().split())\nprint(a + b if a == 3 else 0)", tests)
    assert res == [True, -2] and meta["expected"] == "8"
    import pytest

    with pytest.raises(ValueError, match="func_name"):
        L.normalize_tests([{"input": "1", "output": "1", "testtype": "functional"}])


def json_text(x):
    import json

    return json.dumps(x)


def test_searchcode_env_runs_python_beside_search():
    corpus = ["def add(a, b): return a + b  # adds two numbers"]
    sc = gym.make("searchcode", {}, {"reward_spec": {"ground_truth": {"target": ["5"]}}, "corpus": corpus, "max_turns": 4})
    o = sc.step("<search>add two numbers</search>")
    assert "def add" in o["observations"][0]["content"]
    o = sc.step("<python>print(2 + 3)</python>")
    assert o["observations"][0]["content"] == "\n<information>5</information>\n" and o["metadata"]["tool_name"] == "python"
    o = sc.step("<python>raise ValueError('boom')</python> <search>later</search>")          # the first tag of a turn runs
    assert "ValueError: boom" in o["observations"][0]["content"]
    assert sc.step("<answer>5</answer>")["reward"] == 1.0
    assert sc.get_metrics() == {"turns": 4, "searches": 1, "failed_searches": 0, "python_runs": 2}


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


def test_rlm_env_in_process_repl_with_language_model_and_child_agent_calls():
    from skyrl_isoexec_b200.gym.repl import PersistentREPL

    docs = {"paper_a": "Alpha study. The measured gain was 12 percent.", "paper_b": "Beta study. The measured gain was 30 percent."}
    asked = []

    def lm(prompts):
        asked.extend(prompts)
        return ["30" if "Beta" in p else "12" for p in prompts]

    def child(prompt, context=None):                       # a child agent: gets the sub-task and ITS context, answers with text
        return str([len(context or ""), "gain" in (context or "")])

    ex = {"extra_info": {"context_text": __import__("json").dumps(docs)}, "reward_spec": {"ground_truth": "30"}, "max_turns": 6,
          "lm_callback": lm, "subcall_fn": child, "tools": {"word_count": lambda s: len(s.split()), "TOPK": 1}, "timeout_s": 5}
    env = gym.make("rlm", {}, ex)
    prompt, info = env.init([{"role": "user", "content": "Which paper reports the larger gain, and how large is it?"}])
    sys_text = prompt[0]["content"]
    assert "dict with 2 entries" in sys_text and "llm_query" in sys_text and "word_count()" in sys_text and "TOPK" in sys_text
    assert docs["paper_a"] not in sys_text
    r = env.step("```repl\ngains = llm_query_batched(['Gain in: ' + v for v in context.values()])\nprint(gains, word_count(context['paper_a']), TOPK)\n```")
    assert "['12', '30'] 8 1" in r["observations"][0]["content"] and len(asked) == 2
    r = env.step("```repl\nkids = rlm_query_batched(['check', 'check'], context_list=list(context.values()))\nprint(kids[0], type(kids[1]).__name__)\n```")
    assert "[46, True] list" in r["observations"][0]["content"]                    # a literal answer of a child comes back as an object
    r = env.step("```repl\nimport os\n```")
    assert "not allowed" in r["observations"][0]["content"]
    r = env.step("```repl\nbest = max(gains, key=int)\nFINAL_VAR('best')\n```")      # ends the episode from inside the block
    assert r["done"] and r["reward"] == 1.0 and r["metadata"] == {"final": "30", "how": "FINAL_VAR in block"}
    assert env.get_metrics() == {"rlm/turns": 4, "rlm/blocks_run": 4, "rlm/block_errors": 1, "rlm/lm_calls": 2, "rlm/child_calls": 2}
    # FINAL_VAR in a message of its own, and a variable that does not exist
    env = gym.make("rlm", {"repl": "inprocess"}, {"context": "abc", "reward_spec": {"ground_truth": "3"}, "max_turns": 4})
    env.init([{"role": "user", "content": "length?"}])
    env.step("```repl\nn = len(context)\n```")
    assert "FINAL_VAR failed" in env.step("FINAL_VAR(m)")["observations"][0]["content"]
    assert env.step("FINAL_VAR(n)")["reward"] == 1.0

    class Judge(type(env)):                                # a task adapts scoring, prompt and tools by overriding the hooks
        def get_reward(self, final_answer):
            return 0.5 if "x" in str(final_answer) else 0.0

        def system_prompt(self):
            return "CUSTOM"

        def repl_tools(self):
            return {"shout": lambda s: s.upper()}

    j = Judge({"repl": "inprocess"}, {"context": "abc", "max_turns": 2})
    p, _ = j.init([{"role": "user", "content": "q"}])
    assert p[0]["content"].startswith("CUSTOM") and "shout()" in p[0]["content"]
    assert "ABC" in j.step("```repl\nprint(shout(context))\n```")["observations"][0]["content"]
    assert j.step("FINAL(xyz)")["reward"] == 0.5
    # the REPL on its own: helpers cannot be redefined for the next block, tool names are checked
    r = PersistentREPL(timeout_s=1.0)
    r.execute("SHOW_VARS = None; y = 2")
    assert "y" in r.execute("print(SHOW_VARS())").stdout
    import pytest

    with pytest.raises(ValueError):
        PersistentREPL(tools={"context": 1})


def test_rlm_generator_gives_blocks_the_policy_and_child_trajectories():
    """The engine is scripted: what it 'generates' depends on the prompt, so that the control flow can be checked."""
    import asyncio

    from skyrl_isoexec_b200.engine.interface import InferenceEngineInterface
    from skyrl_isoexec_b200.train.rlm_generator import RLMGymGenerator
    from skyrl_isoexec_b200.utils.tokenizer import ByteTokenizer

    tok = ByteTokenizer()
    calls = []

    class Scripted(InferenceEngineInterface):
        async def generate(self, batch):
            outs = []
            for ids in batch["prompt_token_ids"]:
                text = tok.decode(ids)
                turns = tok.decode(ids, skip_special_tokens=False).count("<|im_start|>assistant\n")
                calls.append((text[-60:], batch["sampling_params"].get("max_generate_length")))
                if "How many words" in text and "REPL" not in text:
                    reply = "three"                                                       # a plain completion (llm_query)
                elif "How long is the document" not in text:                              # a child trajectory (its task: SUBTASK count)
                    reply = "```repl\nn = len(context.split())\n```" if turns == 1 else "FINAL_VAR(n)"
                elif turns == 1:                                                          # the root: asks a child and the plain model
                    reply = "```repl\nk = rlm_query('SUBTASK count', context=context['doc'])\nw = llm_query('How many words?')\nprint(k, w)\n```"
                else:
                    reply = "FINAL_VAR(k)"
                outs.append(tok.encode(reply))
            n = len(outs)
            return {"responses": [tok.decode(o) for o in outs], "response_ids": outs, "stop_reasons": ["stop"] * n,
                    "response_logprobs": [[-0.5] * len(o) for o in outs]}

        async def wake_up(self, *a, **kw): ...
        async def sleep(self, *a, **kw): ...
        async def init_weight_update_communicator(self, init_info): ...
        async def update_named_weights(self, request): ...

    gen = RLMGymGenerator(Scripted(), tok, max_turns=4, max_depth=1, lm_max_tokens=16, train_children=True)
    inp = {"prompts": [[{"role": "user", "content": "How long is the document?"}]], "env_classes": ["rlm"],
           "env_extras": [{"context": {"doc": "one two three four"}, "reward_spec": {"ground_truth": "4"}}],
           "sampling_params": {"max_generate_length": 64}, "trajectory_ids": ["t0"]}
    out = asyncio.run(gen.generate(inp))
    assert out["trajectory_ids"] == ["t0", "t0/c0"] and out["step_source"] == [0, 0]
    assert sum(out["rewards"][0]) == 1.0 and out["rewards"][1][-1] == 1.0 and sum(out["rewards"][1]) == 1.0   # the child inherits the root's outcome
    assert out["rollout_metrics"]["generate/child_trajectories"] == 1 and out["rollout_metrics"]["environment/rlm/child_calls"] == 1
    assert any(m == 16 for _, m in calls) and any(m == 64 for _, m in calls)          # plain completions use lm_max_tokens
    obs_text = tok.decode(out["response_ids"][0])
    assert "4 three" in obs_text                                                        # the block printed the child's answer and the completion
    # without train_children the child is only counted
    gen2 = RLMGymGenerator(Scripted(), tok, max_turns=4, max_depth=1, lm_max_tokens=16)
    out2 = asyncio.run(gen2.generate(inp))
    assert out2["trajectory_ids"] == ["t0"] and "step_source" not in out2 and out2["rollout_metrics"]["generate/child_trajectories"] == 1
    # past max_depth a child call degrades to a plain completion
    gen3 = RLMGymGenerator(Scripted(), tok, max_turns=4, max_depth=0, lm_max_tokens=16)
    out3 = asyncio.run(gen3.generate(inp))
    assert out3["rollout_metrics"]["generate/child_trajectories"] == 0


def test_trainer_builds_the_rlm_generator_and_steps_on_a_repl_environment(tmp_path):
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
    from skyrl_isoexec_b200.train.rlm_generator import RLMGymGenerator
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer
    from skyrl_isoexec_b200.utils.tokenizer import ByteTokenizer

    class Rows:
        rows = [{"prompt": [{"role": "user", "content": f"question {i}"}], "env_class": "rlm",
                 "env_extras": {"context": f"document {i} " * 20, "reward_spec": {"ground_truth": str(i)}}, "uid": f"r{i}"} for i in range(8)]

        def __len__(self):
            return len(self.rows)

        def __getitem__(self, i):
            return self.rows[i]

    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=6", "generator.sampling_params.ignore_eos=true",
        "generator.rlm=true", "generator.batched=false", "generator.max_turns=2", "generator.rlm_train_children=true",
        "trainer.max_prompt_length=2048", "generator.inference_engine.num_kv_pages=96", "trainer.num_steps=1", "trainer.logger=jsonl",
        f"trainer.ckpt_path={tmp_path}", "trainer.resume_mode=none", 'trainer.policy.model_overrides={"max_position": 4096}'])
    tr = RayPPOTrainer(cfg, device="cpu", dataset=Rows(), tokenizer=ByteTokenizer())
    tr.train()
    assert isinstance(tr.generator, RLMGymGenerator) and tr.global_step == 1
    assert tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0
