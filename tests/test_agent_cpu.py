"""Agent layer on CPU with a scripted engine (deterministic 'model') and with the real tiny engine."""
import asyncio
import json

import torch

from skyrl_isoexec_b200.agent.react import AsyncDispatcher, ReActAgent, ToolRegistry, to_generator_output
from skyrl_isoexec_b200.utils.tokenizer import ByteTokenizer


class ScriptedEngine:
    """Answers turn k of every conversation with script[k] (as bytes) and fixed logprobs."""

    def __init__(self, tok, script):
        self.tok, self.script, self.calls = tok, script, {}

    async def generate(self, batch):
        ctx = tuple(batch["prompt_token_ids"][0][:40])
        k = self.calls.get(ctx, 0)
        self.calls[ctx] = k + 1
        ids = self.tok.encode(self.script[min(k, len(self.script) - 1)])
        return {"response_ids": [ids], "response_logprobs": [[-0.5] * len(ids)], "stop_reasons": ["stop"]}


def test_react_agent_calls_tools_and_masks_observations():
    tok = ByteTokenizer()
    assert tok.decode(tok.encode("héllo")) == "héllo"
    tools = ToolRegistry()
    tools.register("add", lambda a, b: {"sum": a + b}, "add two numbers")
    script = ['I need the sum. <tool>{"name": "add", "arguments": {"a": 2, "b": 40}}</tool>', "<tool>not json</tool>", "<finish>42</finish>"]
    agent = ReActAgent(ScriptedEngine(tok, script), tok, tools, max_turns=5)
    inst = [{"id": "q1", "task": "What is 2 + 40?", "judge": lambda ans, tr: 1.0 if ans == "42" else 0.0}]
    trajs = asyncio.run(AsyncDispatcher(agent, max_parallel=2).run(inst, n_samples=2))
    assert len(trajs) == 2
    t = trajs[0]
    assert t.finish == "42" and t.reward == 1.0 and t.turns == 3 and t.tool_calls == ["add"]
    assert len(t.response_ids) == len(t.loss_mask) == len(t.logprobs)
    text = tok.decode(t.response_ids)
    assert '{"sum": 42}' in text and "not valid JSON" in text
    obs_start = text.index('{"sum": 42}')
    n_model = sum(t.loss_mask)
    assert 0 < n_model < len(t.loss_mask) and all(lp == 0.0 for lp, m in zip(t.logprobs, t.loss_mask) if m == 0)
    go, uids = to_generator_output(trajs)
    assert uids == ["q1", "q1"] and sum(go["rewards"][0]) == 1.0
    last_model = max(i for i, m in enumerate(t.loss_mask) if m)
    assert go["rewards"][0][last_model] == 1.0 and obs_start > 0


def test_agent_trajectories_train_through_the_real_engine(tmp_path):
    """Random tiny model, byte tokenizer: the trajectories (model turns + masked tool observations) go through
    convert_to_training_input and the scoring forward reproduces the rollout logprobs on the model tokens."""
    from skyrl_isoexec_b200.engine.interface import NativeInferenceEngine
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2", "generator.n_samples_per_prompt=2",
        "generator.inference_engine.num_kv_pages=64", "trainer.max_prompt_length=400", "generator.sampling_params.max_generate_length=12",
        "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}", "trainer.ckpt_interval=0"])
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.build_models()
    tr.engine.wake_up()
    tok = ByteTokenizer()
    tools = ToolRegistry()
    tools.register("echo", lambda **kw: kw, "returns its arguments")
    agent = ReActAgent(NativeInferenceEngine(tr.engine, tok), tok, tools, max_turns=2, sampling_params={"max_generate_length": 12, "ignore_eos": True})
    inst = [{"id": f"t{i}", "task": f"task {i}", "judge": lambda ans, t: float(len(t.response_ids) % 2)} for i in range(2)]
    trajs = asyncio.run(AsyncDispatcher(agent).run(inst, n_samples=2))
    go, uids = to_generator_output(trajs)
    batch = tr.convert_to_training_input(go, uids)
    lp = tr.policy.forward(batch)
    mask = batch["loss_mask"]
    assert torch.equal((lp * mask), (batch["rollout_logprobs"] * mask))           # model tokens: bitwise on-policy
    assert float(mask.sum()) == 4 * 24 and (batch["response_mask"].sum() > mask.sum())


def test_codeact_agent_runs_code_keeps_state_between_snippets_and_masks_observations():
    from skyrl_isoexec_b200.agent.codeact import CodeActAgent

    tok = ByteTokenizer()
    script = ["First the data.\n<execute_python>\nxs = [3, 4, 5]\nprint(sum(xs))\n</execute_python>",
              "<execute_python>\nprint(1 / 0)\n</execute_python>",                       # an error: not added to the prelude
              "<execute_python>\nprint(sum(x * x for x in xs))\n</execute_python>",      # xs persists; the earlier print does not repeat
              "<execute_bash>ls</execute_bash>",
              "<finish>50</finish>"]
    agent = CodeActAgent(ScriptedEngine(tok, script), tok, max_turns=6)
    inst = [{"id": "c1", "task": "Sum of squares of 3, 4, 5?", "judge": lambda ans, tr: 1.0 if ans == "50" else 0.0}]
    (t,) = asyncio.run(AsyncDispatcher(agent, max_parallel=1).run(inst))
    assert t.finish == "50" and t.reward == 1.0 and t.turns == 5 and t.tool_calls == ["python", "python", "python"]
    text = tok.decode(t.response_ids)
    assert "ZeroDivisionError" in text and "bash is not available" in text
    first = text.index("</execute_python>")
    third_obs = text[text.rindex("</execute_python>"):]
    assert "12" in text[first:first + 80] and "50" in third_obs and "12" not in third_obs.split("<finish>")[0].split("execute_bash")[0]
    assert len(t.response_ids) == len(t.loss_mask) == len(t.logprobs) and 0 < sum(t.loss_mask) < len(t.loss_mask)
    go, uids = to_generator_output([t])
    assert uids == ["c1"] and sum(go["rewards"][0]) == 1.0


def test_agents_run_against_a_tinker_service_and_train_it_on_their_trajectories(tmp_path):
    """The model that a Tinker-style service is training serves the agent's turns; the trajectories go back as
    forward_backward data with observation tokens masked, and the service's forward reproduces the sampled logprobs
    on the model tokens bit for bit."""
    from skyrl_isoexec_b200.agent.integrations import TinkerSamplingEngine, trajectories_to_tinker_batch
    from skyrl_isoexec_b200.tinker.api import TinkerClient, TinkerServer

    srv = TinkerServer(db_path=str(tmp_path / "q.db"), device="cpu").start()
    try:
        cl = TinkerClient(srv.url)
        mid = cl.create_model(base_model="tiny-qwen3", lr=1e-3)
        tok = ByteTokenizer()
        tools = ToolRegistry()
        tools.register("echo", lambda **kw: kw, "returns its arguments")
        eng = TinkerSamplingEngine(cl, mid)
        agent = ReActAgent(eng, tok, tools, max_turns=2, sampling_params={"max_generate_length": 10, "ignore_eos": True})
        inst = [{"id": f"t{i}", "task": f"task {i}", "judge": lambda ans, t: float(t.response_ids[0] % 2)} for i in range(2)]
        trajs = asyncio.run(AsyncDispatcher(agent, max_parallel=2).run(inst, n_samples=1))
        assert eng.calls == 4 and all(t.turns == 2 and sum(t.loss_mask) == 20 < len(t.loss_mask) for t in trajs)
        batch = trajectories_to_tinker_batch(trajs)
        fwd = cl.call("forward", model_id=mid, **batch)
        for t, lp in zip(trajs, fwd["logprobs"]):
            assert [a for a, m in zip(lp, t.loss_mask) if m] == [a for a, m in zip(t.logprobs, t.loss_mask) if m]
        out = cl.call("forward_backward", model_id=mid, loss_fn="importance_sampling", **batch)
        assert out["num_tokens"] == 40                                   # only the model tokens carry loss
        assert cl.call("optim_step", model_id=mid, adam_params={})["step"] == 1
    finally:
        srv.shutdown()


# ------------------------------------------------------------------ function calling, toolkit, history, verifiers, tasks
class TurnEngine:
    """Replies with script[number of assistant turns already in the prompt]."""

    def __init__(self, tok, script, by_call=False):
        self.tok, self.script, self.prompts, self.by_call = tok, script, [], by_call

    async def generate(self, batch):
        ids = batch["prompt_token_ids"][0]
        text = self.tok.decode(ids, skip_special_tokens=False)
        self.prompts.append(text)
        k = len(self.prompts) - 1 if self.by_call else text.count("<|im_start|>assistant\n") - 1       # by_call: one conversation
        out = self.tok.encode(self.script[min(k, len(self.script) - 1)])
        return {"response_ids": [out], "response_logprobs": [[-0.25] * len(out)], "stop_reasons": ["stop"]}


def test_function_calling_text_protocol_round_trips_and_validates():
    import pytest

    from skyrl_isoexec_b200.agent import function_calling as F

    tools = [{"type": "function", "function": {"name": "search", "description": "Search the corpus.", "parameters": {
                  "type": "object", "properties": {"query": {"type": "string", "description": "what to look for"}, "topk": {"type": "integer"},
                                                   "mode": {"type": "string", "enum": ["fast", "deep"]}, "flags": {"type": "array"},
                                                   "strict": {"type": "boolean"}}, "required": ["query"]}}},
             {"type": "function", "function": {"name": "finish", "description": "End."}}]
    prompt = F.tools_prompt(tools)
    assert "BEGIN FUNCTION #1: search" in prompt and "(1) query (string, required): what to look for" in prompt
    assert "Allowed values: [`fast`, `deep`]" in prompt and "No parameters are required" in prompt and "<function=" in prompt
    text = "Let me search.\n\n<function=search>\n<parameter=query>capital of\nFrance</parameter>\n<parameter=topk>2</parameter>\n" \
           "<parameter=flags>[1, 2]</parameter>\n<parameter=strict>True</parameter>\n</function"           # cut at the stop word
    before, call = F.parse_call(text, tools)
    assert before == "Let me search." and call == {"name": "search", "arguments": {"query": "capital of\nFrance", "topk": 2, "flags": [1, 2], "strict": True}}
    assert F.parse_call("just text", tools) == ("just text", None)
    for bad, why in (("<function=nope>\n</function>", "not available"), ("<function=search>\n<parameter=topk>x</parameter>\n</function>", "type integer"),
                     ("<function=search>\n<parameter=topk>1</parameter>\n</function>", "Missing required"),
                     ("<function=search>\n<parameter=query>a</parameter>\n<parameter=mode>slow</parameter>\n</function>", "allowed values"),
                     ("<function=search>\n<parameter=query>a</parameter>\n<parameter=zzz>1</parameter>\n</function>", "not accepted"),
                     ("<function=search>\n<parameter=query>a</parameter>\n<parameter=query>b</parameter>\n</function>", "twice"),
                     ("<function=search>\n<parameter=query>a", "not closed")):
        with pytest.raises(F.FunctionCallValidationError, match=why):
            F.parse_call(bad, tools)
    msgs = [{"role": "system", "content": "sys"}, {"role": "user", "content": "q"},
            {"role": "assistant", "content": "thinking", "tool_calls": [{"id": "c1", "type": "function", "function": {"name": "search", "arguments": '{"query": "x\\ny", "topk": 3}'}}]},
            {"role": "tool", "tool_call_id": "c1", "content": "Doc 1"}, {"role": "assistant", "content": "done"}]
    plain = F.to_text_messages(msgs, tools)
    assert plain[0]["content"].startswith("sys") and prompt in plain[0]["content"]
    assert plain[2]["content"] == "thinking\n\n<function=search>\n<parameter=query>\nx\ny\n</parameter>\n<parameter=topk>3</parameter>\n</function>"
    assert plain[3] == {"role": "user", "content": "EXECUTION RESULT of [search]:\nDoc 1"}
    back = F.to_tool_messages(plain, tools)
    assert back[0]["content"] == "sys" and back[2]["content"] == "thinking" and back[4] == {"role": "assistant", "content": "done"}
    assert json.loads(back[2]["tool_calls"][0]["function"]["arguments"]) == {"query": "x\ny", "topk": 3}
    assert back[3]["role"] == "tool" and back[3]["content"] == "Doc 1" and back[3]["tool_call_id"] == back[2]["tool_calls"][0]["id"]
    with pytest.raises(F.FunctionCallConversionError):
        F.to_text_messages([{"role": "tool", "content": "orphan"}], tools)
    with pytest.raises(F.FunctionCallConversionError):
        F.to_tool_messages([{"role": "user", "content": "EXECUTION RESULT of [search]:\nx"}], tools)
    with pytest.raises(F.FunctionCallConversionError):
        F.call_to_text({"id": "a", "type": "function", "function": {"name": "f", "arguments": "{not json"}})
    assert F.to_text_messages([{"role": "user", "content": "q"}], tools)[0]["role"] == "system"          # no system message: one is made


def test_toolkit_registry_cache_search_sandbox_and_finish_tools(tmp_path):
    import pytest

    from skyrl_isoexec_b200.agent import toolkit as T

    assert {"finish", "em_finish", "local_search", "code_interpreter", "memory"} <= set(T.TOOL_REGISTRY)
    with pytest.raises(ValueError):
        T.register_tool("finish")(type("X", (T.BaseTool,), {}))
    with pytest.raises(KeyError):
        T.make_tools(["nope"])
    tools = T.make_tools(["local_search", "em_finish", "code_interpreter", "memory"],
                         local_search={"corpus": ["Paris is the capital of France.", "Berlin is in Germany."], "topk": 1})
    s = tools["local_search"]
    assert s.schema()["function"]["parameters"]["required"] == ["query"]
    assert s.call({"query": "capital France"}).startswith("Doc 1: Paris") and s.call('{"query": "capital France"}').startswith("Doc 1: Paris")
    assert s.cache.stats() == {"entries": 1, "hits": 1, "misses": 1}
    with pytest.raises(T.ToolError, match="missing required"):
        s.call({})
    with pytest.raises(T.ToolError, match="not valid JSON"):
        s.call("{oops")
    assert tools["em_finish"].call({"answer": "the Paris!"}, ground_truth=["Paris"]) == {"answer": "the Paris!", "reward": 1.0}
    assert tools["em_finish"].call({"answer": "Rome"}, ground_truth="Paris")["reward"] == 0.0 and tools["em_finish"].ends_trajectory
    assert tools["code_interpreter"].call({"code": "print(int(input()) * 2)", "stdin": "21"}) == "42"
    assert "ZeroDivisionError" in tools["code_interpreter"].call({"code": "1/0"})
    state = {}
    assert "Memory updated" in tools["memory"].call({"notes": "remember 7"}, state=state) and state["memory"] == "remember 7"
    # the cache: time-to-live, capacity, persistence
    c = T.ToolCache(capacity=2, ttl_s=0.05, path=str(tmp_path / "cache.json"))
    calls = []
    f = lambda: calls.append(1) or "v"
    assert c.through("t", {"a": 1}, f) == "v" and c.through("t", {"a": 1}, f) == "v" and len(calls) == 1
    import time

    time.sleep(0.08)
    assert c.through("t", {"a": 1}, f) == "v" and len(calls) == 2                                  # expired
    c.put("k1", 1), c.put("k2", 2), c.put("k3", 3)
    assert c.get("t:" + json.dumps({"a": 1})) is None and c.stats()["entries"] == 2                  # the oldest entries went
    c.save()
    assert T.ToolCache(path=str(tmp_path / "cache.json")).get("k3") == 3


def test_history_trims_to_a_budget_and_flags_the_reset():
    from skyrl_isoexec_b200.agent.history import MessageHistory, preview

    h = MessageHistory([{"role": "system", "content": "sys"}, {"role": "user", "content": "task"}])
    assert not h.was_reset()
    for i in range(6):
        h.add_assistant(f"call {i}")
        h.add_tool_response("search", "x" * 1000 + str(i))
    count = lambda ms: sum(len(m["content"]) for m in ms)
    assert not h.fit(count, 10 ** 6) and not h.was_reset()
    assert h.fit(count, 3000) and h.was_reset() and count(h.get_messages()) <= 3000
    msgs = h.get_messages()
    assert msgs[0]["content"] == "sys" and msgs[1]["content"] == "task" and "earlier messages were removed" in msgs[2]["content"]
    assert msgs[3]["role"] == "assistant" and msgs[-1]["content"].endswith("5")                       # the latest result is whole
    assert "characters cut" in msgs[4]["content"]                                                     # older ones are previews
    h.clear_reset_flag()
    h.add_tool_error("search", "down")
    assert '"error": "down"' in h.get_messages()[-1]["content"]
    h.append_to_last(" [2 turns left]")
    assert h.get_messages()[-1]["content"].endswith("[2 turns left]") and len(preview("a" * 1000, 100)) < 200


def test_verifiers_score_qa_math_and_code():
    from skyrl_isoexec_b200.agent import verifiers as V

    s = V.qa_scores("The Eiffel Tower in Paris", ["Eiffel Tower", "tower"])
    assert s["em"] == 0.0 and s["sub_em"] == 1.0 and abs(s["f1"] - 2 / 3) < 1e-9
    assert V.qa_reward("eiffel tower", ["Eiffel Tower"]) == 1.0 and V.qa_reward("x", "y", "f1") == 0.0
    assert V.math_reward("so \\boxed{0.5}", "\\frac{1}{2}") == 1.0 and V.math_reward("\\boxed{3}", "4", wrong_reward=-1.0) == -1.0
    assert V.math_reward("Answer: 1,000", "1000") == 1.0
    tests = [{"input": "2", "output": "4"}, {"input": "3", "output": "7"}]
    prog = "```python\nprint(int(input()) * 2)\n```"
    assert V.code_reward(prog, tests) == 0.0 and V.code_reward(prog, tests, partial=True) == 0.5 and V.code_reward("none", tests) == 0.0


def test_function_call_agent_uses_tools_recovers_from_bad_calls_and_segments_on_trimming():
    from skyrl_isoexec_b200.agent.fc_agent import FunctionCallAgent
    from skyrl_isoexec_b200.agent.toolkit import make_tools

    tok = ByteTokenizer()
    tools = make_tools(["local_search", "memory", "em_finish"], local_search={"corpus": ["Paris is the capital of France.", "Berlin is in Germany."]})
    script = ["I should search.\n<function=local_search>\n<parameter=query>capital of France</parameter>\n</function>",
              "<function=local_search>\n<parameter=topk>two</parameter>\n</function>",                        # wrong type, no query
              "hmm, no call here",
              "<function=memory>\n<parameter=notes>France -> Paris</parameter>\n</function>",
              "<function=em_finish>\n<parameter=answer>Paris</parameter>\n</function"]
    eng = TurnEngine(tok, script)
    agent = FunctionCallAgent(eng, tok, tools, max_turns=8)
    segs = asyncio.run(agent.run("q1", "What is the capital of France?", ground_truth=["Paris"]))
    assert len(segs) == 1
    t = segs[0]
    assert t.finish == "Paris" and t.reward == 1.0 and t.turns == 5 and t.tool_calls == ["local_search", "memory", "em_finish"]
    assert len(t.response_ids) == len(t.loss_mask) == len(t.logprobs) and sum(t.loss_mask) == sum(len(tok.encode(s)) for s in script)
    text = tok.decode(t.response_ids)
    assert "EXECUTION RESULT of [local_search]:\nDoc 1: Paris" in text and "turns left]" in text
    assert "could not be run" in text and "contains no function call" in text
    assert "Your memory" not in eng.prompts[-1]                                    # nothing was dropped: the memory call is still in view
    assert eng.prompts[0].count("BEGIN FUNCTION") == 3 and agent.sp["stop"] == ["</function"]
    assert tok.decode(t.prompt_ids + t.response_ids, skip_special_tokens=False).count("<|im_start|>assistant\n") == 5
    # a small context forces trimming: the trajectory comes back as several self-contained segments with one outcome
    long_doc = ["Paris is the capital of France. " + "filler " * 300]
    tools2 = make_tools(["local_search", "memory", "em_finish"], local_search={"corpus": long_doc})
    script2 = ["<function=memory>\n<parameter=notes>France -> Paris</parameter>\n</function>"] + \
              ["<function=local_search>\n<parameter=query>capital France</parameter>\n</function>"] * 3 + \
              ["<function=em_finish>\n<parameter=answer>Paris</parameter>\n</function>"]
    eng2 = TurnEngine(tok, script2, by_call=True)        # trimming removes turns from the prompt: count the calls instead
    agent2 = FunctionCallAgent(eng2, tok, tools2, max_turns=6, max_context=4200, turn_reminder=False)
    segs2 = asyncio.run(agent2.run("q2", "capital of France?", ground_truth="Paris"))
    assert len(segs2) >= 2 and [s.instance_id for s in segs2][:2] == ["q2", "q2@1"]
    assert all(s.reward == 1.0 and s.finish == "Paris" for s in segs2) and all(len(s.prompt_ids) <= 4200 for s in segs2)
    last_prompt = tok.decode(segs2[-1].prompt_ids)
    assert "earlier messages were removed" in last_prompt and "Your memory:\nFrance -> Paris" in last_prompt


def test_auto_runner_builds_agent_tools_and_task_from_a_config(tmp_path):
    from skyrl_isoexec_b200.agent.tasks import AutoAgentRunner, GeneralReactTask

    tok = ByteTokenizer()
    cfg = {"agent": {"type": "function_call", "max_turns": 4}, "tools": ["local_search", "finish"],
           "tool_kwargs": {"local_search": {"corpus": ["Paris is the capital of France."]}},
           "task": {"type": "general_react", "metric": "sub_em"}, "dispatcher": {"max_parallel": 2, "n_samples": 2}}
    script = ["<function=local_search>\n<parameter=query>capital</parameter>\n</function>",
              "<function=finish>\n<parameter=answer>It is Paris.</parameter>\n</function>"]
    runner = AutoAgentRunner.from_config(cfg, TurnEngine(tok, script), tok)
    rows = [{"id": "a", "prompt": [{"role": "user", "content": "Capital of France?"}], "data_source": "nq", "reward_spec": {"ground_truth": {"target": ["Paris"]}}},
            {"id": "b", "question": "Capital of Spain?", "reward_spec": {"ground_truth": ["Madrid"]}}]
    go, uids = runner.run(rows)
    assert uids == ["a", "a", "b", "b"] and [sum(r) for r in go["rewards"]] == [1.0, 1.0, 0.0, 0.0]
    assert go["rollout_metrics"]["agent/avg_reward"] == 0.5 and go["rollout_metrics"]["agent/segments_per_trajectory"] == 1.0
    # the same from a YAML file; math and code rows are scored by their own verifiers
    import yaml

    (tmp_path / "agent.yaml").write_text(yaml.safe_dump(cfg))
    assert isinstance(AutoAgentRunner.from_config(str(tmp_path / "agent.yaml"), TurnEngine(tok, script), tok).task, GeneralReactTask)
    task = GeneralReactTask()
    assert task.evaluate("1/2", {"data_source": "math", "reward_spec": {"ground_truth": "\\frac{1}{2}"}}) == 1.0       # equal as numbers
    assert task.evaluate("1/3", {"data_source": "math", "reward_spec": {"ground_truth": "\\frac{1}{2}"}}) == 0.0
    assert task.evaluate("\\frac{1}{2}", {"data_source": "aime", "reward_spec": {"ground_truth": "\\frac{1}{2}"}}) == 1.0
    assert task.evaluate("print(int(input()) + 1)", {"data_source": "lcb", "reward_spec": {"ground_truth": [{"input": "1", "output": "2"}]}}) == 1.0
    assert task.evaluate(None, rows[0]) == 0.0
    for kind in ("react", "codeact"):
        assert AutoAgentRunner.from_config({"agent": {"type": kind}, "tools": ["local_search"], "tool_kwargs": {"local_search": {"corpus": ["x"]}}},
                                           TurnEngine(tok, script), tok).agent is not None
