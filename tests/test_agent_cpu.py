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
