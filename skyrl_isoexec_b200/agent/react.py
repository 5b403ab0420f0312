"""ReAct-style tool agent, trajectory dispatcher and the adapter that turns finished trajectories into trainer input
(reference: skyrl-agent/skyrl_agent/{agents/react,dispatcher,integrations/skyrl_train}).

An agent turn: the model writes text; if it contains ``<tool>{"name": ..., "arguments": {...}}</tool>`` the tool runs
and its result is appended as an observation; ``<finish>answer</finish>`` (or the turn limit) ends the trajectory.
Model tokens carry loss mask 1 and their rollout logprobs; observation tokens carry mask 0. The dispatcher runs many
trajectories concurrently against one engine (continuous batching does the rest) with a concurrency limit.
"""

from __future__ import annotations

from ..utils.tokenizer import chat_ids, chat_ids_continuation

import asyncio
import json
import re
import time
from dataclasses import dataclass, field
from typing import Callable

_TOOL = re.compile(r"<tool>(.*?)</tool>", re.S)
_FINISH = re.compile(r"<finish>(.*?)</finish>", re.S)


@dataclass
class Trajectory:
    instance_id: str
    prompt_ids: list = field(default_factory=list)
    response_ids: list = field(default_factory=list)
    loss_mask: list = field(default_factory=list)
    logprobs: list = field(default_factory=list)
    reward: float = 0.0
    finish: str | None = None
    turns: int = 0
    stop_reason: str = "stop"
    tool_calls: list = field(default_factory=list)
    seconds: float = 0.0


class ToolRegistry:
    def __init__(self):
        self.tools: dict[str, Callable] = {}

    def register(self, name: str, fn: Callable, description: str = "") -> None:
        self.tools[name] = fn
        fn.__doc__ = fn.__doc__ or description

    def describe(self) -> str:
        return "\n".join(f"- {n}: {(f.__doc__ or '').strip()}" for n, f in sorted(self.tools.items()))

    def call(self, name: str, arguments: dict):
        if name not in self.tools:
            return {"error": f"unknown tool {name!r}; available: {sorted(self.tools)}"}
        try:
            return self.tools[name](**(arguments or {}))
        except Exception as e:  # noqa: BLE001
            return {"error": f"{type(e).__name__}: {e}"}


class ReActAgent:
    SYSTEM = ("You can call tools by writing <tool>{\"name\": NAME, \"arguments\": {...}}</tool>. "
              "When you are done write <finish>your answer</finish>.\nTools:\n")

    def __init__(self, engine, tokenizer, tools: ToolRegistry, max_turns: int = 8, sampling_params: dict | None = None,
                 max_context: int = 1 << 30):
        self.engine, self.tok, self.tools = engine, tokenizer, tools
        self.max_turns, self.sp, self.max_context = max_turns, sampling_params or {}, max_context

    async def run(self, instance_id: str, task: str, judge: Callable[[str | None, Trajectory], float]) -> Trajectory:
        t0 = time.time()
        tr = Trajectory(instance_id)
        msgs = [{"role": "system", "content": self.SYSTEM + self.tools.describe()}, {"role": "user", "content": task}]
        tr.prompt_ids = chat_ids(self.tok, msgs)
        ctx = list(tr.prompt_ids)
        for _ in range(self.max_turns):
            if len(ctx) >= self.max_context:
                tr.stop_reason = "length"
                break
            out = await self.engine.generate({"prompt_token_ids": [ctx], "sampling_params": self.sp})
            ids = out["response_ids"][0]
            lps = (out.get("response_logprobs") or [[0.0] * len(ids)])[0]
            tr.turns += 1
            tr.stop_reason = out["stop_reasons"][0]
            tr.response_ids += ids
            tr.loss_mask += [1] * len(ids)
            tr.logprobs += lps
            ctx += ids
            text = self.tok.decode(ids)
            fin = _FINISH.search(text)
            if fin:
                tr.finish = fin.group(1).strip()
                break
            call = _TOOL.search(text)
            if call is None:
                obs = "No tool call or <finish> found."
            else:
                try:
                    req = json.loads(call.group(1))
                    res = self.tools.call(req.get("name", ""), req.get("arguments") or {})
                    tr.tool_calls.append(req.get("name", ""))
                except json.JSONDecodeError as e:
                    res = {"error": f"tool call is not valid JSON: {e}"}
                obs = json.dumps(res, default=str)[:4000]
            obs_ids = chat_ids_continuation(self.tok, [{"role": "tool", "content": obs}])
            tr.response_ids += obs_ids
            tr.loss_mask += [0] * len(obs_ids)
            tr.logprobs += [0.0] * len(obs_ids)
            ctx += obs_ids
        tr.reward = float(judge(tr.finish, tr))
        tr.seconds = time.time() - t0
        return tr


class AsyncDispatcher:
    """Run ``agent.run`` over many instances with at most ``max_parallel`` trajectories alive."""

    def __init__(self, agent: ReActAgent, max_parallel: int = 64):
        self.agent, self.sem = agent, None
        self.max_parallel = max_parallel

    async def run(self, instances: list[dict], n_samples: int = 1) -> list[Trajectory]:
        self.sem = asyncio.Semaphore(self.max_parallel)

        async def one(inst, k):
            async with self.sem:
                return await self.agent.run(f"{inst['id']}#{k}", inst["task"], inst["judge"])

        return list(await asyncio.gather(*[one(i, k) for i in instances for k in range(n_samples)]))


def to_generator_output(trajs: list[Trajectory]) -> tuple[dict, list[str]]:
    """Trajectories -> (GeneratorOutput, uids) as ``RayPPOTrainer.convert_to_training_input`` expects; the outcome reward
    sits on the last MODEL token of each trajectory."""
    rewards = []
    for t in trajs:
        r = [0.0] * len(t.response_ids)
        last = max((i for i, m in enumerate(t.loss_mask) if m), default=None)
        if last is not None:
            r[last] = t.reward
        rewards.append(r)
    go = {"prompt_token_ids": [t.prompt_ids for t in trajs], "response_ids": [t.response_ids for t in trajs], "rewards": rewards,
          "loss_masks": [t.loss_mask for t in trajs], "rollout_logprobs": [t.logprobs for t in trajs],
          "stop_reasons": [t.stop_reason for t in trajs], "rollout_metrics": {"agent/avg_turns": sum(t.turns for t in trajs) / max(1, len(trajs)),
                                                                             "agent/finish_rate": sum(t.finish is not None for t in trajs) / max(1, len(trajs))}}
    return go, [t.instance_id.split("#")[0] for t in trajs]
