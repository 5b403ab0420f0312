"""Tasks and the config-driven runner (reference: skyrl-agent/skyrl_agent/tasks/{base,general_react}/, auto.py
``AutoAgentRunner``, config/configuration_utils.py).

A TASK turns a dataset row into an instruction for the agent and scores what the agent answered:

    get_instruction(row) -> str          evaluate(answer, row, trajectory) -> float
    ground_truth(row)                    (what ``em_finish`` compares against)

``GeneralReactTask`` covers the data sets of the reference's ``general_react`` task by a ``data_source`` switch: question
answering (exact match, substring or F1), math (boxed / ``Answer:`` expressions) and code (tests run in the guarded grader).

``AutoAgentRunner.from_config(cfg, engine, tokenizer)`` builds agent, tools, task and dispatch from one mapping (YAML file or
dict):

    agent: {type: function_call | react | codeact, max_turns: 8, max_context: 8192, sampling_params: {...}}
    tools: [local_search, code_interpreter, em_finish]      tool_kwargs: {local_search: {corpus: [...]}}
    task:  {type: general_react, metric: em}
    dispatcher: {max_parallel: 64, n_samples: 4}

and ``run(rows)`` returns ``(GeneratorOutput, uids)`` for the trainer (``agent/react.py::to_generator_output``), every
trajectory segment a row.
"""

from __future__ import annotations

import asyncio

from . import verifiers as V
from .fc_agent import FunctionCallAgent
from .react import Trajectory, to_generator_output
from .toolkit import make_tools

TASKS: dict[str, type] = {}


def register_task(name: str):
    def deco(cls):
        TASKS[name] = cls
        return cls

    return deco


class BaseTask:
    def __init__(self, **cfg):
        self.cfg = cfg

    def get_instruction(self, row: dict) -> str:
        raise NotImplementedError

    def ground_truth(self, row: dict):
        return (row.get("reward_spec") or row.get("reward_model") or {}).get("ground_truth")

    def evaluate(self, answer, row: dict, trajectory: Trajectory | None = None) -> float:
        raise NotImplementedError


@register_task("general_react")
class GeneralReactTask(BaseTask):
    MATH = ("math", "aime", "gsm8k", "dapo")
    CODE = ("code", "lcb", "livecodebench", "codeforces", "taco")

    def get_instruction(self, row: dict) -> str:
        p = row.get("prompt") or row.get("question") or ""
        if isinstance(p, list):
            p = "\n".join(m["content"] for m in p if m.get("role") == "user" and isinstance(m.get("content"), str))
        return str(p)

    def kind(self, row: dict) -> str:
        src = str(row.get("data_source", self.cfg.get("data_source", "qa"))).lower()
        if any(k in src for k in self.MATH):
            return "math"
        if any(k in src for k in self.CODE):
            return "code"
        return "qa"

    def ground_truth(self, row: dict):
        gt = super().ground_truth(row)
        return gt.get("target", gt) if isinstance(gt, dict) and self.kind(row) == "qa" else gt

    def evaluate(self, answer, row: dict, trajectory: Trajectory | None = None) -> float:
        if answer is None:
            return 0.0
        gt, kind = self.ground_truth(row), self.kind(row)
        if kind == "math":
            text = answer if "\\boxed" in answer or "nswer" in answer else f"\\boxed{{{answer}}}"
            return V.math_reward(text, gt)
        if kind == "code":
            text = answer if "```" in answer else f"```python\n{answer}\n```"
            return V.code_reward(text, gt, int(self.cfg.get("timeout_s", 6)), bool(self.cfg.get("partial", False)))
        return V.qa_reward(answer, gt, self.cfg.get("metric", "em"))


class AutoAgentRunner:
    def __init__(self, agent, task: BaseTask, max_parallel: int = 64, n_samples: int = 1):
        self.agent, self.task, self.max_parallel, self.n_samples = agent, task, max_parallel, n_samples

    @classmethod
    def from_config(cls, cfg, engine, tokenizer) -> "AutoAgentRunner":
        if isinstance(cfg, str):
            import yaml

            with open(cfg, encoding="utf-8") as f:
                cfg = yaml.safe_load(f)
        a = dict(cfg.get("agent") or {})
        kind = a.pop("type", "function_call")
        t = dict(cfg.get("task") or {})
        task_type = t.pop("type", "general_react")
        if task_type not in TASKS:
            raise KeyError(f"unknown task {task_type!r}; registered: {sorted(TASKS)}")
        task = TASKS[task_type](**t)
        if kind == "function_call":
            tools = make_tools(list(cfg.get("tools") or ["finish"]), **(cfg.get("tool_kwargs") or {}))
            agent = FunctionCallAgent(engine, tokenizer, tools, **a)
        elif kind == "react":
            from .react import ReActAgent, ToolRegistry

            reg = ToolRegistry()
            for name, tool in make_tools([n for n in (cfg.get("tools") or []) if n not in ("finish", "em_finish")], **(cfg.get("tool_kwargs") or {})).items():
                reg.register(name, (lambda tool: lambda **kw: tool.call(kw))(tool), tool.description)
            agent = ReActAgent(engine, tokenizer, reg, **a)
        elif kind == "codeact":
            from .codeact import CodeActAgent

            agent = CodeActAgent(engine, tokenizer, **a)
        else:
            raise KeyError(f"unknown agent type {kind!r} (function_call | react | codeact)")
        d = cfg.get("dispatcher") or {}
        return cls(agent, task, int(d.get("max_parallel", 64)), int(d.get("n_samples", 1)))

    async def run_async(self, rows: list[dict]) -> list[Trajectory]:
        sem = asyncio.Semaphore(self.max_parallel)

        async def one(i, row, k):
            async with sem:
                uid = f"{row.get('id', row.get('uid', i))}#{k}"
                judge = lambda ans, tr, row=row: self.task.evaluate(ans, row, tr)
                if isinstance(self.agent, FunctionCallAgent):
                    return await self.agent.run(uid, self.task.get_instruction(row), judge, self.task.ground_truth(row))
                return [await self.agent.run(uid, self.task.get_instruction(row), judge)]

        per = await asyncio.gather(*[one(i, row, k) for i, row in enumerate(rows) for k in range(self.n_samples)])
        return [seg for segs in per for seg in segs]

    def run(self, rows: list[dict]):
        trajs = asyncio.run(self.run_async(rows))
        go, uids = to_generator_output(trajs)
        go["rollout_metrics"]["agent/segments_per_trajectory"] = len(trajs) / max(1, len(rows) * self.n_samples)
        go["rollout_metrics"]["agent/avg_reward"] = sum(t.reward for t in trajs) / max(1, len(trajs))
        return go, [u.split("@")[0] for u in uids]
