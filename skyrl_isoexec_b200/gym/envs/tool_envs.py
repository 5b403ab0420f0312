"""Multi-turn tool environments: text-to-SQL, search-augmented QA (plain and code search) and code generation
scored by tests (reference: skyrl-gym/skyrl_gym/envs/{sql,search,searchcode,lcb}/).

Protocol of a turn: the model either calls a tool, ``<sql>...</sql>`` / ``<search>...</search>`` /
``<python>...</python>``, and gets ``<observation>...</observation>`` back, or commits with
``<solution>...</solution>`` (SQL), ``<answer>...</answer>`` (QA) or a final fenced code block (code). The episode
ends on the commit or when ``max_turns`` is used up; reward is 1 for a correct commit, else 0 (with an optional
small format reward).
"""

from __future__ import annotations

import json
import re

from ..core import BaseTextEnv, register
from ..tools import PythonToolGroup, SearchToolGroup, SQLToolGroup


def _tag(text: str, name: str) -> str | None:
    m = re.findall(rf"<{name}>(.*?)</{name}>", text, flags=re.S)
    return m[-1].strip() if m else None


def _obs(s) -> list:
    return [{"role": "user", "content": f"<observation>{s}</observation>"}]


class SQLEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        self.max_turns = int(self.extras.get("max_turns", 5))
        spec = self.extras.get("reward_spec") or {}
        self.gold_sql = spec["ground_truth"]
        self.init_tool_groups([SQLToolGroup(self.extras.get("schema_sql", ""))])

    def step(self, action: str):
        self.turns += 1
        sol = _tag(action, "solution")
        if sol is not None:
            got = self._execute_tool("sql", "sql", [sol])
            want = self._execute_tool("sql", "sql", [self.gold_sql])
            ok = got["ok"] and want["ok"] and sorted(map(tuple, got["rows"])) == sorted(map(tuple, want["rows"]))
            return {"observations": [], "reward": 1.0 if ok else 0.0, "done": True, "metadata": {"executed": got["ok"]}}
        q = _tag(action, "sql")
        done = self.turns >= self.max_turns
        if q is None:
            return {"observations": [] if done else _obs("no <sql> or <solution> tag found"), "reward": 0.0, "done": done, "metadata": {}}
        res = self._execute_tool("sql", "sql", [q])
        text = json.dumps(res["rows"][:20]) if res["ok"] else "error: " + res["error"]
        return {"observations": [] if done else _obs(text), "reward": 0.0, "done": done, "metadata": {}}


def _norm_answer(s: str) -> str:
    s = re.sub(r"\b(a|an|the)\b", " ", s.lower())
    return " ".join(re.sub(r"[^a-z0-9 ]", " ", s).split())


class SearchEnv(BaseTextEnv):
    tool_tag = "search"

    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        self.max_turns = int(self.extras.get("max_turns", 4))
        spec = self.extras.get("reward_spec") or {}
        gt = spec["ground_truth"]
        self.targets = [gt] if isinstance(gt, str) else list(gt.get("target", gt) if isinstance(gt, dict) else gt)
        self.init_tool_groups([SearchToolGroup(self.extras.get("corpus") or self.env_config.get("corpus") or [])])
        self.topk = int(self.env_config.get("topk", 3))

    def step(self, action: str):
        self.turns += 1
        ans = _tag(action, "answer")
        if ans is not None:
            ok = any(_norm_answer(ans) == _norm_answer(t) for t in self.targets)
            return {"observations": [], "reward": 1.0 if ok else 0.0, "done": True, "metadata": {}}
        q = _tag(action, self.tool_tag)
        done = self.turns >= self.max_turns
        if q is None:
            return {"observations": [] if done else _obs("use <search>query</search> or <answer>...</answer>"), "reward": 0.0, "done": done, "metadata": {}}
        hits = self._execute_tool("search", "search", [q, self.topk])
        text = "\n".join(f"Doc {i + 1}: {h['text']}" for i, h in enumerate(hits)) or "no results"
        return {"observations": [] if done else _obs(text), "reward": 0.0, "done": done, "metadata": {"hits": len(hits)}}


class SearchCodeEnv(SearchEnv):
    """Search over a code corpus; the commit is a code block judged by tests, like ``LCBEnv``."""

    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        self.tests = (self.extras.get("reward_spec") or {}).get("tests") or []
        self.py = PythonToolGroup(float(self.env_config.get("timeout_s", 5)))

    def step(self, action: str):
        code = extract_code(action)
        if code is not None and _tag(action, self.tool_tag) is None:
            self.turns += 1
            return {"observations": [], "reward": run_tests(self.py, code, self.tests), "done": True, "metadata": {}}
        return super().step(action)


def extract_code(text: str) -> str | None:
    m = re.findall(r"```(?:python)?\n(.*?)```", text, flags=re.S)
    return m[-1] if m else None


def run_tests(py: PythonToolGroup, code: str, tests: list[dict]) -> float:
    """tests: [{"input": stdin text, "output": expected stdout}] (stdin/stdout style, as LiveCodeBench) or
    [{"assert": python expression/statements appended to the code}]. Reward 1.0 only if all pass."""
    if not tests:
        return 0.0
    for t in tests:
        if "assert" in t:
            r = py.python(code + "\n" + t["assert"])
            if not r["ok"]:
                return 0.0
        else:
            r = py.python(code, stdin=t.get("input", ""))
            if not r["ok"] or r["stdout"].strip() != str(t.get("output", "")).strip():
                return 0.0
    return 1.0


class LCBEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        self.tests = (self.extras.get("reward_spec") or {}).get("ground_truth") or (self.extras.get("reward_spec") or {}).get("tests") or []
        if isinstance(self.tests, str):
            self.tests = json.loads(self.tests)
        self.py = PythonToolGroup(float(self.env_config.get("timeout_s", 5)))

    def step(self, action: str):
        code = extract_code(action)
        r = run_tests(self.py, code, self.tests) if code is not None else 0.0
        return {"observations": [], "reward": r, "done": True, "metadata": {"has_code": code is not None}}


register("sql", lambda c, e: SQLEnv(c, e))
register("search", lambda c, e: SearchEnv(c, e))
register("searchcode", lambda c, e: SearchCodeEnv(c, e))
register("lcb", lambda c, e: LCBEnv(c, e))
