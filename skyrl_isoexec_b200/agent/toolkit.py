"""Tools for the agents (reference: skyrl-agent/skyrl_agent/tools/{base,finish,em_finish,local_search,sandbox_fusion,cache,
next_memagent}.py): a tool is a name, a description, a JSON schema of its parameters and ``call(params, **context)``.

* ``register_tool(name)`` / ``TOOL_REGISTRY`` / ``make_tools(names, **kw)``: tools are looked up by name from a run's config;
* ``BaseTool.schema()``                       the OpenAI function-tool entry (what ``agent/function_calling.py`` prints);
* ``BaseTool.checked(params)``                parameters as a dict (JSON text is accepted), required ones present;
* ``FinishTool``                              ends a trajectory with an answer;
* ``EMFinishTool``                            the same, and scores the answer by normalised exact match against the
                                              trajectory's ground truth (``context["ground_truth"]``);
* ``LocalSearchTool``                         BM25 over a corpus given at construction (``gym/tools.py``), or a retrieval
                                              server (``gym/envs/search.py::RemoteSearch``), through a ``ToolCache``;
* ``PythonSandboxTool``                       a fresh interpreter with a time limit per call (``code_interpreter``);
* ``MemoryTool``                              a scratch memory that persists over the turns of ONE trajectory: the agent
                                              overwrites it with what it wants to keep when its context is trimmed;
* ``ToolCache``                               thread-safe LRU with a time-to-live, keyed by tool name and arguments, with
                                              hit / miss counters; optional JSON file persistence.
"""

from __future__ import annotations

import json
import os
import threading
import time
from collections import OrderedDict

from ..gym.tools import PythonToolGroup, SearchToolGroup

TOOL_REGISTRY: dict[str, type] = {}


class ToolError(Exception):
    """A tool failed in a way the model should read about (bad arguments, a service that is down)."""


def register_tool(name: str, allow_overwrite: bool = False):
    def deco(cls):
        if name in TOOL_REGISTRY and not allow_overwrite:
            raise ValueError(f"tool {name!r} is registered already")
        cls.name = name
        TOOL_REGISTRY[name] = cls
        return cls

    return deco


def make_tools(names: list[str], **kwargs) -> dict:
    """{name: tool instance}; ``kwargs[name]`` (a dict) goes to that tool's constructor."""
    out = {}
    for n in names:
        if n not in TOOL_REGISTRY:
            raise KeyError(f"unknown tool {n!r}; registered: {sorted(TOOL_REGISTRY)}")
        out[n] = TOOL_REGISTRY[n](**(kwargs.get(n) or {}))
    return out


class BaseTool:
    name = ""
    description = ""
    parameters: dict = {"type": "object", "properties": {}, "required": []}
    ends_trajectory = False

    def schema(self) -> dict:
        return {"type": "function", "function": {"name": self.name, "description": self.description, "parameters": self.parameters}}

    def checked(self, params) -> dict:
        if isinstance(params, str):
            try:
                params = json.loads(params) if params.strip() else {}
            except json.JSONDecodeError:
                raise ToolError(f"the arguments of {self.name} are not valid JSON") from None
        if not isinstance(params, dict):
            raise ToolError(f"the arguments of {self.name} must be an object")
        missing = [k for k in self.parameters.get("required", []) if k not in params]
        if missing:
            raise ToolError(f"{self.name}: missing required parameters {missing}")
        return params

    def call(self, params, **context):
        raise NotImplementedError


@register_tool("finish")
class FinishTool(BaseTool):
    description = "Finish the task and give the final answer."
    parameters = {"type": "object", "properties": {"answer": {"type": "string", "description": "the final answer"}}, "required": ["answer"]}
    ends_trajectory = True

    def call(self, params, **context):
        return {"answer": str(self.checked(params)["answer"])}


def normalize_answer(s: str) -> str:
    from ..gym.envs.search import normalize_answer as norm

    return norm(str(s))


@register_tool("em_finish")
class EMFinishTool(FinishTool):
    description = "Finish the task with a short final answer; it is compared with the reference answer."

    def call(self, params, **context):
        ans = str(self.checked(params)["answer"])
        gt = context.get("ground_truth")
        golds = [gt] if isinstance(gt, (str, int, float)) else list(gt or [])
        hit = any(normalize_answer(g) == normalize_answer(ans) for g in golds)
        return {"answer": ans, "reward": 1.0 if hit else 0.0}


class ToolCache:
    def __init__(self, capacity: int = 4096, ttl_s: float | None = None, path: str = ""):
        self.capacity, self.ttl_s, self.path = capacity, ttl_s, path
        self._d: OrderedDict[str, tuple[float, object]] = OrderedDict()
        self._lock = threading.Lock()
        self.hits = self.misses = 0
        if path and os.path.exists(path):
            with open(path, encoding="utf-8") as f:
                for k, (t, v) in json.load(f).items():
                    self._d[k] = (t, v)

    @staticmethod
    def key(tool: str, params: dict) -> str:
        return tool + ":" + json.dumps(params, sort_keys=True, default=str)

    def get(self, key: str):
        with self._lock:
            e = self._d.get(key)
            if e is None or (self.ttl_s is not None and time.time() - e[0] > self.ttl_s):
                self._d.pop(key, None)
                self.misses += 1
                return None
            self._d.move_to_end(key)
            self.hits += 1
            return e[1]

    def put(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = (time.time(), value)
            self._d.move_to_end(key)
            while len(self._d) > self.capacity:
                self._d.popitem(last=False)

    def through(self, tool: str, params: dict, fn):
        k = self.key(tool, params)
        v = self.get(k)
        if v is None:
            v = fn()
            self.put(k, v)
        return v

    def save(self) -> None:
        if self.path:
            with self._lock:
                tmp = self.path + ".tmp"
                with open(tmp, "w", encoding="utf-8") as f:
                    json.dump(self._d, f)
                os.replace(tmp, self.path)

    def stats(self) -> dict:
        return {"entries": len(self._d), "hits": self.hits, "misses": self.misses}


@register_tool("local_search")
class LocalSearchTool(BaseTool):
    description = "Search the document collection and return the best matching passages."
    parameters = {"type": "object", "properties": {"query": {"type": "string", "description": "what to look for"},
                                                   "topk": {"type": "integer", "description": "how many passages (default 3)"}},
                  "required": ["query"]}

    def __init__(self, corpus: list[str] | None = None, search_url: str = "", topk: int = 3, cache: ToolCache | None = None, **remote_kw):
        self.topk, self.cache = topk, cache if cache is not None else ToolCache()
        if search_url:
            from ..gym.envs.search import RemoteSearch

            self.remote, self.index = RemoteSearch(search_url, topk, **remote_kw), None
        else:
            self.remote, self.index = None, SearchToolGroup(corpus or [])

    def call(self, params, **context):
        p = self.checked(params)
        query, k = str(p["query"]).strip(), int(p.get("topk") or self.topk)
        if not query:
            raise ToolError("local_search: the query is empty")

        def run():
            if self.remote is not None:
                self.remote.topk = k
                text, meta = self.remote.search(query)
                if meta.get("status") == "api_error":
                    raise ToolError(text)
                return text
            hits = self.index.search(query, k)
            return "".join(f"Doc {i + 1}: {h['text'].strip()}\n" for i, h in enumerate(hits)) or "No search results found."

        return self.cache.through(self.name, {"query": query, "topk": k}, run)


@register_tool("code_interpreter")
class PythonSandboxTool(BaseTool):
    description = "Run Python code in a fresh interpreter and return what it prints."
    parameters = {"type": "object", "properties": {"code": {"type": "string", "description": "the program"},
                                                   "stdin": {"type": "string", "description": "text for standard input"}},
                  "required": ["code"]}

    def __init__(self, timeout_s: float = 10.0, max_output_chars: int = 4000):
        self.py, self.max_out = PythonToolGroup(timeout_s), max_output_chars

    def call(self, params, **context):
        p = self.checked(params)
        r = self.py.python(str(p["code"]), stdin=str(p.get("stdin") or ""))
        text = r["stdout"] + (("\n[stderr]\n" + r["stderr"]) if r["stderr"] else "")
        return (text.strip() or "(no output)")[-self.max_out:]


@register_tool("memory")
class MemoryTool(BaseTool):
    description = ("Overwrite your scratch memory with the notes you want to keep. Earlier turns may be dropped from the context; "
                   "the memory is shown to you again at the start of every turn.")
    parameters = {"type": "object", "properties": {"notes": {"type": "string", "description": "the new content of the memory"}},
                  "required": ["notes"]}

    def __init__(self, max_chars: int = 4000):
        self.max_chars = max_chars

    def call(self, params, **context):
        notes = str(self.checked(params)["notes"])[:self.max_chars]
        state = context.get("state")
        if state is not None:
            state["memory"] = notes
        return f"Memory updated ({len(notes)} characters)."
