"""Search-augmented question answering, plain and with code (reference: skyrl-gym/skyrl_gym/envs/search/{env,utils}.py,
envs/searchcode/env.py, tools/search.py).

A turn is either ``<search>query</search>``, answered with ``<information>Doc 1: ... Doc k: ...</information>``, or the
commit ``<answer>...</answer>``; the episode ends on the commit or when the turns are used up. The reward is computed on
the WHOLE transcript: the last ``<answer>`` block is normalised (lower case, punctuation and articles removed, whitespace
folded) and must equal one of ``reward_spec.ground_truth.target`` (exact match), or contain one with
``env_config.match = "substring"``; an answer that is there but wrong scores ``env_config.format_score`` (default 0).

Where the documents come from:

* ``env_config.search_url`` (the reference's mode): ``POST {"query", "topk", "return_scores"}`` to a retrieval server that
  answers ``{"result": [[{"document": {"contents": ...}, "score": ...}, ...]]}``. Server errors (500 / 502 / 503 / 504),
  refused connections and timeouts are retried with a delay that grows by ``retry_delay_s`` per attempt, up to
  ``max_retries``; any other failure is reported at once. A failed search is an observation, not an exception: the model
  reads ``Search error: ...`` and the episode goes on.
* otherwise a BM25 index over ``extras.corpus`` / ``env_config.corpus`` in this process (``gym/tools.py``); the same index
  can be put behind HTTP with ``python -m skyrl_isoexec_b200.gym.retrieval_server``.

``searchcode`` adds a ``<python>...</python>`` tool (a fresh interpreter with a time limit) beside the search tool.
"""

from __future__ import annotations

import json
import re
import string
import time
import urllib.error
import urllib.request

from ..core import BaseTextEnv, register
from ..tools import PythonToolGroup, SearchToolGroup

_RETRY_STATUS = (500, 502, 503, 504)


def normalize_answer(s: str) -> str:
    s = "".join(ch for ch in s.lower() if ch not in set(string.punctuation))
    return " ".join(re.sub(r"\b(a|an|the)\b", " ", s).split())


def last_answer(transcript: str) -> str | None:
    m = re.findall(r"<answer>(.*?)</answer>", transcript, flags=re.S)
    return m[-1].strip() if m else None


def _targets(ground_truth) -> list[str]:
    t = ground_truth.get("target", ground_truth) if isinstance(ground_truth, dict) else ground_truth
    if hasattr(t, "tolist"):
        t = t.tolist()
    return [str(t)] if isinstance(t, (str, int, float)) else [str(x) for x in t]


def compute_score(transcript: str, ground_truth, match: str = "exact", format_score: float = 0.0, score: float = 1.0) -> float:
    ans = last_answer(transcript)
    if ans is None:
        return 0.0
    a = normalize_answer(ans)
    golds = [normalize_answer(g) for g in _targets(ground_truth)]
    hit = any(g == a for g in golds) if match == "exact" else any(g and g in a for g in golds)
    return score if hit else format_score


class RemoteSearch:
    """Client of a retrieval server. ``search`` never raises: it returns (text for the model, metadata)."""

    name = "search"

    def __init__(self, url: str, topk: int = 3, timeout_s: float = 30.0, max_retries: int = 10, retry_delay_s: float = 1.0):
        self.url, self.topk, self.timeout_s, self.max_retries, self.retry_delay_s = url, topk, timeout_s, max_retries, retry_delay_s
        self.attempts = 0

    def tools(self):
        return ["search"]

    def _call(self, query: str):
        body = json.dumps({"query": query, "topk": self.topk, "return_scores": True}).encode()
        last = None
        for attempt in range(self.max_retries):
            self.attempts += 1
            try:
                req = urllib.request.Request(self.url, data=body, headers={"Content-Type": "application/json", "Accept": "application/json"})
                with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
                    return json.loads(r.read()), None
            except urllib.error.HTTPError as e:
                last = f"server error ({e.code})"
                if e.code not in _RETRY_STATUS:
                    return None, f"request error: HTTP {e.code}"
            except (urllib.error.URLError, ConnectionError, TimeoutError) as e:
                last = f"connection error: {getattr(e, 'reason', e)}"
            except json.JSONDecodeError as e:
                return None, f"the server's answer is not JSON: {e}"
            if attempt < self.max_retries - 1:
                time.sleep(self.retry_delay_s * (attempt + 1))
        return None, f"{last} after {self.max_retries} attempts"

    def search(self, query: str | None):
        if query is None:
            return "", {"status": "no_query"}
        query = query.strip()
        resp, err = self._call(query)
        if err:
            return f"Search error: {err}", {"status": "api_error", "query": query, "error": err}
        groups = resp.get("result") or []
        if not groups or not any(groups):
            return "No search results found.", {"status": "no_results", "query": query, "total_results": 0}
        texts = ["".join(f"Doc {i + 1}: {d['document']['contents'].strip()}\n" for i, d in enumerate(g)) for g in groups]
        return "\n---\n".join(texts), {"status": "success", "query": query, "total_results": sum(len(g) for g in groups)}


class LocalSearch(SearchToolGroup):
    """The in-process BM25 index behind the same ``search(query) -> (text, metadata)`` call."""

    def __init__(self, corpus: list[str], topk: int = 3):
        super().__init__(corpus)
        self.topk = topk

    def search(self, query: str | None, topk: int | None = None):
        if query is None:
            return "", {"status": "no_query"}
        hits = super().search(query.strip(), topk or self.topk)
        if not hits:
            return "No search results found.", {"status": "no_results", "query": query, "total_results": 0}
        return "".join(f"Doc {i + 1}: {h['text'].strip()}\n" for i, h in enumerate(hits)), \
            {"status": "success", "query": query, "total_results": len(hits)}


class SearchEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        spec = self.extras.get("reward_spec") or {}
        if "ground_truth" not in spec:
            raise KeyError("the search environment needs reward_spec.ground_truth")
        self.ground_truth = spec["ground_truth"]
        self.max_turns = int(self.extras.get("max_turns", 2))
        c = self.env_config
        if c.get("search_url"):
            self.tool = RemoteSearch(c["search_url"], int(c.get("topk", 3)), float(c.get("timeout", 30)),
                                     int(c.get("max_retries", 10)), float(c.get("retry_delay_s", 1.0)))
        else:
            self.tool = LocalSearch(self.extras.get("corpus") or c.get("corpus") or [], int(c.get("topk", 3)))
        self.init_tool_groups([self.tool])
        self.match = c.get("match", "exact")
        self.format_score = float(c.get("format_score", 0.0))
        self.chat_history: list[dict] = []
        self.searches = self.failed = 0

    # one tool call per turn: (tool name, its input) or (None, None)
    def _parse(self, action: str):
        m = re.search(r"<search>(.*?)</search>", action, re.S)
        return ("search", m.group(1)) if m else (None, None)

    def _run_tool(self, tool: str, arg: str) -> tuple[str, dict]:
        self.searches += 1
        text, meta = self.tool.search(arg)
        self.failed += meta.get("status") == "api_error"
        return "\n<information>" + text + "</information>\n", meta

    def _done(self, action: str) -> bool:
        return self.turns >= self.max_turns or ("<answer>" in action and "</answer>" in action)

    def step(self, action: str):
        self.turns += 1
        self.chat_history.append({"role": "assistant", "content": action})
        if self._done(action):
            transcript = "".join(m["content"] for m in self.chat_history)
            r = compute_score(transcript, self.ground_truth, self.match, self.format_score)
            return {"observations": [], "reward": r, "done": True, "metadata": {}}
        tool, arg = self._parse(action)
        if tool is None:
            return {"observations": [], "reward": 0.0, "done": False, "metadata": {"tool_name": None}}   # nothing to answer: the model goes on
        text, meta = self._run_tool(tool, arg)
        obs = {"role": "user", "content": text}
        self.chat_history.append(obs)
        return {"observations": [obs], "reward": 0.0, "done": False, "metadata": dict(meta, tool_group=self.tool.name, tool_name=tool, tool_input=arg)}

    def get_metrics(self) -> dict:
        return {"turns": self.turns, "searches": self.searches, "failed_searches": self.failed}


class SearchCodeEnv(SearchEnv):
    """``<search>`` and ``<python>`` tools; the first tool tag of a turn is the one that runs."""

    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        self.py = PythonToolGroup(float(self.env_config.get("python_timeout_s", 10)))
        self.init_tool_groups([self.tool, self.py])
        self.runs = 0

    def _parse(self, action: str):
        found = [(m.start(), name, m.group(1)) for name in ("search", "python")
                 for m in [re.search(rf"<{name}>(.*?)</{name}>", action, re.S)] if m]
        if not found:
            return None, None
        _, name, arg = min(found)
        return name, arg

    def _run_tool(self, tool: str, arg: str) -> tuple[str, dict]:
        if tool == "search":
            return super()._run_tool(tool, arg)
        self.runs += 1
        r = self.py.python(arg)
        text = r["stdout"] if r["ok"] else (r["stdout"] + r["stderr"])
        return "\n<information>" + (text.strip() or "(no output)") + "</information>\n", {"status": "success" if r["ok"] else "python_error"}

    def get_metrics(self) -> dict:
        return dict(super().get_metrics(), python_runs=self.runs)


register("search", lambda c, e: SearchEnv(c, e))
register("searchcode", lambda c, e: SearchCodeEnv(c, e))
