"""REPL environment over a long context ("recursive language model" task family; reference:
skyrl-gym/skyrl_gym/envs/rlm/env.py:180-405 and its persistent REPL, repl.py).

The query comes with a ``context`` that may be far longer than what the model wants to read at once. The model does
not get it in the prompt; it gets a Python REPL in which ``context`` is a variable and works on it in turns:

    ```repl
    print(len(context)); hits = [l for l in context.splitlines() if "invoice" in l]; print(hits[:5])
    ```

Every fenced ``repl`` block is executed and what it printed comes back as the observation; variables persist between
blocks, ``SHOW_VARS()`` lists them. The episode ends when the model writes ``FINAL(answer)`` or ``FINAL_VAR(name)``
(the value of a REPL variable), or when ``max_turns`` is used up. Reward: 1 for an answer equal to the ground truth
after normalisation (exact match, or containment when ``reward_spec.match == "contains"``), else 0.

Two REPLs:

* isolated (default): persistence without a long-lived interpreter: blocks that ran cleanly are kept and replayed silently
  in a fresh, isolated interpreter before the next block (``gym/tools.py::PythonToolGroup``: ``python -I``, time limit),
  with the context handed over on stdin;
* in-process (``extras.lm_callback`` / ``extras.subcall_fn`` / ``extras.tools`` given, or ``env_config.repl =
  "inprocess"``): ``gym/repl.py::PersistentREPL``, whose blocks can call ``llm_query`` / ``llm_query_batched`` (plain
  completions of the policy) and ``rlm_query`` / ``rlm_query_batched`` (a child agent with its own REPL on a sub-task and
  its own ``context``), plus task tools. Here ``FINAL_VAR(name)`` may also be called INSIDE a block: the episode ends with
  that variable's value.

Subclasses adapt a task by overriding ``get_reward(final_answer)``, ``system_prompt()`` and ``repl_tools()``. The context is
``extras.context``, else ``extras.extra_info.context_text`` (a JSON object there becomes a dict, e.g. one entry per
document), else the prompt's own text; the system message states its type, total size and the sizes of its parts.
"""

from __future__ import annotations

import json
import re

from ..core import BaseTextEnv, register
from ..tools import PythonToolGroup

_BLOCK = re.compile(r"```repl\s*\n(.*?)```", re.S)
_FINAL = re.compile(r"FINAL\((.*)\)", re.S)
_FINAL_VAR = re.compile(r"FINAL_VAR\(\s*([A-Za-z_][A-Za-z0-9_]*)\s*\)")

_PRELUDE = (
    "import sys as _sys, io as _io, json as _json\n"
    "context = _json.loads(_sys.stdin.read())\n"
    "def SHOW_VARS():\n"
    "    return sorted(k for k in globals() if not k.startswith('_') and k not in ('context', 'SHOW_VARS'))\n"
)
_SILENT = "_o = _sys.stdout\n_sys.stdout = _io.StringIO()\n{body}\n_sys.stdout = _o\n"

SYSTEM_PROMPT = (
    "Answer the query using the REPL. The variable `context` holds the material you need; it may be long, so inspect and "
    "filter it with code instead of printing all of it. Run code by writing a fenced block that starts with ```repl. "
    "Variables persist between blocks; SHOW_VARS() lists them. Finish with FINAL(your answer) or, for a value you built in "
    "the REPL, FINAL_VAR(variable_name) in a separate message after the block that created it."
)


def _norm(s) -> str:
    return " ".join(re.sub(r"[^a-z0-9. ]", " ", str(s).lower()).split())


LM_TOOLS_PROMPT = (
    " Inside a block you can also call llm_query(prompt) / llm_query_batched(prompts) for a plain completion, and "
    "rlm_query(prompt, context=...) / rlm_query_batched(prompts, context_list=...) to hand a sub-task with its own context to a "
    "child agent that has a REPL of its own; FINAL_VAR(name) inside a block ends the episode with that variable."
)


def describe_context(ctx) -> str:
    """Type, total size and the sizes of the parts of a context (what the model is told instead of the context itself)."""
    if isinstance(ctx, dict):
        sizes = [len(str(v)) for v in ctx.values()]
        return f"`context` is a dict with {len(ctx)} entries and {sum(sizes)} characters in total (entry sizes: {_sizes(sizes)})."
    if isinstance(ctx, (list, tuple)):
        sizes = [len(str(v)) for v in ctx]
        return f"`context` is a {type(ctx).__name__} of length {len(ctx)} with {sum(sizes)} characters in total (item sizes: {_sizes(sizes)})."
    n = len(ctx) if hasattr(ctx, "__len__") else 0
    return f"`context` is a {type(ctx).__name__} of length {n}."


def _sizes(sizes: list[int], show: int = 20) -> str:
    return ", ".join(map(str, sizes[:show])) + (f", ... {len(sizes) - show} more" if len(sizes) > show else "")


class RLMEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        ex = self.extras
        self.max_turns = int(ex.get("max_turns", 8))
        spec = ex.get("reward_spec") or {}
        self.truth = spec.get("ground_truth")
        self.match = spec.get("match", "exact")
        self.context = ex.get("context")
        if self.context is None:
            self.context = (ex.get("extra_info") or {}).get("context_text")
            if isinstance(self.context, str):
                try:
                    decoded = json.loads(self.context)
                    if isinstance(decoded, dict):
                        self.context = decoded
                except ValueError:
                    pass
        self.lm_callback, self.subcall_fn = ex.get("lm_callback"), ex.get("subcall_fn")
        self.inprocess = bool(self.lm_callback or self.subcall_fn or ex.get("tools") or self.env_config.get("repl") == "inprocess")
        self.timeout_s = float(ex.get("timeout_s", ex.get("repl_timeout", 180.0 if self.inprocess else 5.0)))
        self.python = PythonToolGroup(timeout_s=self.timeout_s)
        self.repl = None
        self.kept: list[str] = []                     # isolated mode: blocks that ran without an error, in order
        self.blocks_run = self.errors = 0

    # ---- hooks for task-specific subclasses
    def get_reward(self, final_answer) -> float:
        """Score a final answer (called only when there is one; the turn limit scores 0 without it)."""
        if self.truth is None:
            return 1.0 if final_answer else 0.0
        a, t = _norm(final_answer), _norm(self.truth)
        return 1.0 if (a == t or (self.match == "contains" and t and t in a)) else 0.0

    def system_prompt(self) -> str:
        return SYSTEM_PROMPT + (LM_TOOLS_PROMPT if self.lm_callback is not None else "")

    def repl_tools(self) -> dict:
        """``{name: callable or value}`` put into the in-process REPL; called after the context is known."""
        return dict(self.extras.get("tools") or {})

    # ---- protocol
    def init(self, prompt):
        msgs = list(prompt) if isinstance(prompt, list) else [{"role": "user", "content": str(prompt)}]
        if self.context is None:
            self.context = "\n".join(m["content"] for m in msgs if isinstance(m.get("content"), str))
        size = len(self.context) if hasattr(self.context, "__len__") else 0
        tools = self.repl_tools() if self.inprocess else {}
        if self.inprocess:
            from ..repl import PersistentREPL

            self.repl = PersistentREPL(self.timeout_s, tools, self.lm_callback, self.subcall_fn)
            self.repl.set_context(self.context)
            self.repl._scaffold["FINAL_VAR"] = self.repl.ns["FINAL_VAR"] = self._final_var_in_block
        extra = ""
        if tools:
            extra = " Task tools in the REPL: " + ", ".join(
                f"{k}{'()' if callable(v) else ''}" + (f" - {v.__doc__.strip().splitlines()[0]}" if callable(v) and v.__doc__ else "")
                for k, v in tools.items()) + "."
        head = {"role": "system", "content": self.system_prompt() + extra + "\n" + describe_context(self.context)}
        return [head] + [m for m in msgs if m.get("role") != "system"], {"context_len": size}

    def _run(self, code: str) -> dict:
        if self.repl is not None:
            r = self.repl.execute(code)
            return {"ok": r.ok, "stdout": r.stdout, "stderr": r.stderr}
        silent = "".join(_SILENT.format(body=b) for b in self.kept)
        return self.python.python(_PRELUDE + silent + code, stdin=json.dumps(self.context))

    def _done(self, answer, how: str):
        meta = {"final": None if answer is None else str(answer), "how": how}
        if isinstance(self.extras.get("result_box"), dict):          # a parent trajectory reads its child's answer here
            self.extras["result_box"].update(meta)
        return {"observations": [], "reward": self.get_reward(answer) if answer is not None else 0.0, "done": True, "metadata": meta}

    def step(self, action: str):
        self.turns += 1
        block = _BLOCK.search(action)
        if block is None:                                  # a final answer only counts in a message without code
            var = _FINAL_VAR.search(action)
            if var is not None and self.repl is not None:
                text = self.repl.final_var(var.group(1))
                if not text.startswith("Error: variable"):
                    return self._done(text, "FINAL_VAR")
                obs = "FINAL_VAR failed: " + text
            elif var is not None:
                res = self._run(f"print(_json.dumps({var.group(1)}, default=str))")
                if res["ok"]:
                    try:
                        return self._done(json.loads(res["stdout"].strip().splitlines()[-1]), "FINAL_VAR")
                    except (ValueError, IndexError):
                        return self._done(res["stdout"].strip(), "FINAL_VAR")
                obs = f"FINAL_VAR failed: {res['stderr'].strip().splitlines()[-1] if res['stderr'].strip() else 'no such variable'}"
            else:
                fin = _FINAL.search(action)
                if fin is not None:
                    return self._done(fin.group(1).strip(), "FINAL")
                obs = "No ```repl block and no FINAL(...) found."
        else:
            code = block.group(1)
            if self.repl is not None:
                self.repl.ns.pop("_final_answer", None)
            res = self._run(code)
            self.blocks_run += 1
            if self.repl is not None and "_final_answer" in self.repl.ns:
                return self._done(self.repl.ns.pop("_final_answer"), "FINAL_VAR in block")
            if res["ok"]:
                self.kept.append(code)
            else:
                self.errors += 1
            obs = (res["stdout"] or "") + (("\n[stderr]\n" + res["stderr"]) if res["stderr"] else "")
            obs = obs[-4000:] or "(no output)"
        if self.turns >= self.max_turns:
            return self._done(None, "turn limit")
        return {"observations": [{"role": "user", "content": f"<observation>{obs}</observation>"}], "reward": 0.0, "done": False,
                "metadata": {}}

    def _final_var_in_block(self, name):
        text = self.repl.final_var(name)
        if not text.startswith("Error: variable"):
            self.repl.ns["_final_answer"] = text
        return text

    def get_metrics(self) -> dict:
        out = {"rlm/turns": self.turns, "rlm/blocks_run": self.blocks_run, "rlm/block_errors": self.errors}
        if self.repl is not None:
            out.update({"rlm/lm_calls": self.repl.lm_calls, "rlm/child_calls": self.repl.child_calls})
        return out


register("rlm", lambda c, e: RLMEnv(c, e))
