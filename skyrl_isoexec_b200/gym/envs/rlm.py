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

Persistence without a long-lived interpreter: blocks that ran cleanly are kept and replayed silently in a fresh,
isolated interpreter before the next block (``gym/tools.py::PythonToolGroup``: ``python -I``, time limit), with the
context handed over on stdin.
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


class RLMEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        self.max_turns = int(self.extras.get("max_turns", 8))
        spec = self.extras.get("reward_spec") or {}
        self.truth = spec.get("ground_truth")
        self.match = spec.get("match", "exact")
        self.context = self.extras.get("context", "")
        self.python = PythonToolGroup(timeout_s=float(self.extras.get("timeout_s", 5.0)))
        self.kept: list[str] = []                     # blocks that ran without an error, in order
        self.blocks_run = self.errors = 0

    # ---- protocol
    def init(self, prompt):
        msgs = list(prompt) if isinstance(prompt, list) else [{"role": "user", "content": str(prompt)}]
        kind = type(self.context).__name__
        size = len(self.context) if hasattr(self.context, "__len__") else 0
        head = {"role": "system", "content": SYSTEM_PROMPT + f"\n`context` is a {kind} of length {size}."}
        return [head] + [m for m in msgs if m.get("role") != "system"], {"context_len": size}

    def _run(self, code: str) -> dict:
        silent = "".join(_SILENT.format(body=b) for b in self.kept)
        return self.python.python(_PRELUDE + silent + code, stdin=json.dumps(self.context))

    def _reward(self, answer) -> float:
        if self.truth is None or answer is None:
            return 0.0
        a, t = _norm(answer), _norm(self.truth)
        return 1.0 if (a == t or (self.match == "contains" and t and t in a)) else 0.0

    def _done(self, answer, how: str):
        return {"observations": [], "reward": self._reward(answer), "done": True,
                "metadata": {"final": None if answer is None else str(answer), "how": how}}

    def step(self, action: str):
        self.turns += 1
        block = _BLOCK.search(action)
        if block is None:                                  # a final answer only counts in a message without code
            var = _FINAL_VAR.search(action)
            if var is not None:
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
            res = self._run(code)
            self.blocks_run += 1
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

    def get_metrics(self) -> dict:
        return {"rlm/turns": self.turns, "rlm/blocks_run": self.blocks_run, "rlm/block_errors": self.errors}


register("rlm", lambda c, e: RLMEnv(c, e))
