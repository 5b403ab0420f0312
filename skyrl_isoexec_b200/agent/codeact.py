"""CodeAct-style agent: the model acts by writing code, the environment answers with what the code printed
(reference: skyrl-agent/skyrl_agent/agents, the OpenHands CodeAct agent family). A turn ends with one of

    <execute_python> ...code... </execute_python>     run in a fresh interpreter (``gym/tools.py::PythonToolGroup``)
    <execute_bash> ...command... </execute_bash>      only if a bash runner was given (off by default)
    <finish> answer </finish>

Model tokens carry loss mask 1 and their rollout logprobs, observation tokens mask 0, exactly as in the ReAct agent, so
``to_generator_output`` and ``AsyncDispatcher`` of ``agent/react.py`` work on these trajectories unchanged. Snippets of
one trajectory share state through a growing prelude: every snippet that ran without an error is replayed (silently)
in front of the next one, which gives notebook-like persistence without a long-lived interpreter process.
"""

from __future__ import annotations

from ..utils.tokenizer import chat_ids, chat_ids_continuation

import json
import re
import time
from typing import Callable

from ..gym.tools import PythonToolGroup
from .react import Trajectory

_PY = re.compile(r"<execute_python>(.*?)</execute_python>", re.S)
_SH = re.compile(r"<execute_bash>(.*?)</execute_bash>", re.S)
_FINISH = re.compile(r"<finish>(.*?)</finish>", re.S)

_SILENCE = "import sys as _s, io as _io\n_o = _s.stdout\n_s.stdout = _io.StringIO()\n{body}\n_s.stdout = _o\n"


class CodeActAgent:
    SYSTEM = ("You solve the task by writing Python. Put code between <execute_python> and </execute_python>; you will see "
              "what it prints. Variables persist between snippets. When you are done write <finish>your answer</finish>.")

    def __init__(self, engine, tokenizer, max_turns: int = 8, sampling_params: dict | None = None, python: PythonToolGroup | None = None,
                 bash: Callable[[str], dict] | None = None, max_context: int = 1 << 30, max_observation_chars: int = 4000):
        self.engine, self.tok = engine, tokenizer
        self.max_turns, self.sp, self.max_context = max_turns, sampling_params or {}, max_context
        self.python, self.bash, self.max_obs = python or PythonToolGroup(), bash, max_observation_chars

    def _run_python(self, code: str, prelude: list[str]) -> tuple[dict, bool]:
        silent = "".join(_SILENCE.format(body=p) for p in prelude)
        res = self.python.python(silent + code)
        return res, bool(res.get("ok"))

    async def run(self, instance_id: str, task: str, judge: Callable[[str | None, Trajectory], float]) -> Trajectory:
        t0 = time.time()
        tr = Trajectory(instance_id)
        msgs = [{"role": "system", "content": self.SYSTEM}, {"role": "user", "content": task}]
        tr.prompt_ids = chat_ids(self.tok, msgs)
        ctx, prelude = list(tr.prompt_ids), []
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
            py, sh = _PY.search(text), _SH.search(text)
            if py is not None:
                code = py.group(1).strip("\n")
                res, ok = self._run_python(code, prelude)
                if ok:
                    prelude.append(code)
                tr.tool_calls.append("python")
                obs = (res.get("stdout") or "") + (("\n[stderr]\n" + res["stderr"]) if res.get("stderr") else "")
                obs = obs or "(no output)"
            elif sh is not None and self.bash is not None:
                res = self.bash(sh.group(1).strip())
                tr.tool_calls.append("bash")
                obs = json.dumps(res, default=str)
            elif sh is not None:
                obs = "bash is not available here; use <execute_python>."
            else:
                obs = "No <execute_python> block or <finish> found."
            obs_ids = chat_ids_continuation(self.tok, [{"role": "tool", "content": obs[:self.max_obs]}])
            tr.response_ids += obs_ids
            tr.loss_mask += [0] * len(obs_ids)
            tr.logprobs += [0.0] * len(obs_ids)
            ctx += obs_ids
        tr.reward = float(judge(tr.finish, tr))
        tr.seconds = time.time() - t0
        return tr
