"""A tool agent on the function-calling text protocol, with tool schemas, a trimmed history and an optional scratch memory (shown in front of the history once earlier turns were dropped)
(reference: skyrl-agent/skyrl_agent/agents/react/react_agent.py and agents/oh_codeact/codeact_agent.py, which drive their
tools through ``functional/function_calling.py``; ``tools/next_memagent.py`` for the memory).

A turn: the history is rendered through the tokenizer's chat template and sent to the engine; the reply is parsed with
``function_calling.parse_call``; a valid call runs the tool (``toolkit.BaseTool``) and its result goes back as
``EXECUTION RESULT of [tool]``; a call that does not fit the schema goes back as its validation message; a reply without
a call gets a nudge. A tool with ``ends_trajectory`` (``finish``, ``em_finish``) ends the trajectory.

Token bookkeeping follows the other agents (model tokens: loss mask 1 and rollout logprobs; everything the template and
the tools add: mask 0) as long as every new prompt EXTENDS the previous context. When the history had to be trimmed to
``max_context`` tokens that no longer holds, and the trajectory starts a new SEGMENT: ``run`` returns a list of
``Trajectory`` segments of one instance (``instance_id`` ``"<id>"``, ``"<id>@1"``, ...), each a self-contained training
sample; the outcome reward is given to every segment.
"""

from __future__ import annotations

from ..utils.tokenizer import chat_ids

import time

from . import function_calling as fc
from .history import MessageHistory
from .react import Trajectory
from .toolkit import BaseTool, ToolError

SYSTEM = "You are a helpful assistant that can use tools to solve the task step by step."
NO_CALL = "Your reply contains no function call. Call a function, or call `{finish}` with your final answer."


class FunctionCallAgent:
    def __init__(self, engine, tokenizer, tools: dict[str, BaseTool], max_turns: int = 8, sampling_params: dict | None = None,
                 max_context: int = 1 << 30, system_prompt: str = SYSTEM, turn_reminder: bool = True, max_observation_chars: int = 4000):
        self.engine, self.tok, self.tools = engine, tokenizer, tools
        self.schemas = [t.schema() for t in tools.values()]
        self.max_turns, self.sp, self.max_context = max_turns, dict(sampling_params or {}), max_context
        self.system_prompt, self.turn_reminder, self.max_obs = system_prompt, turn_reminder, max_observation_chars
        self.finish_name = next((n for n, t in tools.items() if t.ends_trajectory), "finish")
        if not self.sp.get("stop"):
            self.sp["stop"] = list(fc.STOP_WORDS)

    def _encode(self, messages: list[dict]) -> list[int]:
        return chat_ids(self.tok, messages)

    def _count(self, messages: list[dict]) -> int:
        return len(self._encode(messages))

    def _messages(self, hist: MessageHistory, state: dict) -> list[dict]:
        msgs = hist.get_messages()
        if state.get("memory") and hist.dropped > 0:          # while nothing was dropped the memory call itself is still in view
            msgs = msgs[:1] + [{"role": "user", "content": "Your memory:\n" + state["memory"]}] + msgs[1:]
        return msgs

    async def run(self, instance_id: str, task: str, judge=None, ground_truth=None) -> list[Trajectory]:
        t0 = time.time()
        hist = MessageHistory([{"role": "system", "content": self.system_prompt + fc.tools_prompt(self.schemas)}, {"role": "user", "content": task}])
        state: dict = {"memory": ""}
        segments: list[Trajectory] = []
        seg: Trajectory | None = None
        ctx: list[int] = []
        answer, tool_reward, stop = None, None, "stop"
        turns = 0
        while turns < self.max_turns:
            if hist.fit(lambda ms: self._count(ms), self.max_context) or seg is None or hist.was_reset():
                hist.clear_reset_flag()
                seg = Trajectory(instance_id if not segments else f"{instance_id}@{len(segments)}")
                segments.append(seg)
                seg.prompt_ids = self._encode(self._messages(hist, state))
                ctx = list(seg.prompt_ids)
            else:
                new = self._encode(self._messages(hist, state))
                if new[:len(ctx)] != ctx:                       # the template rewrote history: start a segment rather than mis-align
                    seg = Trajectory(f"{instance_id}@{len(segments)}")
                    segments.append(seg)
                    seg.prompt_ids, ctx = new, list(new)
                else:
                    extra = new[len(ctx):]
                    seg.response_ids += extra
                    seg.loss_mask += [0] * len(extra)
                    seg.logprobs += [0.0] * len(extra)
                    ctx = new
            if len(ctx) >= self.max_context:
                stop = "length"
                break
            out = await self.engine.generate({"prompt_token_ids": [ctx], "sampling_params": self.sp})
            ids = list(out["response_ids"][0])
            lps = list((out.get("response_logprobs") or [[0.0] * len(ids)])[0])
            stop = out["stop_reasons"][0]
            turns += 1
            seg.turns += 1
            seg.response_ids += ids
            seg.loss_mask += [1] * len(ids)
            seg.logprobs += lps
            ctx = ctx + ids
            text = self.tok.decode(ids)
            hist.add_assistant(text)
            try:
                _, call = fc.parse_call(text, self.schemas)
            except fc.FunctionCallValidationError as e:
                hist.add_user_guidance(f"The function call could not be run: {e}")
                continue
            if call is None:
                hist.add_user_guidance(NO_CALL.format(finish=self.finish_name))
                continue
            tool = self.tools[call["name"]]
            seg.tool_calls.append(call["name"])
            try:
                result = tool.call(call["arguments"], state=state, ground_truth=ground_truth, instance_id=instance_id)
            except ToolError as e:
                hist.add_tool_error(call["name"], str(e))
                continue
            except Exception as e:  # noqa: BLE001 - a broken tool is an observation, not the end of the rollout
                hist.add_tool_error(call["name"], f"{type(e).__name__}: {e}")
                continue
            if tool.ends_trajectory:
                answer = result.get("answer") if isinstance(result, dict) else str(result)
                tool_reward = result.get("reward") if isinstance(result, dict) else None
                break
            text_out = result if isinstance(result, str) else __import__("json").dumps(result, default=str)
            hist.add_tool_response(call["name"], text_out[:self.max_obs])
            if self.turn_reminder:
                left = self.max_turns - turns
                hist.append_to_last(f"\n\n[{left} turn{'s' if left != 1 else ''} left]")
        reward = float(tool_reward) if tool_reward is not None else (float(judge(answer, segments[-1])) if judge is not None else 0.0)
        for s in segments:
            s.finish, s.reward, s.stop_reason, s.seconds = answer, reward, stop, time.time() - t0
        return segments
