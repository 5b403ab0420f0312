"""Conversation history of an agent trajectory and its trimming to a token budget (reference: skyrl-agent/skyrl_agent/
functional/history.py ``MessageHistory`` / ``MessageEncoder`` and the memory agent's context reset).

``MessageHistory`` is a message list with typed adders (assistant text, tool result, tool error, user guidance, a reminder
appended to the last message). ``fit(count_tokens, budget)`` makes it fit: the system message, the first user message (the
task) and the most recent messages stay; older tool results are first shortened to a preview, then whole old
assistant / tool exchanges are dropped from the front, and a note says how many were dropped. A trim RESETS what the
token-level trajectory can assume about prefixes: ``was_reset()`` tells the agent that the next prompt does not extend
the previous context, so it must start a new training segment there (``clear_reset_flag`` acknowledges).
"""

from __future__ import annotations

import copy
import json


def preview(output, max_chars: int = 400) -> str:
    s = output if isinstance(output, str) else json.dumps(output, default=str)
    return s if len(s) <= max_chars else s[:max_chars // 2] + f" ...[{len(s) - max_chars} characters cut]... " + s[-max_chars // 2:]


class MessageHistory:
    def __init__(self, messages: list[dict] | None = None):
        self.messages: list[dict] = []
        self._reset = False
        self.dropped = 0
        if messages:
            self.initialize(messages)
            self._reset = False

    # ---- adders
    def add_assistant(self, content: str) -> None:
        self.messages.append({"role": "assistant", "content": content})

    def add_tool_response(self, name: str, output) -> None:
        text = output if isinstance(output, str) else json.dumps(output, default=str)
        self.messages.append({"role": "user", "content": f"EXECUTION RESULT of [{name}]:\n{text}", "tool": name})

    def add_tool_error(self, name: str, error: str) -> None:
        self.add_tool_response(name, {"error": error})

    def add_user_guidance(self, text: str) -> None:
        self.messages.append({"role": "user", "content": text})

    def append_to_last(self, text: str) -> None:
        if not self.messages:
            raise ValueError("cannot append to the last message of an empty history")
        self.messages[-1]["content"] += text

    def initialize(self, messages: list[dict]) -> None:
        self.messages = copy.deepcopy(messages)
        self._reset = True

    def was_reset(self) -> bool:
        return self._reset

    def clear_reset_flag(self) -> None:
        self._reset = False

    def get_messages(self) -> list[dict]:
        return [{"role": m["role"], "content": m["content"]} for m in self.messages]

    def __len__(self) -> int:
        return len(self.messages)

    # ---- trimming
    def _head(self) -> int:
        """Messages that always stay in front: system messages and the first user message."""
        n = 0
        while n < len(self.messages) and self.messages[n]["role"] == "system":
            n += 1
        return n + 1 if n < len(self.messages) and self.messages[n]["role"] == "user" else n

    def fit(self, count_tokens, budget: int, keep_last: int = 2, preview_chars: int = 400) -> bool:
        """Returns whether anything was changed. ``count_tokens(messages) -> int``."""
        if count_tokens(self.get_messages()) <= budget:
            return False
        head = self._head()
        # 1. old tool results become previews
        for m in self.messages[head:max(head, len(self.messages) - keep_last)]:
            if m.get("tool") and len(m["content"]) > preview_chars + 80:
                m["content"] = preview(m["content"], preview_chars)
        # 2. drop the oldest exchanges
        note_at = None
        while count_tokens(self.get_messages()) > budget and len(self.messages) - head - (note_at is not None) > keep_last:
            start = head + (note_at is not None)
            del self.messages[start]
            self.dropped += 1
            while start < len(self.messages) - keep_last and self.messages[start]["role"] != "assistant":
                del self.messages[start]                      # never leave a tool result without the call in front of it
                self.dropped += 1
            note = {"role": "user", "content": f"[{self.dropped} earlier messages were removed to save space]"}
            if note_at is None:
                self.messages.insert(head, note)
                note_at = head
            else:
                self.messages[note_at] = note
        self._reset = True
        return True
