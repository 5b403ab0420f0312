"""A model grades the answer (reference: examples/train/llm_as_a_judge/llm_judge_env.py:41-104).

The judge is any OpenAI-compatible ``/v1/chat/completions`` endpoint (``env_config["base_url"]``, for instance this
framework's own inference server running a grader model) or, for tests and in-process graders, a callable
``env_config["judge_fn"](messages) -> str``. The grader is shown the gold and the predicted solution and must end its reply
with ``### Final Score: 1`` or ``### Final Score: 0``; a bare ``1`` / ``0`` is accepted; anything else, and any transport
error after the retries, scores 0 and is counted in the metrics so that a broken judge is visible in the logs instead of
looking like a hard task."""

from __future__ import annotations

import json
import re
import time
import urllib.request

from ..core import BaseTextEnv, register

JUDGE_PROMPT = (
    "You are a strict evaluation assistant. Compare the GOLD and the PREDICTED solution and decide whether the predicted "
    "solution reaches the same final answer as the gold one. You may reason first. End with a separate last line of the "
    "form\n### Final Score: 1\nor\n### Final Score: 0\nand write nothing after it.")

_SCORE = re.compile(r"###\s*Final Score:\s*([01](?:\.0)?)\s*$", re.MULTILINE)


def parse_judge_reply(reply: str) -> float | None:
    reply = (reply or "").strip()
    m = _SCORE.findall(reply)
    if m:
        return float(m[-1])
    if reply in ("0", "1"):
        return float(reply)
    return None


class LLMJudgeEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        spec = self.extras.get("reward_spec") or {}
        if "ground_truth" not in spec:
            raise ValueError("the llm_judge environment needs extras['reward_spec']['ground_truth']")
        self.ground_truth = str(spec["ground_truth"])
        self.judge_fn = self.env_config.get("judge_fn")
        self.base_url = self.env_config.get("base_url")
        if self.judge_fn is None and not self.base_url:
            raise ValueError("llm_judge needs env_config['base_url'] (an OpenAI-compatible endpoint) or env_config['judge_fn']")
        self.model = self.env_config.get("model", "judge")
        self.retries = int(self.env_config.get("retries", 2))
        self.timeout = float(self.env_config.get("timeout", 60.0))
        self.stats = {"judge_calls": 0, "judge_unparsed": 0, "judge_errors": 0}

    def _ask(self, messages: list[dict]) -> str:
        if self.judge_fn is not None:
            return self.judge_fn(messages)
        body = json.dumps({"model": self.model, "messages": messages, "temperature": 0.0,
                           "max_tokens": int(self.env_config.get("max_tokens", 512))}).encode()
        req = urllib.request.Request(self.base_url.rstrip("/") + "/v1/chat/completions", data=body,
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=self.timeout) as r:
            return json.loads(r.read())["choices"][0]["message"]["content"]

    def _get_reward(self, action: str) -> float:
        messages = [{"role": "user", "content": f"{JUDGE_PROMPT}\n\nGOLD SOLUTION:\n{self.ground_truth}\n\n"
                                                f"PREDICTED SOLUTION:\n{action}\n\nAnswer:"}]
        for attempt in range(self.retries + 1):
            self.stats["judge_calls"] += 1
            try:
                score = parse_judge_reply(self._ask(messages))
            except Exception:  # noqa: BLE001 -- transport or grader failure: retry, then score 0
                self.stats["judge_errors"] += 1
                time.sleep(min(0.05 * 2 ** attempt, 1.0))
                continue
            if score is None:
                self.stats["judge_unparsed"] += 1
                return 0.0
            return score
        return 0.0

    def step(self, action: str):
        self.turns += 1
        return {"observations": [], "reward": self._get_reward(action), "done": True, "metadata": {}}

    def get_metrics(self):
        return dict(self.stats)


register("llm_judge", lambda c, e: LLMJudgeEnv(c, e))
