"""GSM8K-style math environment: exact-match of the final number against ``reward_spec.ground_truth``
(reference: skyrl-gym/skyrl_gym/envs/gsm8k/)."""

from __future__ import annotations

import re

from ..core import BaseTextEnv, register

_STRICT = re.compile(r"#### (\-?[0-9\.\,]+)")
_FLEX = re.compile(r"(\-?[0-9\.\,]+)")


def extract_solution(text: str, method: str = "strict"):
    if method == "strict":
        m = _STRICT.search(text)
        if m is None:
            return None
        return m.group(1).replace(",", "").replace("$", "")
    nums = [n for n in _FLEX.findall(text) if n not in ("", ".", ",")]
    return nums[-1].replace(",", "") if nums else None


def compute_score(text: str, ground_truth: str, method: str = "strict", format_score: float = 0.0, score: float = 1.0):
    ans = extract_solution(text, method)
    if ans is None:
        return 0.0
    return score if ans == str(ground_truth) else format_score


class GSM8kEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        spec = self.extras.get("reward_spec") or {}
        if "ground_truth" not in spec:
            raise ValueError("gsm8k needs extras['reward_spec']['ground_truth']")
        self.ground_truth = spec["ground_truth"]

    def step(self, action: str):
        r = compute_score(action, self.ground_truth, self.env_config.get("method", "strict"))
        return {"observations": [], "reward": r, "done": True, "metadata": {}}


class GSM8kMultiTurnEnv(BaseTextEnv):
    """Several attempts with a reward per turn (reference: skyrl-gym/skyrl_gym/envs/gsm8k/multi_turn_env.py): a turn scores
    1 when its ``#### answer`` is right (the episode ends), ``0.2 / max_turns`` when it is well formed but wrong, else 0;
    between turns the model is asked for reasoning plus a tentative answer, and before the last turn for the final answer
    only. ``max_turns`` comes from ``extras.max_turns`` or ``extras.extra_info.max_turns`` (default 5)."""

    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        spec = self.extras.get("reward_spec") or {}
        if "ground_truth" not in spec:
            raise ValueError("gsm8k_multi_turn needs extras['reward_spec']['ground_truth']")
        self.ground_truth = spec["ground_truth"]
        self.max_turns = int(self.extras.get("max_turns", (self.extras.get("extra_info") or {}).get("max_turns", 5)))
        self.format_score = float(self.env_config.get("format_score", 0.2)) / self.max_turns
        self.solved = False

    def _nudge(self) -> list[dict]:
        left = self.max_turns - self.turns
        if left <= 0:
            return []
        if left > 1:
            text = ("Please provide your step-by-step reasoning, and also include a tentative numeric answer at the end in the "
                    "exact format: '#### ANSWER'.")
        else:
            text = "Now provide only the final numeric answer in the exact format: '#### ANSWER'."
        return [{"role": "user", "content": text}]

    def step(self, action: str):
        self.turns += 1
        r = compute_score(action, self.ground_truth, "strict", self.format_score, 1.0)
        self.solved = r == 1.0
        done = self.solved or self.turns >= self.max_turns
        return {"observations": [] if done else self._nudge(), "reward": r, "done": done, "metadata": {}}

    def get_metrics(self) -> dict:
        return {"steps": self.turns, "solved": float(self.solved)}

    @staticmethod
    def aggregate_metrics(metrics: list[dict]) -> dict:
        if not metrics:
            return {}
        n = len(metrics)
        return {"avg_steps": sum(float(m.get("steps", 0)) for m in metrics) / n, "solved": sum(float(m.get("solved", 0)) for m in metrics) / n}


register("gsm8k", lambda c, e: GSM8kEnv(c, e))
register("gsm8k_multi_turn", lambda c, e: GSM8kMultiTurnEnv(c, e))
