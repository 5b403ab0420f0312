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


register("gsm8k", lambda c, e: GSM8kEnv(c, e))
