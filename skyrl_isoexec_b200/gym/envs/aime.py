"""AIME-style math environment: the last ``\\boxed{...}`` (or ``Answer:`` line) is compared with the ground truth after
normalisation (reference: skyrl-gym/skyrl_gym/envs/aime/)."""

from __future__ import annotations

import re

from ..core import BaseTextEnv, register


def last_boxed(text: str) -> str | None:
    i = text.rfind("\\boxed")
    if i < 0:
        return None
    j = text.find("{", i)
    if j < 0:
        return None
    depth = 0
    for k in range(j, len(text)):
        if text[k] == "{":
            depth += 1
        elif text[k] == "}":
            depth -= 1
            if depth == 0:
                return text[j + 1:k]
    return None


def normalize(ans: str) -> str:
    a = ans.strip().strip("$").replace("\\!", "").replace("\\,", "").replace(" ", "")
    a = re.sub(r"\\text\{([^}]*)\}", r"\1", a).replace("\\%", "").replace("%", "").rstrip(".")
    a = a.replace(",", "") if re.fullmatch(r"-?[\d,]+(\.\d+)?", a) else a
    if re.fullmatch(r"-?\d+\.0+", a):
        a = a.split(".")[0]
    return a.lstrip("0") or "0" if re.fullmatch(r"\d+", a) else a


def compute_score(text: str, ground_truth: str) -> float:
    ans = last_boxed(text)
    if ans is None:
        m = re.findall(r"(?i)answer\s*[:=]\s*([^\n]+)", text)
        ans = m[-1] if m else None
    if ans is None:
        return 0.0
    return 1.0 if normalize(ans) == normalize(str(ground_truth)) else 0.0


class AIMEEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        spec = self.extras.get("reward_spec") or {}
        if "ground_truth" not in spec:
            raise ValueError("aime needs extras['reward_spec']['ground_truth']")
        self.ground_truth = spec["ground_truth"]

    def step(self, action: str):
        return {"observations": [], "reward": compute_score(action, self.ground_truth), "done": True, "metadata": {}}


register("aime", lambda c, e: AIMEEnv(c, e))
