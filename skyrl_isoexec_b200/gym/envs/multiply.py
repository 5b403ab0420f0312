"""Multi-turn toy environment: the model must answer ``a * b`` inside ``\\boxed{}``; a wrong answer
gets one line of feedback and another turn (reference: examples/train/multiply/)."""

from __future__ import annotations

import re

from ..core import BaseTextEnv, register


class MultiplyEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        spec = self.extras.get("reward_spec") or {}
        self.ground_truth = str(spec.get("ground_truth", ""))

    def step(self, action: str):
        self.turns += 1
        m = re.search(r"\\boxed\{([^}]*)\}", action)
        ok = m is not None and m.group(1).strip() == self.ground_truth
        done = ok or self.turns >= self.max_turns
        if ok:
            return {"observations": [], "reward": 1.0, "done": True, "metadata": {"parsed": m.group(1)}}
        reward = 0.5 if m is not None else 0.0
        obs = [] if done else [{"role": "user", "content": "That is not correct. Try again and box the answer."}]
        return {"observations": obs, "reward": reward if done else 0.0, "done": done, "metadata": {}}


register("multiply", lambda c, e: MultiplyEnv(c, e))
