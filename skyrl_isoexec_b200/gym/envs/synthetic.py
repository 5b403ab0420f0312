"""Deterministic synthetic token environments used by the benchmark configurations."""

from __future__ import annotations

from ..core import Env, register


class EvenTokensEnv(Env):
    """Reward = fraction of even token ids in the response (single turn)."""

    accepts_tokens = True

    def __init__(self, env_config=None, extras=None):
        self.last = 0.0

    def step(self, action):
        toks = list(action)
        self.last = (sum(1 for t in toks if t % 2 == 0) / len(toks)) if toks else 0.0
        return {"observations": [], "reward": self.last, "done": True, "metadata": {}}

    def get_metrics(self):
        return {"even_fraction": self.last}


class TokenSumParityEnv(Env):
    """Reward 1 if the sum of response token ids is even, else 0 (sparse binary reward)."""

    accepts_tokens = True

    def __init__(self, env_config=None, extras=None):
        pass

    def step(self, action):
        r = 1.0 if sum(action) % 2 == 0 else 0.0
        return {"observations": [], "reward": r, "done": True, "metadata": {}}


register("even_tokens", lambda c, e: EvenTokensEnv(c, e))
register("token_sum_parity", lambda c, e: TokenSumParityEnv(c, e))
