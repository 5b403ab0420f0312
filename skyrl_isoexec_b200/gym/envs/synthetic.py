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


class EvenTokensTurnsEnv(Env):
    """Several model turns without observations: the episode ends after ``max_turns`` turns and the outcome reward
    (fraction of even token ids over ALL turns) arrives with the last one. A token-level stand-in for a multi-turn task."""

    accepts_tokens = True

    def __init__(self, env_config=None, extras=None):
        self.max_turns = int((extras or {}).get("max_turns", 2))
        self.toks: list[int] = []
        self.turns = 0

    def step(self, action):
        self.toks += list(action)
        self.turns += 1
        done = self.turns >= self.max_turns
        frac = (sum(1 for t in self.toks if t % 2 == 0) / len(self.toks)) if self.toks else 0.0
        return {"observations": [], "reward": frac if done else 0.0, "done": done, "metadata": {}}

    def get_metrics(self):
        return {"turns": self.turns}


register("even_tokens", lambda c, e: EvenTokensEnv(c, e))
register("even_tokens_turns", lambda c, e: EvenTokensTurnsEnv(c, e))
register("token_sum_parity", lambda c, e: TokenSumParityEnv(c, e))
