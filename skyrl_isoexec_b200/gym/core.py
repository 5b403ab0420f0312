"""Environment protocol (reference: skyrl-gym/skyrl_gym/core.py:12-93, envs/base_text_env.py:9-100).

``init(prompt) -> (prompt, info)``; ``step(action) -> {observations, reward, done, metadata}``;
``close()``; ``get_metrics()``; static ``aggregate_metrics(list)``. Text environments receive the
model's decoded string as the action and return OpenAI-style messages as observations; token
environments (``accepts_tokens = True``) receive the sampled token ids directly, which is what
the synthetic benchmark environments use.
"""

from __future__ import annotations

from typing import Any, Callable, TypedDict


class BaseTextEnvStepOutput(TypedDict, total=False):
    observations: list
    reward: float
    done: bool
    metadata: dict
    postprocessed_action: str


class Env:
    accepts_tokens = False

    def init(self, prompt):
        return prompt, {}

    def step(self, action) -> BaseTextEnvStepOutput:
        raise NotImplementedError

    def close(self) -> None:
        pass

    def get_metrics(self) -> dict:
        return {}

    @staticmethod
    def aggregate_metrics(metrics: list[dict]) -> dict:
        out: dict[str, float] = {}
        keys = {k for m in metrics for k in m}
        for k in keys:
            vals = [m[k] for m in metrics if k in m and isinstance(m[k], (int, float))]
            if vals:
                out[k] = sum(vals) / len(vals)
        return out


class BaseTextEnv(Env):
    """Text environment with optional tool groups (``init_tool_groups`` / ``_execute_tool``)."""

    def __init__(self, env_config: dict | None = None, extras: dict | None = None):
        self.env_config = env_config or {}
        self.extras = extras or {}
        self.turns = 0
        self.max_turns = int(self.extras.get("max_turns", 1))
        self.tool_groups: dict[str, Any] = {}
        self.tool_to_group: dict[str, str] = {}

    def init_tool_groups(self, tool_groups: list) -> None:
        for g in tool_groups:
            name = getattr(g, "name", type(g).__name__)
            self.tool_groups[name] = g
            for tool in getattr(g, "tools", lambda: [])():
                self.tool_to_group[tool] = name

    def _execute_tool(self, group: str, tool: str, tool_input: list):
        g = self.tool_groups[group]
        return getattr(g, tool)(*tool_input)


_REGISTRY: dict[str, Callable[..., Env]] = {}


def register(name: str, factory: Callable[..., Env]) -> None:
    if name in _REGISTRY:
        raise ValueError(f"environment {name!r} already registered")
    _REGISTRY[name] = factory


def make(name: str, env_config: dict | None = None, extras: dict | None = None) -> Env:
    if name not in _REGISTRY:
        raise KeyError(f"unknown environment {name!r}; registered: {sorted(_REGISTRY)}")
    return _REGISTRY[name](env_config or {}, extras or {})


def registered_envs() -> list[str]:
    return sorted(_REGISTRY)
