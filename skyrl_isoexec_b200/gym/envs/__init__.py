from . import synthetic, gsm8k, multiply, aime, tool_envs, rlm  # noqa: F401
