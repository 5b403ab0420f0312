from . import synthetic, gsm8k, multiply, aime, tool_envs  # noqa: F401
