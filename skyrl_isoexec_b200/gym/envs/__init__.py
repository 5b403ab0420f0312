from . import synthetic, gsm8k, multiply, aime, tool_envs, rlm, llm_judge, visual  # noqa: F401
