from . import synthetic, gsm8k, multiply, aime, sql, search, lcb, rlm, llm_judge, visual  # noqa: F401
