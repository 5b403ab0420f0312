from . import synthetic, gsm8k, multiply  # noqa: F401
