"""Environment package (the reference's skyrl-gym): a Gymnasium-style ``Env`` protocol for
text/token environments, a registry keyed by ``env_class`` and a few built-in environments."""

from .core import Env, BaseTextEnv, BaseTextEnvStepOutput, register, make, registered_envs  # noqa: F401
from . import envs  # noqa: F401  (registers the built-ins)
