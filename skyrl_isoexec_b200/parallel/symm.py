"""Symmetric (peer-mapped) memory transport for the fused compute+collective kernels.
Filled in by ``parallel/symm_runtime.py`` once a process group has been registered."""

from __future__ import annotations

_registry: dict = {}


def enabled(group) -> bool:
    return group in _registry


def register(group, runtime) -> None:
    _registry[group] = runtime


def get(group):
    return _registry[group]


def tree_all_reduce(partial, group):
    return _registry[group].tree_all_reduce(partial)
