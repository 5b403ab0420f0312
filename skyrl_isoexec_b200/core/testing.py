"""Gate primitives the bitwise tests instantiate (reference: ISO/core/contracts.py:40-152):
integer-view equality, the hazard-exercised rule (a bitwise test must prove its inputs actually
hit the hazard it claims to cover, else it fails) and gradient-set equality."""

from __future__ import annotations

import torch

from .registry import HAZARDS

_INT_VIEW = {torch.float32: torch.int32, torch.bfloat16: torch.int16, torch.float16: torch.int16, torch.float64: torch.int64}


def bitwise_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Equality of the raw bits (so +0/-0 and NaN payloads count), not of the values."""
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    if a.dtype in _INT_VIEW:
        return bool(torch.equal(a.contiguous().view(_INT_VIEW[a.dtype]), b.contiguous().view(_INT_VIEW[b.dtype])))
    return bool(torch.equal(a, b))


def count_bit_mismatches(a: torch.Tensor, b: torch.Tensor) -> int:
    if a.dtype in _INT_VIEW:
        return int((a.contiguous().view(_INT_VIEW[a.dtype]) != b.contiguous().view(_INT_VIEW[b.dtype])).sum())
    return int((a != b).sum())


def hazard_present(name: str, **t) -> bool:
    """Does the input population exercise ``name``? Callers pass the tensors the hazard lives in."""
    if name not in HAZARDS:
        raise KeyError(f"unknown hazard {name!r}")
    x = t.get("x")
    if name == "subnormals":
        tiny = torch.finfo(x.dtype).tiny
        return bool(((x != 0) & (x.abs() < tiny)).any())
    if name == "signed_zero":
        return bool(((x == 0) & torch.signbit(x)).any())
    if name == "tie_boundaries":
        s = torch.sort(x.float(), dim=-1).values
        return bool((s[..., 1:] == s[..., :-1]).any())
    if name == "t_zero":
        return bool(t.get("num_tokens", 1) == 0 or t.get("has_empty", False))
    if name == "null_lanes":
        return bool(t.get("has_padding", False))
    if name == "non_contiguous":
        return not x.is_contiguous()
    if name == "e_mismatch":
        return bool(t.get("experts_unused", False))
    if name == "profiling_shapes":
        return bool(t.get("shapes_vary", False))
    return False


def assert_hazard_exercised(name: str, **t) -> None:
    if not hazard_present(name, **t):
        raise AssertionError(f"test claims to cover hazard {name!r} but its inputs never exercise it")


def check_hazard_coverage(declared: tuple[str, ...], exercised: set[str]) -> list[str]:
    return [h for h in declared if h not in exercised]


def assert_grad_set_equality(params_a: dict, params_b: dict) -> None:
    """Both runs produced gradients for exactly the same parameter names."""
    ga = {k for k, p in params_a.items() if p.grad is not None}
    gb = {k for k, p in params_b.items() if p.grad is not None}
    if ga != gb:
        raise AssertionError(f"gradient sets differ: only A {sorted(ga - gb)}; only B {sorted(gb - ga)}")
