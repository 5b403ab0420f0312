"""Static alignment of what the registry declares with what the tree contains (the reference keeps such a check in
ISO/core/tests/test_op_gate_alignment.py): every implementation names a source file that exists, a reference-preserving
implementation names a registered reference of the same hardware, every native entry point that Python binds is exported by
a kernel source and the other way round, every declared hazard has a detector, and every hazard declared by a CPU
implementation is exercised by name somewhere in the CPU tests."""

import glob
import os
import re

import torch

from skyrl_isoexec_b200.core import testing
from skyrl_isoexec_b200.core.declarations import build_registry
from skyrl_isoexec_b200.core.registry import HAZARDS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "skyrl_isoexec_b200")


def _impls():
    r = build_registry()
    return r, [i for op in r.ops for i in r.impls_for(op if isinstance(op, str) else op.name)]


def test_every_implementation_names_existing_source_and_a_registered_reference():
    r, impls = _impls()
    assert len(impls) >= 30
    for i in impls:
        assert i.kernel and os.path.isfile(os.path.join(PKG, i.kernel)), f"{i.op}/{i.impl_id}: kernel source {i.kernel!r} is missing"
        if i.route == "reference_preserving":
            assert i.reference, f"{i.op}/{i.impl_id}: a reference-preserving implementation must name its reference"
            refs = [j for j in impls if j.impl_id == i.reference]
            assert refs, f"{i.op}/{i.impl_id}: reference {i.reference!r} is not registered"
            assert any(set(j.supported_archs) & set(i.supported_archs) for j in refs), \
                f"{i.op}/{i.impl_id}: reference {i.reference!r} is declared for other hardware only"
        else:
            assert i.reference is None
    # every op has an implementation (its own, or a kernel of another op that subsumes it) for both the GPU and the CPU route
    for op in r.ops:
        name = op if isinstance(op, str) else op.name
        own = [set(i.supported_archs) for i in r.impls_for(name)]
        fused_into = [set(i.supported_archs) for i in impls if name in i.subsumes]      # served inside another op's kernel
        archs = set().union(*own, *fused_into) if own or fused_into else set()
        assert {"sm100", "cpu"} <= archs, f"{name}: implementations cover {sorted(archs)} only"


def _exports(pattern, prefix):
    names = set()
    for f in glob.glob(os.path.join(PKG, pattern)):
        src = open(f).read()
        for m in re.finditer(r'(?:IX_API|extern\s+"C")\s+(?:__attribute__\(\([^)]*\)\)\s+)?[\w\s\*]*?\b(' + prefix + r'\w+)\s*\(', src):
            names.add(m.group(1))
        for blk in re.finditer(r'extern\s+"C"\s*\{(.*?)\n\}', src, re.S):
            names.update(re.findall(r'\b(' + prefix + r'\w+)\s*\(', blk.group(1)))
    return names


def test_python_bindings_and_native_exports_agree():
    from skyrl_isoexec_b200.ops import _native

    bound = set(_native._SIGS)
    for f in glob.glob(os.path.join(PKG, "**", "*.py"), recursive=True):     # modules that type their own entry points
        bound |= set(re.findall(r"\.(ix_\w+)\.(?:argtypes|restype)\b", open(f).read()))
    exported = _exports("csrc/*.cu", "ix_")
    assert bound, "no native signatures are declared"
    missing = sorted(bound - exported)
    assert not missing, f"typed in Python but exported by no kernel source: {missing}"
    # an export without a binding is dead weight or a forgotten signature (ctypes would guess int arguments)
    allowed_unbound = {n for n in exported if "_noalloc" in n}                # C-only entry points, declared in a header
    unbound = sorted(exported - bound - allowed_unbound)
    assert not unbound, f"exported by a kernel source but without argument types anywhere in the package: {unbound}"


def test_every_hazard_has_a_detector_that_can_say_yes_and_no():
    pos = {"subnormals": dict(x=torch.tensor([1e-42, 1.0])), "signed_zero": dict(x=torch.tensor([-0.0, 1.0])),
           "tie_boundaries": dict(x=torch.tensor([[1.0, 2.0, 1.0]])), "t_zero": dict(x=None, num_tokens=0),
           "null_lanes": dict(x=None, has_padding=True), "non_contiguous": dict(x=torch.zeros(4, 4).t()[1:]),
           "e_mismatch": dict(x=None, experts_unused=True), "profiling_shapes": dict(x=None, shapes_vary=True)}
    neg = {"subnormals": dict(x=torch.tensor([0.0, 1.0])), "signed_zero": dict(x=torch.tensor([0.0, 1.0])),
           "tie_boundaries": dict(x=torch.tensor([[1.0, 2.0, 3.0]])), "t_zero": dict(x=None, num_tokens=3),
           "null_lanes": dict(x=None), "non_contiguous": dict(x=torch.zeros(4, 4)), "e_mismatch": dict(x=None),
           "profiling_shapes": dict(x=None)}
    assert set(pos) == set(HAZARDS) == set(neg)
    for h in HAZARDS:
        assert testing.hazard_present(h, **pos[h]) and not testing.hazard_present(h, **neg[h]), h
        testing.assert_hazard_exercised(h, **pos[h])
    _, impls = _impls()
    declared = {h for i in impls for h in i.hazards}
    assert declared <= set(HAZARDS)
    assert testing.check_hazard_coverage(tuple(sorted(declared)), set(HAZARDS)) == []
    assert testing.check_hazard_coverage(("subnormals", "t_zero"), {"t_zero"}) == ["subnormals"]


def test_hazards_declared_by_cpu_implementations_are_exercised_by_name_in_the_cpu_tests():
    _, impls = _impls()
    declared = {h for i in impls if "cpu" in i.supported_archs for h in i.hazards}
    text = "".join(open(f).read() for f in glob.glob(os.path.join(ROOT, "tests", "test_*.py")) if not f.endswith("test_op_alignment_cpu.py"))
    named = {h for h in declared if re.search(r"[\"']" + h + r"[\"']", text)}
    assert declared == named, f"declared but never exercised by name in tests/: {sorted(declared - named)}"
