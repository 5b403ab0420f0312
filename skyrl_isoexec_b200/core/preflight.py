"""Launch-readiness gate (reference: ISO/core/tests/preflight_launch.py prints PREFLIGHT: READY/BLOCKED after running
its battery with the GPUs hidden; ISO/core/tests/test_op_gate_alignment.py statically checks that every registered
claim maps to a test).

    python -m skyrl_isoexec_b200.core.preflight [--model qwen3-8b]

Runs on a CPU box before a job is submitted. Checks, each reported as ok / BLOCKED with the reason:
  registry        every implementation names a kernel source that exists; subsumption and pins are consistent
  alignment       every registered op family has at least one test file that mentions it
  contract        the execution contract builds for the model on both roles and the two hashes agree
  flags           the flag table is self-consistent and this environment has no split-brain function flag
  fusion ledger   the CPU-checkable fused regions equal their unfused chains on hazard inputs
  native          both native libraries are present (built in-tree)
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REPO = ROOT.parent


def check_registry() -> list[str]:
    from .declarations import build_registry

    reg = build_registry()
    reg.check()
    errs = []
    for im in reg.impls.values():
        for src in filter(None, (k.strip() for k in im.kernel.replace("+", ",").split(","))):
            if not (ROOT / src.split("::")[0]).exists():
                errs.append(f"{im.op}/{im.impl_id}: kernel source {src} does not exist")
    return errs


def check_alignment() -> list[str]:
    """Every op family is named by some test (a claim nobody tests blocks the launch)."""
    from .declarations import build_registry

    reg = build_registry()
    tests = "\n".join(p.read_text() for p in (REPO / "tests").glob("test_*.py"))
    needles = {"mm": ("gemm_nt", "gemm"), "attention": ("attention",), "rope": ("rope",), "norms": ("rmsnorm",), "logprobs": ("logprob",),
               "collectives": ("tree_all_reduce", "row_parallel", "tree_fold"), "gdn": ("gdn",), "moe": ("moe", "router"),
               "activation": ("swiglu", "sigmoid_gate"), "sampling": ("Sampler", "sampler"), "loss": ("ppo_loss", "policy_loss"),
               "embedding": ("embed", "DecoderLM"), "residual": ("rmsnorm", "residual")}
    errs = []
    fams = sorted({op.split(".")[0] for op in reg.ops})
    for fam in fams:
        keys = needles.get(fam, (fam,))
        if not any(k in tests for k in keys):
            errs.append(f"op family {fam!r}: no test mentions it")
    return errs


def check_contract(model: str) -> list[str]:
    from ..models.config import get_config
    from . import process as P
    from .compose import contract_for_model

    cfg = get_config(model)
    a = contract_for_model(cfg, "sm100")       # what the trainer process builds
    b = contract_for_model(cfg, "sm100")       # what the engine process builds from the same declarations
    ha, hb = P.contract_hash(a), P.contract_hash(b)
    errs = [] if ha == hb else [f"two builds of the contract for {model} differ: {ha} vs {hb}"]
    cpu = P.contract_hash(contract_for_model(cfg, "cpu"))
    if cpu == ha:
        errs.append("the CPU and sm100 contracts hash alike: the architecture is missing from the numerical policy")
    return errs


def check_flags() -> list[str]:
    from . import flags

    errs = list(flags.check_table())
    errs += [f"split-brain: {m}" for m in flags.latent_split_brain(dict(os.environ), dict(os.environ))]
    return errs


def check_fusion_ledger() -> list[str]:
    from . import fusion_ledger as FL

    try:
        res = FL.run_checkers("cpu")
    except LookupError as e:
        return [str(e)]
    return [f"fused region {name!r} differs from its unfused chain" for name, ok in res.items() if ok is False]


def check_native() -> list[str]:
    lib = ROOT / "lib"
    return [f"{n} is missing: run python -m skyrl_isoexec_b200.build" for n in ("libisoexec_b200.so", "libisoexec_cpu.so") if not (lib / n).exists()]


def run(model: str = "qwen3-8b") -> tuple[bool, dict]:
    checks = {"registry": check_registry, "alignment": check_alignment, "contract": lambda: check_contract(model),
              "flags": check_flags, "fusion ledger": check_fusion_ledger, "native": check_native}
    report = {}
    for name, fn in checks.items():
        try:
            report[name] = fn()
        except Exception as e:  # noqa: BLE001
            report[name] = [f"{type(e).__name__}: {e}"]
    return all(not v for v in report.values()), report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    args = ap.parse_args(argv)
    os.environ.setdefault("CUDA_VISIBLE_DEVICES", "")
    ok, report = run(args.model)
    for name, errs in report.items():
        print(f"  {name:14s} {'ok' if not errs else 'BLOCKED'}")
        for e in errs:
            print(f"      {e}")
    print("PREFLIGHT: READY" if ok else "PREFLIGHT: BLOCKED")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
