"""The obligation ledger: every check the contract requires, derived from the contract itself,
recorded per process and closed per phase (reference: ISO/core/enforce.py:25-78,215-248,354-487,618-707).

Phases: INSTALL -> FIRST_FORWARD -> WEIGHT_SYNC -> STEP1. ``derive_obligation_plan`` lists what
must be reported in each phase (an install attestation and a fingerprint per (op, site) of this
side, a ``served`` record per op at first forward, the handshake at weight sync, the gate at step
1, a domain check per topology claim, a hook check per state claim). ``close_phase`` turns every
unreported obligation into a violation. ``refuse()`` raises unless strictness was turned off
(``SKYRL_ISOEXEC_MANIFEST_STRICT=0``) or debug tracing is on. Each process writes a verdict JSON
``enforcement.<side>.r<rank>.json``; ``merge_verdicts`` folds them.
"""

from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass, field

from ..contract import model as M

PHASES = ("INSTALL", "FIRST_FORWARD", "WEIGHT_SYNC", "STEP1")
KINDS = ("build_valid", "install_attest", "fingerprint", "served", "domain_check", "hook_exists", "gate", "handshake",
         "installed_backstop")
SEVERITY = {"build_valid": "fatal", "install_attest": "fatal", "fingerprint": "fatal", "served": "fatal",
            "domain_check": "fatal", "hook_exists": "error", "gate": "fatal", "handshake": "fatal",
            "installed_backstop": "error"}
# obligations that are knowingly not enforced, each with its reason (kept explicit so they are visible)
EXCEPTIONS: tuple[tuple[str, str, str], ...] = (
    ("served", "collectives.nccl_pin", "a declaration about what is NOT on the wire; nothing is served"),
    ("served", "logprobs.lm_head_slice", "counted under mm at the engine sites"),
)


class ContractViolation(RuntimeError):
    pass


@dataclass(frozen=True)
class Obligation:
    phase: str
    kind: str
    key: str

    @property
    def severity(self) -> str:
        return SEVERITY[self.kind]


@dataclass
class Record:
    ok: bool
    detail: str = ""


def strict() -> bool:
    if os.environ.get("SKYRL_ISOEXEC_MANIFEST_STRICT", "1") == "0":
        return False
    return not os.environ.get("SKYRL_ISOEXEC_DEBUG_TRACE")


def refuse(msg: str) -> None:
    """Refuse, don't warn: raise unless strictness is demoted."""
    if strict():
        raise ContractViolation(msg)
    import warnings

    warnings.warn(f"[isoexec, non-strict] {msg}", stacklevel=2)


def derive_obligation_plan(contract: M.ExecutionContract, side: str) -> list[Obligation]:
    role = {c.id: c.runtime_role for c in contract.cases}
    exempt = {(k, key) for k, key, _ in EXCEPTIONS}
    plan = [Obligation("INSTALL", "build_valid", "contract")]
    ops_this_side: set[str] = set()
    for e in contract.composition:
        for cid in e.cases:
            if role[cid] != side:
                continue
            for op in e.region:
                ops_this_side.add(op)
                plan.append(Obligation("INSTALL", "install_attest", f"{op}@{cid}"))
                plan.append(Obligation("INSTALL", "fingerprint", f"{op}@{cid}"))
    for t in contract.claims.topology:
        plan.append(Obligation("INSTALL", "domain_check", f"topology:{t.axis}"))
    for s in contract.claims.state:
        plan.append(Obligation("INSTALL", "hook_exists", f"state:{s.state_id}"))
    for op in sorted(ops_this_side):
        if ("served", op) not in exempt:
            plan.append(Obligation("FIRST_FORWARD", "served", op))
    plan.append(Obligation("WEIGHT_SYNC", "handshake", "contract_hash"))
    for s in contract.claims.state:
        if side == "engine" and "weight_sync" in s.invalidated_by:
            plan.append(Obligation("WEIGHT_SYNC", "installed_backstop", f"invalidate:{s.state_id}"))
    if side == "trainer":
        plan.append(Obligation("STEP1", "gate", "forward_gate"))
    # de-duplicate, keep order
    seen, out = set(), []
    for o in plan:
        if o not in seen:
            seen.add(o)
            out.append(o)
    return out


class Ledger:
    def __init__(self, contract: M.ExecutionContract, side: str, rank: int = 0):
        assert side in ("trainer", "engine")
        self.contract, self.side, self.rank = contract, side, rank
        self.plan = derive_obligation_plan(contract, side)
        self.records: dict[Obligation, Record] = {}
        self.closed: list[str] = []
        self.violations: list[str] = []

    def report(self, kind: str, key: str, ok: bool, detail: str = "", phase: str | None = None) -> None:
        matches = [o for o in self.plan if o.kind == kind and o.key == key and (phase is None or o.phase == phase)]
        if not matches:
            # unplanned reports are kept (they show up in the verdict) but satisfy nothing
            matches = [Obligation(phase or "INSTALL", kind, key)]
        for o in matches:
            self.records[o] = Record(ok, detail)
        if not ok:
            msg = f"[{self.side} r{self.rank}] {kind}:{key} failed: {detail}"
            self.violations.append(msg)
            if SEVERITY.get(kind) == "fatal":
                refuse(msg)

    def close_phase(self, phase: str) -> list[str]:
        """A planned obligation with no record is a violation (silence is not consent)."""
        assert phase in PHASES
        missing = [o for o in self.plan if o.phase == phase and o not in self.records]
        msgs = [f"[{self.side} r{self.rank}] {o.kind}:{o.key} was never reported in phase {phase}" for o in missing]
        self.violations += msgs
        self.closed.append(phase)
        if any(o.severity == "fatal" for o in missing):
            refuse("; ".join(msgs))
        return msgs

    def verdict(self) -> dict:
        return {
            "side": self.side, "rank": self.rank, "numerical_policy": self.contract.identities.numerical_policy,
            "closed": list(self.closed), "ok": not self.violations, "violations": list(self.violations),
            "records": {f"{o.phase}/{o.kind}/{o.key}": {"ok": r.ok, "detail": r.detail} for o, r in self.records.items()},
            "exceptions": [list(x) for x in EXCEPTIONS],
        }

    def write_verdict(self, directory: str) -> str:
        from ..utils import io as uio

        path = directory.rstrip("/") + f"/enforcement.{self.side}.r{self.rank}.json"
        with uio.open_file(path, "w") as f:               # makes the directory when local; any fsspec scheme otherwise
            json.dump(self.verdict(), f, indent=1, sort_keys=True)
        return path


def merge_verdicts(directory: str) -> dict:
    """Fold every ``enforcement.*.json`` of a run: ok only if all are ok and all carry one hash."""
    from ..utils import io as uio

    files = sorted(f for f in uio.list_dir(directory) if f.startswith("enforcement.") and f.endswith(".json"))
    verdicts = []
    for f in files:
        with uio.open_file(directory.rstrip("/") + "/" + f) as fh:
            verdicts.append(json.load(fh))
    hashes = {v["numerical_policy"] for v in verdicts}
    viol = [m for v in verdicts for m in v["violations"]]
    if len(hashes) > 1:
        viol.append(f"processes disagree on numerical_policy: {sorted(h[:12] for h in hashes)}")
    return {"files": files, "ok": bool(verdicts) and not viol, "violations": viol, "numerical_policy": sorted(hashes)}


def install_attestation_digest(installed: dict[tuple[str, str], str]) -> str:
    """Digest of what was actually installed, {(op, site): impl_id}; folded into the handshake so
    two sides that declared the same contract but installed something else cannot agree."""
    blob = json.dumps(sorted([op, site, impl] for (op, site), impl in installed.items()), separators=(",", ":"))
    return hashlib.sha256(blob.encode()).hexdigest()
