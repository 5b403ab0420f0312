"""Structural validation of a frozen contract, as a table of independent rules (each yields
violation strings). Rule set follows the reference validator (ISO/contract/validate.py:35-168):
partition totality, no duplicate (region, case), asymmetric region => discharge, route
requirements, deployment half => neutrality proof, finite tolerance bounds, state events in the
vocabulary, pinned / invariant topology rules, stored identities == recomputed identities.
"""

from __future__ import annotations

import math
import re
from collections.abc import Mapping

from .codec import SUPPORTED_SCHEMA_VERSIONS, SerializationError
from .digest import compute_identities
from .model import (COVERAGE_KINDS, DISCHARGE_KINDS, HALVES, ROUTES, STATE_EVENTS, TOPOLOGY_KINDS, BitPattern,
                    ExecutionContract)

_HEX = re.compile(r"^[0-9a-fA-F]+$")


class ValidationError(Exception):
    pass


def _finite_threshold(b) -> bool:
    if isinstance(b, bool):
        return False
    if isinstance(b, int):
        return True
    if isinstance(b, str):
        try:
            return math.isfinite(float(b))
        except ValueError:
            return False
    return False


def _rule_header(c, _req):
    if c.schema_version not in SUPPORTED_SCHEMA_VERSIONS:
        yield f"unsupported schema_version {c.schema_version!r}"
    if len({x.id for x in c.cases}) != len(c.cases):
        yield "duplicate case ids"
    if not c.composition:
        yield ("empty composition: a contract that names no entry claims nothing, so two processes that both "
               "failed to derive a composition would agree perfectly")


def _rule_entries(c, _req):
    case_ids = {x.id for x in c.cases}
    seen = set()
    for e in c.composition:
        name = f"entry {e.region}@{e.impl.id}"
        if not e.region:
            yield f"{name}: empty region"
        if tuple(sorted(e.region)) != e.region:
            yield f"{name}: region tuple must be sorted"
        if e.route not in ROUTES:
            yield f"{name}: unknown route {e.route!r}"
        if e.half not in HALVES:
            yield f"{name}: unknown half {e.half!r}"
        if e.discharge is not None:
            if e.discharge.kind not in DISCHARGE_KINDS:
                yield f"{name}: unknown discharge kind {e.discharge.kind!r}"
            if not e.discharge.ref.strip():
                yield f"{name}: {e.discharge.kind} discharge with an empty ref"
        if e.coverage is not None and e.coverage.kind not in COVERAGE_KINDS:
            yield f"{name}: unknown coverage kind {e.coverage.kind!r}"
        for cid in e.cases:
            if cid not in case_ids:
                yield f"{name}: unknown case {cid!r}"
            if (e.region, cid) in seen:
                yield f"{name}: duplicate (region, case) claim for {cid!r}"
            seen.add((e.region, cid))
        if e.route == "composition_defining" and e.artifact is None:
            yield f"{name}: composition_defining requires an artifact"
        if e.route == "reference_preserving" and e.reference is None:
            yield f"{name}: reference_preserving requires a reference"
        if e.half == "deployment" and (e.discharge is None or e.discharge.kind != "neutrality_proof"):
            yield f"{name}: deployment-half entry requires a neutrality_proof discharge"
        for k, v in e.constants:
            if isinstance(v, float):
                yield f"{name}: constant {k!r} is a raw float"
            if isinstance(v, BitPattern) and not _HEX.match(v.bits):
                yield f"{name}: constant {k!r} has invalid bit pattern {v.bits!r}"


def _rule_partition(c, required_ops):
    for case in c.cases:
        owned: dict[str, tuple] = {}
        for e in c.composition:
            if case.id not in e.cases:
                continue
            for op in e.region:
                if op in owned and owned[op] != e.region:
                    yield f"case {case.id!r}: op {op!r} owned by both {owned[op]} and {e.region}"
                owned[op] = e.region
        if required_ops is not None and case.id in required_ops:
            missing = set(required_ops[case.id]) - set(owned)
            if missing:
                yield f"case {case.id!r}: uncovered required op(s) {sorted(missing)}"


def _rule_asymmetry(c, _req):
    by_region: dict[tuple, list] = {}
    for e in c.composition:
        by_region.setdefault(e.region, []).append(e)
    for region, entries in by_region.items():
        if len({e.impl.id for e in entries}) > 1:
            for e in entries:
                if e.discharge is None:
                    yield f"entry {region}@{e.impl.id}: asymmetric region requires a discharge"


def _rule_claims(c, _req):
    case_ids = {x.id for x in c.cases}
    for t in c.claims.tolerances:
        for cid in t.case_pair:
            if cid not in case_ids:
                yield f"tolerance {t.case_pair}: unknown case {cid!r}"
        if not t.bounds:
            yield f"tolerance {t.case_pair}: no bounds (an envelope with no threshold admits everything)"
        for k, b in t.bounds:
            if not _finite_threshold(b):
                yield f"tolerance {t.case_pair}: bound {k}={b!r} is not a finite threshold"
    for s in c.claims.state:
        if not s.ref.strip():
            yield f"state {s.state_id!r}: empty ref (the claim names no implementing hook)"
        if not s.invalidated_by:
            yield f"state {s.state_id!r}: empty invalidated_by (a state invalidated by nothing is not a claim)"
        bad = sorted(set(s.invalidated_by) - STATE_EVENTS)
        if bad:
            yield (f"state {s.state_id!r}: unknown lifecycle event(s) {bad}; the vocabulary is {sorted(STATE_EVENTS)}")
    axes = [t.axis for t in c.claims.topology]
    if len(axes) != len(set(axes)):
        yield "duplicate topology axes"
    for t in c.claims.topology:
        if t.proof is not None and not t.proof.strip():
            yield f"topology {t.axis!r}: empty proof ref"
        if t.kind not in TOPOLOGY_KINDS:
            yield f"topology {t.axis!r}: unknown kind {t.kind!r}"
        elif t.kind == "pinned":
            if t.degree is None or t.collective_plan is None:
                yield f"topology {t.axis!r}: pinned requires degree and collective_plan"
            elif t.degree < 1:
                yield f"topology {t.axis!r}: pinned degree {t.degree} is not a deployable degree (>= 1)"
        elif not t.domain or not t.proof:
            yield f"topology {t.axis!r}: invariant requires a non-empty domain and a proof"
        elif len(set(t.domain)) < 2:
            yield (f"topology {t.axis!r}: invariant over the single degree {sorted(set(t.domain))} is a tautology; "
                   "pin the axis instead")


def _rule_identities(c, _req):
    try:
        computed = compute_identities(c)
    except SerializationError as exc:
        yield f"identity recomputation failed: {exc}"
        return
    if c.identities != computed:
        yield "stored identities do not match recomputed identities"


RULES = (_rule_header, _rule_entries, _rule_partition, _rule_asymmetry, _rule_claims, _rule_identities)


def validate(contract: ExecutionContract, required_ops: Mapping[str, frozenset[str]] | None = None) -> list[str]:
    """All violations as readable strings; an empty list means the contract is valid."""
    out: list[str] = []
    for rule in RULES:
        out.extend(rule(contract, required_ops))
    return out


def validate_or_raise(contract: ExecutionContract, required_ops=None) -> None:
    v = validate(contract, required_ops)
    if v:
        raise ValidationError("; ".join(v))
