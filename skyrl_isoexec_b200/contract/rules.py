"""Structural validation of a frozen contract.

The contract is first flattened into rows of a few kinds ("contract", "entry", "claim pair", "tolerance", "state",
"axis"), then every row is run against a table of checks ``(rule id, row kind, test, message)``. A check's test returns
``None`` when the row is fine, or the detail to put into the message. The result is a list of ``Finding`` records;
``validate`` renders them as ``"[RULE] where: what"`` strings. Callers and tests key on the rule id, never on the prose.

The rule SET is the compatibility surface shared with the reference validator (ISO/contract/validate.py:35-168): a
contract accepted there must be accepted here and the other way round. The rules, by id:

  C-SCHEMA     schema version is one the codec can read             C-CASEDUP   case ids are unique
  C-EMPTY      at least one composition entry                       C-IDENT     stored identities == recomputed
  E-REGION     region non-empty and sorted                          E-ROUTE / E-HALF / E-DISKIND / E-COVKIND  vocabularies
  E-DISREF     a discharge names a ref                              E-CASE      entry cases exist
  E-ARTIFACT   composition_defining carries an artifact             E-REFERENCE reference_preserving carries a reference
  E-DEPLOY     deployment half needs a neutrality_proof             E-FLOAT / E-BITS  constants are not raw floats; hex bits
  P-DUP        one claim per (region, case)                         P-OVERLAP   within a case an op sits in one region only
  P-COVER      required ops of a case are all owned                 P-ASYM      a region with two impls needs discharges
  T-CASE / T-NOBOUND / T-BOUND   tolerance claims name cases, have bounds, bounds are finite numbers
  S-REF / S-NOEVENT / S-EVENT    state claims name a hook, at least one event, events from the vocabulary
  A-DUP / A-PROOF / A-KIND / A-PINNED / A-DEGREE / A-INVARIANT / A-SINGLE   topology claims
"""

from __future__ import annotations

import math
import re
from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any, Callable

from .codec import SUPPORTED_SCHEMA_VERSIONS, SerializationError
from .digest import compute_identities
from .model import (COVERAGE_KINDS, DISCHARGE_KINDS, HALVES, ROUTES, STATE_EVENTS, TOPOLOGY_KINDS, BitPattern,
                    ExecutionContract)


class ValidationError(Exception):
    pass


@dataclass(frozen=True)
class Finding:
    rule: str
    where: str
    what: str

    def __str__(self) -> str:
        return f"[{self.rule}] {self.where}: {self.what}"


@dataclass(frozen=True)
class Row:
    kind: str
    where: str
    obj: Any
    ctx: "View"


class View:
    """Everything the checks look up more than once, computed once per contract."""

    def __init__(self, c: ExecutionContract, required_ops: Mapping[str, frozenset[str]] | None):
        self.c = c
        self.required = required_ops or {}
        self.case_names = [k.id for k in c.cases]
        self.case_set = set(self.case_names)
        # (region, case) -> how many entries claim it;  region -> set of impl ids
        self.pair_count: dict[tuple, int] = {}
        self.impls_of: dict[tuple, set] = {}
        # case -> op -> set of regions that contain the op for that case
        self.homes: dict[str, dict[str, set]] = {k: {} for k in self.case_names}
        for e in c.composition:
            self.impls_of.setdefault(e.region, set()).add(e.impl.id)
            for k in e.cases:
                self.pair_count[(e.region, k)] = self.pair_count.get((e.region, k), 0) + 1
                if k in self.homes:
                    for op in e.region:
                        self.homes[k].setdefault(op, set()).add(e.region)
        self.axis_count: dict[str, int] = {}
        for t in c.claims.topology:
            self.axis_count[t.axis] = self.axis_count.get(t.axis, 0) + 1

    def rows(self):
        c = self.c
        yield Row("contract", "contract", c, self)
        for e in c.composition:
            tag = f"{'+'.join(e.region) or '<no ops>'} by {e.impl.id}"
            yield Row("entry", tag, e, self)
            for k in e.cases:
                yield Row("pair", f"{tag} at {k}", (e, k), self)
        for k in self.case_names:
            yield Row("case", f"case {k}", k, self)
        for t in c.claims.tolerances:
            yield Row("tolerance", f"tolerance {'~'.join(t.case_pair)}", t, self)
        for s in c.claims.state:
            yield Row("state", f"state {s.state_id}", s, self)
        for t in c.claims.topology:
            yield Row("axis", f"axis {t.axis}", t, self)


# ------------------------------------------------------------------------------------ small predicates
_HEXDIGITS = re.compile(r"\A[0-9a-fA-F]+\Z")


def _is_number_text(b) -> bool:
    """A bound is an int, or text that parses to a finite number. bool is not a number here; floats never reach a
    contract (the codec refuses them), so a float bound is a defect too."""
    if isinstance(b, bool) or isinstance(b, float):
        return False
    if isinstance(b, int):
        return True
    if not isinstance(b, str):
        return False
    try:
        return math.isfinite(float(b))
    except ValueError:
        return False


def _blank(s) -> bool:
    return s is None or not str(s).strip()


def _not_in(vocab):
    return lambda value: None if value in vocab else f"{value!r} is not one of {sorted(vocab)}"


# ------------------------------------------------------------------------------------ the checks
def _c_ident(c, v):
    try:
        return None if c.identities == compute_identities(c) else "the stored identities are stale: recomputing them from the body gives other digests"
    except SerializationError as exc:
        return f"the identities cannot be recomputed ({exc})"


def _e_constants(kind):
    def test(e, v):
        for name, val in e.constants:
            if kind == "float" and isinstance(val, float):
                return f"constant {name!r} is a Python float; carry it as a BitPattern"
            if kind == "bits" and isinstance(val, BitPattern) and not _HEXDIGITS.match(val.bits):
                return f"constant {name!r}: {val.bits!r} is not a hex bit pattern"
        return None
    return test


def _p_overlap(case, v):
    clash = {op: homes for op, homes in v.homes[case].items() if len(homes) > 1}
    if clash:
        op = sorted(clash)[0]
        return f"op {op!r} belongs to {len(clash[op])} different regions {sorted(clash[op])}; regions of one case must not overlap"
    return None


def _p_cover(case, v):
    need = v.required.get(case)
    if need is None:
        return None
    lost = sorted(set(need) - set(v.homes[case]))
    return f"no entry owns {lost}" if lost else None


def _p_asym(e, v):
    if len(v.impls_of[e.region]) > 1 and e.discharge is None:
        return (f"the region is served by {sorted(v.impls_of[e.region])} depending on the case, so each of its entries must say "
                f"why the results agree (a discharge)")
    return None


def _a_shape(t, v):
    if t.kind == "pinned":
        if t.degree is None or t.collective_plan is None:
            return "A-PINNED", "a pinned axis states its degree and its collective plan"
        if t.degree < 1:
            return "A-DEGREE", f"degree {t.degree} cannot be deployed"
    elif t.kind == "invariant":
        if not t.domain or not t.proof:
            return "A-INVARIANT", "an invariant axis lists the degrees it holds for and points at the proof"
        if len(set(t.domain)) < 2:
            return "A-SINGLE", f"invariance over one degree {sorted(set(t.domain))} says nothing; pin the axis"
    return None


Check = tuple[str, str, Callable[[Any, View], Any], str]

CHECKS: tuple[Check, ...] = (
    ("C-SCHEMA", "contract", lambda c, v: None if c.schema_version in SUPPORTED_SCHEMA_VERSIONS else c.schema_version,
     "schema version {d!r} cannot be read"),
    ("C-CASEDUP", "contract", lambda c, v: None if len(v.case_set) == len(v.case_names) else sorted(k for k in v.case_set if v.case_names.count(k) > 1),
     "case ids repeat: {d}"),
    ("C-EMPTY", "contract", lambda c, v: None if c.composition else True,
     "the composition is empty; a contract has to bind at least one op, otherwise any two processes trivially agree"),
    ("C-IDENT", "contract", _c_ident, "{d}"),
    ("E-REGION", "entry", lambda e, v: "it lists no op" if not e.region else ("ops must be in sorted order" if tuple(sorted(e.region)) != e.region else None),
     "bad region: {d}"),
    ("E-ROUTE", "entry", lambda e, v: _not_in(ROUTES)(e.route), "route {d}"),
    ("E-HALF", "entry", lambda e, v: _not_in(HALVES)(e.half), "half {d}"),
    ("E-DISKIND", "entry", lambda e, v: None if e.discharge is None else _not_in(DISCHARGE_KINDS)(e.discharge.kind), "discharge kind {d}"),
    ("E-DISREF", "entry", lambda e, v: True if e.discharge is not None and _blank(e.discharge.ref) else None,
     "the discharge points nowhere (blank ref)"),
    ("E-COVKIND", "entry", lambda e, v: None if e.coverage is None else _not_in(COVERAGE_KINDS)(e.coverage.kind), "coverage kind {d}"),
    ("E-ARTIFACT", "entry", lambda e, v: True if e.route == "composition_defining" and e.artifact is None else None,
     "route composition_defining comes with the artifact that defines the composition"),
    ("E-REFERENCE", "entry", lambda e, v: True if e.route == "reference_preserving" and e.reference is None else None,
     "route reference_preserving names the reference it preserves"),
    ("E-DEPLOY", "entry", lambda e, v: True if e.half == "deployment" and (e.discharge is None or e.discharge.kind != "neutrality_proof") else None,
     "an entry of the deployment half must carry a neutrality_proof discharge"),
    ("E-FLOAT", "entry", _e_constants("float"), "{d}"),
    ("E-BITS", "entry", _e_constants("bits"), "{d}"),
    ("P-ASYM", "entry", _p_asym, "{d}"),
    ("E-CASE", "pair", lambda p, v: None if p[1] in v.case_set else p[1], "case {d!r} is not declared"),
    ("P-DUP", "pair", lambda p, v: v.pair_count[(p[0].region, p[1])] if v.pair_count[(p[0].region, p[1])] > 1 else None,
     "{d} entries claim this region for this case; exactly one may"),
    ("P-OVERLAP", "case", _p_overlap, "{d}"),
    ("P-COVER", "case", _p_cover, "{d}"),
    ("T-CASE", "tolerance", lambda t, v: next((k for k in t.case_pair if k not in v.case_set), None), "case {d!r} is not declared"),
    ("T-NOBOUND", "tolerance", lambda t, v: None if t.bounds else True, "no bound given, so nothing is limited"),
    ("T-BOUND", "tolerance", lambda t, v: next((f"{k}={b!r}" for k, b in t.bounds if not _is_number_text(b)), None),
     "bound {d} is not a finite number"),
    ("S-REF", "state", lambda s, v: True if _blank(s.ref) else None, "no hook is named (blank ref)"),
    ("S-NOEVENT", "state", lambda s, v: None if s.invalidated_by else True, "lists no event that invalidates it"),
    ("S-EVENT", "state", lambda s, v: sorted(set(s.invalidated_by) - STATE_EVENTS) or None,
     "events {d} are not lifecycle events (known: " + ", ".join(sorted(STATE_EVENTS)) + ")"),
    ("A-DUP", "axis", lambda t, v: v.axis_count[t.axis] if v.axis_count[t.axis] > 1 else None, "claimed {d} times"),
    ("A-PROOF", "axis", lambda t, v: True if t.proof is not None and _blank(t.proof) else None, "the proof ref is blank"),
    ("A-KIND", "axis", lambda t, v: _not_in(TOPOLOGY_KINDS)(t.kind), "kind {d}"),
    ("A-*", "axis", _a_shape, "{d}"),
)


def findings(contract: ExecutionContract, required_ops: Mapping[str, frozenset[str]] | None = None) -> list[Finding]:
    view = View(contract, required_ops)
    out: list[Finding] = []
    seen = set()
    for row in view.rows():
        for rule, kind, test, msg in CHECKS:
            if kind != row.kind:
                continue
            d = test(row.obj, view)
            if d is None:
                continue
            if rule == "A-*":                    # one test, several rule ids
                rule, d = d
            f = Finding(rule, row.where, msg.format(d=d))
            if f not in seen:                    # P-DUP / A-DUP fire once per claimant with the same text
                seen.add(f)
                out.append(f)
    return out


def validate(contract: ExecutionContract, required_ops: Mapping[str, frozenset[str]] | None = None) -> list[str]:
    """All defects as ``"[RULE] where: what"`` strings; an empty list means the contract is well formed."""
    return [str(f) for f in findings(contract, required_ops)]


def validate_or_raise(contract: ExecutionContract, required_ops=None) -> None:
    v = validate(contract, required_ops)
    if v:
        raise ValidationError("; ".join(v))
