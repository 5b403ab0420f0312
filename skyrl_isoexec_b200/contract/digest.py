"""The three identity hashes of a contract (reference: ISO/contract/identity.py:30-106).

* ``semantic``          what the model means: model ref, the set of logical ops, the cases;
* ``numerical_policy``  everything that can move bits: function-half entries (projected),
                        the cases, the topology claims -- THE HANDSHAKE KEY;
* ``deployment``        comparison-worthy facts proven not to move bits: deployment-half
                        entries, state claims, tolerance claims.
Lists are sorted by their canonical bytes so declaration order never rotates a hash.
"""

from __future__ import annotations

import hashlib

from .codec import canonical_bytes, to_plain
from .model import CompositionEntry, ExecutionCase, ExecutionContract, Identities


def _case_view(c: ExecutionCase) -> dict:
    d = to_plain(c)
    d["constraints"] = sorted(d["constraints"])
    return d


def _entry_view(e: CompositionEntry) -> dict:
    d = to_plain(e)
    d.pop("half")
    d["cases"] = sorted(d["cases"])
    d["coverage"] = None if e.coverage is None else e.coverage.kind  # prose edits rotate nothing
    return d


def _canon_sorted(items) -> list:
    return sorted(items, key=canonical_bytes)


def function_half(c: ExecutionContract) -> dict:
    return {
        "schema_version": c.schema_version,
        "cases": _canon_sorted(_case_view(x) for x in c.cases),
        "entries": _canon_sorted(_entry_view(e) for e in c.composition if e.half == "function"),
        "topology": _canon_sorted(to_plain(t) for t in c.claims.topology),
    }


def deployment_half(c: ExecutionContract) -> dict:
    return {
        "entries": _canon_sorted(_entry_view(e) for e in c.composition if e.half == "deployment"),
        "state": _canon_sorted(to_plain(s) for s in c.claims.state),
        "tolerances": _canon_sorted(to_plain(t) for t in c.claims.tolerances),
    }


def semantic_inputs(c: ExecutionContract) -> dict:
    return {
        "model": {"family": c.model.family, "architectures": sorted(c.model.architectures),
                  "profile_ref": c.model.profile_ref},
        "logical_ops": sorted({op for e in c.composition for op in e.region}),
        "cases": _canon_sorted(_case_view(x) for x in c.cases),
    }


def sha256_of(plain) -> str:
    return hashlib.sha256(canonical_bytes(plain)).hexdigest()


def compute_identities(c: ExecutionContract) -> Identities:
    return Identities(semantic=sha256_of(semantic_inputs(c)), numerical_policy=sha256_of(function_half(c)),
                      deployment=sha256_of(deployment_half(c)))
