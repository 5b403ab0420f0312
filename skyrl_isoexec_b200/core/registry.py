"""Op / implementation registry the execution contract resolves against.

Every op on the logprob path is declared once (``OpSpec``) with the sites it runs at, and every
implementation (``ImplSpec``) declares the architectures it is qualified on, its *rounding
schedule* (which constants pin its arithmetic and may be asserted by machine, plus prose for
what cannot), the ops it subsumes when fused, the state it invalidates and the numerical hazards
its tests exercise. Vocabulary follows the reference (ISO/core/registry.py:14-35,46-121,136-247):
four sites, eight hazards, pin values that are literals, ``PER_MODEL`` or ``OneOf(...)``; a pin
key the schedule does not declare is refused.
"""

from __future__ import annotations

from dataclasses import dataclass, field

SITES = ("trainer_fwd", "trainer_score", "engine_prefill", "engine_decode")
TRAINER_SITES = ("trainer_fwd", "trainer_score")
ENGINE_SITES = ("engine_prefill", "engine_decode")
HAZARDS = ("null_lanes", "t_zero", "non_contiguous", "e_mismatch", "profiling_shapes", "tie_boundaries", "subnormals",
           "signed_zero")
FAMILY_ORDER = ("mm", "attention", "rope", "norms", "activation", "logprobs", "gdn", "moe", "collectives")


class _PerModel:
    def __repr__(self):
        return "PER_MODEL"


PER_MODEL = _PerModel()


class OneOf(tuple):
    def __new__(cls, *vals):
        return super().__new__(cls, vals)


def pin_values_equal(a, b) -> bool:
    """Sequence-insensitive (list == tuple) and bool-strict (True != 1) comparison of pin values."""
    if isinstance(a, bool) != isinstance(b, bool):
        return False
    if isinstance(a, (list, tuple)) and isinstance(b, (list, tuple)):
        return len(a) == len(b) and all(pin_values_equal(x, y) for x, y in zip(a, b))
    return a == b


@dataclass(frozen=True)
class RoundingSchedule:
    machine_assertable: tuple = ()   # ((key, literal | PER_MODEL | OneOf), ...)
    documentary: str = ""

    @staticmethod
    def of(documentary: str = "", **pins) -> "RoundingSchedule":
        return RoundingSchedule(tuple(sorted(pins.items())), documentary)

    def check_pin(self, pins: dict) -> list[str]:
        """Violations of ``pins`` against this schedule: undeclared keys, missing keys, wrong values."""
        decl = dict(self.machine_assertable)
        out = []
        for k in pins:
            if k not in decl:
                out.append(f"pin {k!r} is not declared by the rounding schedule")
        for k, want in decl.items():
            if k not in pins:
                out.append(f"pin {k!r} missing")
                continue
            got = pins[k]
            if want is PER_MODEL:
                continue
            if isinstance(want, OneOf):
                if not any(pin_values_equal(got, w) for w in want):
                    out.append(f"pin {k!r}={got!r} not one of {tuple(want)!r}")
            elif not pin_values_equal(got, want):
                out.append(f"pin {k!r}={got!r} != declared {want!r}")
        return out


@dataclass(frozen=True)
class OpSpec:
    name: str
    sites: tuple[str, ...] = SITES
    doc: str = ""

    @property
    def family(self) -> str:
        return self.name.split(".")[0]


@dataclass(frozen=True)
class ImplSpec:
    op: str
    impl_id: str
    version: int = 1
    supported_archs: frozenset = frozenset({"sm100"})
    rounding: RoundingSchedule = field(default_factory=RoundingSchedule)
    capabilities: frozenset = frozenset()
    subsumes: tuple[str, ...] = ()
    state_invalidation: tuple[str, ...] = ()
    hazards: tuple[str, ...] = ()
    route: str = "canonical"
    reference: str | None = None      # impl_id this one is bitwise-equal to / preserves
    kernel: str = ""                  # source file of the kernel (documentation + claim_refs)
    sites: tuple[str, ...] | None = None  # restrict to a subset of the op's sites

    def __post_init__(self):
        bad = set(self.hazards) - set(HAZARDS)
        if bad:
            raise ValueError(f"{self.op}/{self.impl_id}: unknown hazard(s) {sorted(bad)}")


class Registry:
    def __init__(self):
        self.ops: dict[str, OpSpec] = {}
        self.impls: dict[tuple[str, str], ImplSpec] = {}

    def add_op(self, spec: OpSpec) -> OpSpec:
        if spec.name in self.ops:
            raise ValueError(f"op {spec.name!r} registered twice")
        if set(spec.sites) - set(SITES):
            raise ValueError(f"op {spec.name!r}: unknown site(s) {sorted(set(spec.sites) - set(SITES))}")
        self.ops[spec.name] = spec
        return spec

    def add_impl(self, spec: ImplSpec) -> ImplSpec:
        if spec.op not in self.ops:
            raise ValueError(f"impl {spec.impl_id!r} names unknown op {spec.op!r}")
        key = (spec.op, spec.impl_id)
        if key in self.impls:
            raise ValueError(f"impl {key} registered twice")
        self.impls[key] = spec
        return spec

    def check(self) -> None:
        """Cross-family consistency, run once every family is registered."""
        for key, spec in self.impls.items():
            for sub in spec.subsumes:
                if sub not in self.ops:
                    raise ValueError(f"impl {key} subsumes unknown op {sub!r}")

    def impl(self, op: str, impl_id: str) -> ImplSpec:
        try:
            return self.impls[(op, impl_id)]
        except KeyError:
            raise KeyError(f"no impl {impl_id!r} registered for op {op!r}; known: "
                           f"{sorted(i for (o, i) in self.impls if o == op)}") from None

    def impls_for(self, op: str) -> list[ImplSpec]:
        return [s for (o, _), s in self.impls.items() if o == op]

    def archs(self) -> set[str]:
        return {a for s in self.impls.values() for a in s.supported_archs}
