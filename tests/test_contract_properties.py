"""Property-based tests of the contract layer (hypothesis): for generated contracts the canonical form is a fixed point
of encode / decode, the identities are stable under every reordering the schema declares irrelevant and move under
every change it declares relevant, and raw floats never get into a document."""
import dataclasses
import json

import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from skyrl_isoexec_b200.contract import codec, digest, rules
from skyrl_isoexec_b200.contract import model as M

_name = st.text(alphabet="abcdefghijklmnopqrstuvwxyz_", min_size=1, max_size=8)
_const = st.one_of(st.integers(-1000, 1000), st.booleans(), _name,
                   st.floats(allow_nan=False, allow_infinity=False, width=32).map(M.BitPattern.of))


@st.composite
def contracts(draw):
    n_cases = draw(st.integers(1, 3))
    case_ids = draw(st.lists(_name, min_size=n_cases, max_size=n_cases, unique=True))
    cases = tuple(M.ExecutionCase(cid, draw(st.sampled_from(["trainer", "engine"])), draw(st.sampled_from(["no_grad", "grad"])),
                                  draw(st.sampled_from(["fresh", "continued"])), draw(st.sampled_from(["variable", "shape_static"])),
                                  tuple(sorted(draw(st.lists(_name, max_size=2, unique=True)))))
                  for cid in case_ids)
    ops = draw(st.lists(_name, min_size=1, max_size=4, unique=True))
    entries = []
    for op in ops:
        consts = draw(st.dictionaries(_name, _const, max_size=3))
        entries.append(M.CompositionEntry((op,), tuple(case_ids), M.ImplRef(draw(_name), draw(st.integers(1, 9)), "sm100"), "canonical", consts,
                                          coverage=M.Coverage("symbolic_domain", "all shapes")))
    c = M.ExecutionContract("2", M.ModelRef(draw(_name), (draw(_name),), draw(_name)), M.Identities("", "", ""), cases, tuple(entries),
                            M.Claims(topology=(M.TopologyClaim("tp", "pinned", draw(st.integers(1, 8)), "none"),),
                                     tolerances=(M.ToleranceClaim(tuple(sorted(case_ids)), {"max": "0"}),)))
    return dataclasses.replace(c, identities=digest.compute_identities(c))


_settings = settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])


@_settings
@given(contracts())
def test_canonical_form_is_a_fixed_point(c):
    raw = codec.to_canonical_json(c)
    back = codec.from_canonical_json(raw)
    assert back == c and codec.to_canonical_json(back) == raw
    assert raw == json.dumps(json.loads(raw), sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode()
    assert digest.compute_identities(back) == c.identities
    assert not any(isinstance(x, float) for x in _walk(json.loads(raw)))          # floats travel as bit patterns only


def _walk(o):
    if isinstance(o, dict):
        for v in o.values():
            yield from _walk(v)
    elif isinstance(o, list):
        for v in o:
            yield from _walk(v)
    else:
        yield o


@_settings
@given(contracts(), st.randoms(use_true_random=False))
def test_identities_ignore_declared_orderings_and_follow_content(c, rnd):
    # the order of composition entries and of the cases inside an entry is not content
    ents = list(c.composition)
    rnd.shuffle(ents)
    ents = [dataclasses.replace(e, cases=tuple(rnd.sample(list(e.cases), len(e.cases)))) for e in ents]
    shuffled = dataclasses.replace(c, composition=tuple(ents))
    assert digest.compute_identities(shuffled) == c.identities
    # a changed implementation version, or one more constant, is
    e0 = c.composition[0]
    bumped = dataclasses.replace(c, composition=(dataclasses.replace(e0, impl=dataclasses.replace(e0.impl, version=e0.impl.version + 1)),)
                                 + c.composition[1:])
    assert digest.compute_identities(bumped).numerical_policy != c.identities.numerical_policy
    more = dataclasses.replace(c, composition=(dataclasses.replace(e0, constants=dict(e0.constants) | {"zz_extra": 7}),) + c.composition[1:])
    assert digest.compute_identities(more).numerical_policy != c.identities.numerical_policy
    # stale identities on a changed document are reported by the validator
    assert any("IDENT" in f or "identit" in f.lower() for f in rules.validate(bumped))


@_settings
@given(st.recursive(st.one_of(st.integers(), _name, st.floats(allow_nan=False)), lambda ch: st.one_of(st.lists(ch, max_size=3), st.dictionaries(_name, ch, max_size=3)),
                    max_leaves=8))
def test_raw_floats_are_refused_wherever_they_hide(doc):
    has_float = any(isinstance(x, float) for x in _walk(doc))
    if has_float:
        with pytest.raises(codec.SerializationError):
            codec.canonical_bytes(doc)
    else:
        assert json.loads(codec.canonical_bytes(doc)) == doc
