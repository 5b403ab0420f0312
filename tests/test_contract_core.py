"""Contract layer: canonical codec, identities, validator refusals, registry pins, composition
for every model family, process handshake, obligation ledger and adapter (all CPU)."""
import dataclasses
import json
import os

import pytest

from skyrl_isoexec_b200.contract import codec, digest, rules
from skyrl_isoexec_b200.contract import model as M
from skyrl_isoexec_b200.core import ledger as L
from skyrl_isoexec_b200.core import process as P
from skyrl_isoexec_b200.core.adapter import ContractAdapter, resolve_ref, served_ops_of
from skyrl_isoexec_b200.core.compose import (CASES, ContractBuildError, Selection, build_execution_contract,
                                             contract_for_model, derive_selections, profile_from_model_config)
from skyrl_isoexec_b200.core.declarations import build_registry
from skyrl_isoexec_b200.core.registry import HAZARDS, SITES, OneOf, PER_MODEL, RoundingSchedule, pin_values_equal
from skyrl_isoexec_b200.core.signatures import SignatureTable
from skyrl_isoexec_b200.models.config import get_config


def _fixture():
    cases = (M.ExecutionCase("trainer_score", "trainer", "no_grad", "fresh", "variable"),
             M.ExecutionCase("engine_decode", "engine", "no_grad", "continued", "shape_static", ("b", "a")))
    e1 = M.CompositionEntry(("mm",), ("trainer_score", "engine_decode"), M.ImplRef("k", 1, "sm100"), "canonical",
                            {"block_k": 64, "eps": M.BitPattern.of(1e-6)}, coverage=M.Coverage("symbolic_domain", "all shapes"))
    c = M.ExecutionContract("2", M.ModelRef("fam", ("Arch",), "ref"), M.Identities("", "", ""), cases, (e1,),
                            M.Claims(topology=(M.TopologyClaim("tp", "pinned", 1, "none"),),
                                     tolerances=(M.ToleranceClaim(("engine_decode", "trainer_score"), {"max": "0"}),)))
    return dataclasses.replace(c, identities=digest.compute_identities(c))


def test_roundtrip_and_canonical_form():
    c = _fixture()
    raw = codec.to_canonical_json(c)
    assert codec.from_canonical_json(raw) == c
    assert raw == json.dumps(json.loads(raw), sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode()
    assert rules.validate(c) == []


def test_codec_refusals():
    c = _fixture()
    plain = codec.to_plain(c)
    with pytest.raises(codec.SerializationError):
        codec.canonical_bytes({"x": 1.5})                                   # raw float
    bad = dict(plain, surprise=1)
    with pytest.raises(codec.UnknownFieldError):
        codec.from_plain(M.ExecutionContract, bad)                          # unknown field
    with pytest.raises(codec.SerializationError):
        codec.from_canonical_json(json.dumps(dict(plain, schema_version="1")))   # old schema refused, never rehashed
    with pytest.raises(codec.SerializationError):
        codec.from_canonical_json('{"schema_version":"2","x":1.0}')         # JSON float in a document


def test_identity_projections():
    c = _fixture()
    # reordering constraints / cases inside an entry rotates nothing
    e = c.composition[0]
    c2 = dataclasses.replace(c, composition=(dataclasses.replace(e, cases=tuple(reversed(e.cases))),))
    assert digest.compute_identities(c2) == c.identities
    # coverage prose is not hashed, coverage kind is
    c3 = dataclasses.replace(c, composition=(dataclasses.replace(e, coverage=M.Coverage("symbolic_domain", "other words")),))
    assert digest.compute_identities(c3).numerical_policy == c.identities.numerical_policy
    c4 = dataclasses.replace(c, composition=(dataclasses.replace(e, coverage=M.Coverage("enumerated_shapes", "all shapes")),))
    assert digest.compute_identities(c4).numerical_policy != c.identities.numerical_policy
    # a pinned constant moves the handshake key; a tolerance only the deployment identity
    c5 = dataclasses.replace(c, composition=(dataclasses.replace(e, constants={"block_k": 32, "eps": M.BitPattern.of(1e-6)}),))
    assert digest.compute_identities(c5).numerical_policy != c.identities.numerical_policy
    c6 = dataclasses.replace(c, claims=dataclasses.replace(c.claims, tolerances=(M.ToleranceClaim(("engine_decode", "trainer_score"), {"max": "1e-6"}),)))
    i6 = digest.compute_identities(c6)
    assert i6.numerical_policy == c.identities.numerical_policy and i6.deployment != c.identities.deployment


@pytest.mark.parametrize("mutate,needle", [
    (lambda c, e: dataclasses.replace(c, composition=()), "[C-EMPTY]"),
    (lambda c, e: dataclasses.replace(c, composition=(dataclasses.replace(e, route="fast"),)), "[E-ROUTE]"),
    (lambda c, e: dataclasses.replace(c, composition=(dataclasses.replace(e, cases=("nope",)),)), "[E-CASE]"),
    (lambda c, e: dataclasses.replace(c, composition=(dataclasses.replace(e, route="reference_preserving"),)), "[E-REFERENCE]"),
    (lambda c, e: dataclasses.replace(c, composition=(dataclasses.replace(e, route="composition_defining"),)), "[E-ARTIFACT]"),
    (lambda c, e: dataclasses.replace(c, composition=(dataclasses.replace(e, half="deployment"),)), "[E-DEPLOY]"),
    (lambda c, e: dataclasses.replace(c, composition=(e, dataclasses.replace(e, impl=M.ImplRef("other", 1, "sm100"), cases=("trainer_score",)),)), "[P-DUP]"),
    (lambda c, e: dataclasses.replace(c, composition=(dataclasses.replace(e, cases=("trainer_score",)), dataclasses.replace(e, impl=M.ImplRef("other", 1, "sm100"), cases=("engine_decode",)))), "[P-ASYM]"),
    (lambda c, e: dataclasses.replace(c, claims=M.Claims(tolerances=(M.ToleranceClaim(("engine_decode", "trainer_score"), {"max": "inf"}),))), "[T-BOUND]"),
    (lambda c, e: dataclasses.replace(c, claims=M.Claims(state=(M.StateClaim("kv", ("reboot",), False, "x::y"),))), "[S-EVENT]"),
    (lambda c, e: dataclasses.replace(c, claims=M.Claims(topology=(M.TopologyClaim("tp", "invariant", domain=(2,), proof="p"),))), "[A-SINGLE]"),
    (lambda c, e: dataclasses.replace(c, claims=M.Claims(topology=(M.TopologyClaim("tp", "pinned"),))), "[A-PINNED]"),
])
def test_validator_refusals(mutate, needle):
    c = _fixture()
    bad = mutate(c, c.composition[0])
    bad = dataclasses.replace(bad, identities=digest.compute_identities(bad))
    assert any(needle in v for v in rules.validate(bad)), rules.validate(bad)


def test_stale_identities_are_caught():
    c = _fixture()
    bad = dataclasses.replace(c, identities=M.Identities("0" * 64, c.identities.numerical_policy, c.identities.deployment))
    assert any("[C-IDENT]" in v for v in rules.validate(bad))


def test_rounding_schedule_pins():
    s = RoundingSchedule.of("doc", block=4096, leaves=PER_MODEL, kind=OneOf("a", "b"), window=(-1, 0))
    assert s.check_pin({"block": 4096, "leaves": 8, "kind": "b", "window": [-1, 0]}) == []
    assert any("not declared" in e for e in s.check_pin({"block": 4096, "leaves": 8, "kind": "a", "window": (-1, 0), "extra": 1}))
    assert any("missing" in e for e in s.check_pin({"block": 4096, "kind": "a", "window": (-1, 0)}))
    assert any("not one of" in e for e in s.check_pin({"block": 4096, "leaves": 8, "kind": "c", "window": (-1, 0)}))
    assert pin_values_equal([1, 2], (1, 2)) and not pin_values_equal(True, 1)


def test_registry_vocabulary_and_every_family_builds():
    reg = build_registry()
    assert len(SITES) == 4 and len(HAZARDS) == 8
    assert {"mm", "attention.varlen", "rope.rope", "norms.rms", "logprobs.log_softmax", "gdn.core", "moe.router",
            "collectives.tree_all_reduce"} <= set(reg.ops)
    assert reg.archs() == {"sm100", "cpu"}
    hashes = {}
    for name, arch in [("tiny-qwen3", "cpu"), ("qwen3-8b", "sm100"), ("qwen3-32b", "sm100"), ("qwen3-30b-a3b", "sm100"),
                       ("qwen3.5-hybrid", "sm100"), ("tiny-moe", "cpu"), ("tiny-hybrid", "cpu")]:
        c = contract_for_model(get_config(name), arch, registry=reg)
        assert rules.validate(c) == [] and [x.id for x in c.cases] == [x.id for x in CASES]
        hashes[(name, arch)] = (c.identities.numerical_policy, c.identities.semantic)
    assert len({s for _, s in hashes.values()}) == len(hashes)              # every model has its own semantic identity
    # two dense Qwen3 sizes run the same ops with the same pins: one numerical policy; other families differ
    assert hashes[("qwen3-8b", "sm100")][0] == hashes[("qwen3-32b", "sm100")][0]
    assert len({n for n, _ in hashes.values()}) == len(hashes) - 1
    # the same model on another arch is a different numerical policy (k-step differs per tensor-core generation)
    assert contract_for_model(get_config("tiny-qwen3-bf16"), "cpu").identities.numerical_policy != \
        contract_for_model(get_config("tiny-qwen3-bf16"), "sm100").identities.numerical_policy


def test_contract_build_refusals():
    reg = build_registry()
    cfg = get_config("qwen3-8b")
    prof = profile_from_model_config(cfg)
    sel = derive_selections(prof, "sm100")
    with pytest.raises(ContractBuildError, match="not declared by any"):
        build_execution_contract(prof, reg, sel, "sm90")
    bad = dict(sel)
    bad[("mm", "engine_decode")] = Selection.of("tcgen05_batch_invariant", block_k=64, mma_k=16, split_k=4, accum="fp32_tmem",
                                                tile_m=128, tile_n=256)
    with pytest.raises(ContractBuildError, match="split_k"):
        build_execution_contract(prof, reg, bad, "sm100")
    with pytest.raises(ContractBuildError, match="not qualified"):
        build_execution_contract(prof, reg, derive_selections(prof, "cpu"), "sm100")
    with pytest.raises(ContractBuildError, match="outside the invariant domain"):
        profile_from_model_config(cfg, trainer_tp=4, engine_tp=3)
    inv = contract_for_model(cfg, "sm100", trainer_tp=4, engine_tp=2)
    tp = [t for t in inv.claims.topology if t.axis == "tp"][0]
    assert tp.kind == "invariant" and set(tp.domain) == {1, 2, 4, 8}
    assert resolve_ref(tp.proof)


def test_gdn_is_declared_asymmetric_with_discharge():
    c = contract_for_model(get_config("qwen3.5-hybrid"), "sm100")
    core = [e for e in c.composition if "gdn.core" in e.region]
    assert {e.impl.id for e in core} == {"cpr_chunk_scan", "cpr_recurrent_step"}
    assert all(e.discharge is not None and e.discharge.kind == "bitwise_equal_to" for e in core)


def test_handshake_hash_extensions_and_negative_control(monkeypatch):
    c = _fixture()
    P.clear_contract_extensions()
    assert P.composite_hash(c.identities.numerical_policy) == c.identities.numerical_policy
    h1 = P.composite_hash("base", {"a": lambda: "1"})
    assert h1 != "base" and h1 == P.composite_hash("base", {"a": lambda: "1"})

    def boom():
        raise KeyError("x")
    assert P.composite_hash("base", {"a": boom}) != h1                      # a failing extension poisons the hash
    P.assert_contract_agreement("x", "x")
    with pytest.raises(P.ContractMismatch):
        P.assert_contract_agreement("x", "y")
    with pytest.raises(P.ContractMismatch):
        P.assert_contract_agreement("x", None)
    monkeypatch.setenv(P.ENV_NEGATIVE_CONTROL, "1")
    assert P.contract_hash(c) != c.identities.numerical_policy


def test_contract_delivery(tmp_path, monkeypatch):
    c = _fixture()
    path = str(tmp_path / "contract.json")
    P.write_contract(c, path)
    assert P.load_contract(path) == c
    monkeypatch.setenv(P.ENV_CONTRACT_HASH, "f" * 64)
    with pytest.raises(P.ContractDeliveryError):
        P.load_contract(path)
    monkeypatch.delenv(P.ENV_CONTRACT_HASH)
    raw = json.loads(open(path).read())
    raw["cases"][0]["grad_mode"] = "grad"
    open(path, "w").write(json.dumps(raw))
    with pytest.raises(P.ContractDeliveryError, match="do not match"):
        P.load_contract(path)
    assert ("mm", "trainer_score") in P.expected_installed_keys(c, "trainer")


def test_ledger_missing_record_is_a_violation(tmp_path, monkeypatch):
    c = contract_for_model(get_config("tiny-qwen3"), "cpu")
    lg = L.Ledger(c, "trainer", 3)
    kinds = {o.kind for o in lg.plan}
    assert {"build_valid", "install_attest", "fingerprint", "served", "domain_check", "hook_exists", "handshake", "gate"} <= kinds
    with pytest.raises(L.ContractViolation):
        lg.close_phase("INSTALL")                                            # nothing was reported
    monkeypatch.setenv("SKYRL_ISOEXEC_MANIFEST_STRICT", "0")
    lg2 = L.Ledger(c, "engine", 0)
    with pytest.warns(UserWarning):
        msgs = lg2.close_phase("INSTALL")
    assert msgs and not lg2.verdict()["ok"]
    lg2.write_verdict(str(tmp_path))
    merged = L.merge_verdicts(str(tmp_path))
    assert not merged["ok"] and merged["files"] == ["enforcement.engine.r0.json"]


def test_adapter_full_lifecycle_and_negative_install(monkeypatch):
    from skyrl_isoexec_b200.models.decoder import DecoderLM

    P.clear_contract_extensions()
    model = DecoderLM(get_config("tiny-qwen3"))
    tr, en = ContractAdapter("trainer", model), ContractAdapter("engine", model)
    tr.run_install()
    h_tr = P.contract_hash(tr.contract)
    en.run_install()
    assert P.contract_hash(en.contract) == h_tr
    for ad in (tr, en):
        ad.note_served(served_ops_of(model.cfg))
        ad.on_first_forward()
    en.on_weight_sync(h_tr, ["engine_kv_cache"])
    tr.on_weight_sync(P.contract_hash(en.contract))
    tr.on_gate(True)
    assert tr.ledger.verdict()["ok"] and en.ledger.verdict()["ok"]
    # an engine that installed something else than it declared cannot agree with the trainer
    bad = ContractAdapter("engine", model)
    bad.run_install()
    bad.fingerprint.record_install("mm", "engine_decode", "some_other_gemm")
    assert bad.attestation_digest().startswith("INSTALL-MISMATCH")
    # declared but never served
    t2 = ContractAdapter("trainer", model)
    t2.run_install()
    with pytest.raises(L.ContractViolation, match="never executed"):
        t2.on_first_forward()
    # failed handshake refuses
    t3 = ContractAdapter("trainer", model)
    t3.run_install()
    with pytest.raises(L.ContractViolation, match="handshake"):
        t3.on_weight_sync("0" * 64)


def test_signature_table_needs_proof():
    t = SignatureTable()
    with pytest.raises(ValueError):
        t.admit("m", "h", "sm100", (0.0, 0.0), proof_ref=" ")
    t.admit("m", "h", "sm100", (0.0, 0.0), proof_ref="tests/test_gpu_kernels.py::test_engine_and_trainer")
    assert t.check("m", "h", "sm100", 0.0)[0] and not t.check("m", "h", "sm100", 1e-7)[0]
    assert not t.check("m", "other", "sm100", 0.0)[0]


def _tiny_trainer(tmp_path, model="tiny-qwen3"):
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    cfg = SkyRLTrainConfig.from_cli_overrides([
        f"trainer.policy.model={model}", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=6",
        "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=8",
        "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=8", "trainer.logger=jsonl",
        f"trainer.ckpt_path={tmp_path}", "trainer.ckpt_interval=0"])
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.build_models()
    tr.sync_weights()
    return tr


def test_ledger_refuses_when_an_op_is_served_by_another_path(tmp_path, monkeypatch):
    """Enforcement observes: the served records come from what the op layer really dispatched. An activation that is
    quietly computed by torch instead of the contract's kernel makes the first forward refuse."""
    import torch

    from skyrl_isoexec_b200.core import ledger as LG
    from skyrl_isoexec_b200.core import observe
    from skyrl_isoexec_b200.ops import functional as F

    tr = _tiny_trainer(tmp_path)
    m = tr.train_step(next(iter(tr.loader)))                       # the honest run closes every phase
    assert m["policy/rollout_train_logprob_bit_mismatches"] == 0
    assert tr.adapter_trainer.ledger.verdict()["ok"] and tr.adapter_engine.ledger.verdict()["ok"]
    rec = tr.adapter_engine.ledger.verdict()["records"]
    assert "cpu_swiglu" in rec["FIRST_FORWARD/served/activation.swiglu"]["detail"]      # observed, with the impl that ran

    def eager_swiglu(x):                                           # same maths, another implementation
        observe.note("activation.swiglu", "torch_eager")
        f = x.shape[1] // 2
        return (torch.nn.functional.silu(x[:, :f].float()) * x[:, f:].float()).to(x.dtype)

    monkeypatch.setattr(F, "swiglu_fwd", eager_swiglu)
    tr2 = _tiny_trainer(tmp_path)
    with pytest.raises(LG.ContractViolation) as ei:
        tr2.train_step(next(iter(tr2.loader)))
    assert "activation.swiglu" in str(ei.value) and "torch_eager" in str(ei.value)


def test_ledger_sees_a_weight_sync_that_did_not_invalidate_the_cache(tmp_path, monkeypatch):
    """The installed_backstop records come from the invalidation hooks' own counters, not from the caller's word."""
    tr = _tiny_trainer(tmp_path)
    tr.train_step(next(iter(tr.loader)))
    assert tr.adapter_engine.ledger.verdict()["ok"]
    monkeypatch.setattr(tr.engine.cache, "invalidate", lambda event: False)           # a hook that no longer does its job
    tr.sync_weights()
    v = tr.adapter_engine.ledger.verdict()
    assert not v["ok"] and any("invalidate:engine_kv_cache" in m for m in v["violations"])


def test_install_fingerprint_is_taken_from_the_library_on_the_models_device(tmp_path):
    """A contract that names sm100 kernels cannot be attested by a model that lives on the CPU."""
    from skyrl_isoexec_b200.core import ledger as LG
    from skyrl_isoexec_b200.core.adapter import ContractAdapter
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM

    model = DecoderLM(get_config("tiny-qwen3"), device="cpu", seed=0)
    ok = ContractAdapter("trainer", model)
    ok.run_install()
    assert ok.library["version"] >= 1 and not ok.library["missing"] and ok.ledger.verdict()["ok"]
    with pytest.raises(LG.ContractViolation) as ei:
        ContractAdapter("trainer", model, arch="sm100").run_install()
    assert "wrong-device" in str(ei.value)
