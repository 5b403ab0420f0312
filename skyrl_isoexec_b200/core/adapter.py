"""ContractAdapter: drives contract enforcement for one runtime (trainer or engine).

``run_install`` = build the contract -> check every claim against the live deployment -> record
what is actually installed per (op, site) -> compare that fingerprint with the contract ->
close the INSTALL phase. ``on_first_forward`` reports the served counters, ``on_weight_sync``
the handshake and state invalidation, ``on_gate`` the step-1 forward gate
(reference: ISO/core/adapter.py:48-134,182-261,288-411; ISO/core/fingerprint.py:46-206).

In this framework both runtimes execute the same ``DecoderLM`` through ``ops.functional``, so
"what is installed" is read off the dispatch the model will take on its device: the native
sm_100a library on a GPU, the C++ CPU library otherwise. The fingerprint also pins the
library build (its version symbol) and the model's numerics constants.
"""

from __future__ import annotations

import importlib
from collections import Counter
from dataclasses import dataclass, field

from ..contract import model as M
from . import ledger as L
from . import process as P
from .arch import detect_arch
from .compose import (ContractBuildError, build_execution_contract, derive_selections, profile_from_model_config)
from .declarations import build_registry


@dataclass
class InstallRecord:
    op: str
    site: str
    impl_id: str
    pinned: dict
    obj: str = ""


class Fingerprint:
    """What the process actually installed, keyed by (op, site)."""

    def __init__(self):
        self.records: dict[tuple[str, str], InstallRecord] = {}

    def record_install(self, op: str, site: str, impl_id: str, obj=None, pinned: dict | None = None) -> None:
        self.records[(op, site)] = InstallRecord(op, site, impl_id, dict(pinned or {}),
                                                 getattr(obj, "__qualname__", repr(obj)) if obj is not None else "")

    def compare(self, contract: M.ExecutionContract, side: str) -> list[tuple[str, bool, str]]:
        """[(key, ok, detail)] for every (op, site) the contract expects on ``side``."""
        role = {c.id: c.runtime_role for c in contract.cases}
        out = []
        for e in contract.composition:
            for cid in e.cases:
                if role[cid] != side:
                    continue
                for op in e.region:
                    rec = self.records.get((op, cid))
                    key = f"{op}@{cid}"
                    if rec is None:
                        out.append((key, False, "nothing installed"))
                        continue
                    if op == e.region[0] or op in e.region:
                        ok = rec.impl_id == e.impl.id
                        detail = "" if ok else f"installed {rec.impl_id!r}, contract says {e.impl.id!r}"
                        if ok:
                            consts = dict(e.constants)
                            for k, v in rec.pinned.items():
                                want = consts.get(k)
                                if isinstance(want, M.BitPattern):
                                    want = want.value()
                                if isinstance(want, list):
                                    want = tuple(want)
                                if k in consts and want != (tuple(v) if isinstance(v, list) else v):
                                    ok, detail = False, f"pin {k}: live {v!r} != contract {want!r}"
                        out.append((key, ok, detail))
        return out

    def table(self) -> str:
        rows = [f"  {op:<28} {site:<15} {r.impl_id}" for (op, site), r in sorted(self.records.items())]
        return "installed implementations:\n" + "\n".join(rows)


def resolve_ref(ref: str) -> bool:
    """True if ``path::Symbol[.attr]`` names real code in this package (hook / proof refs)."""
    if "::" not in ref:
        return False
    path, sym = ref.split("::", 1)
    if not path.endswith(".py"):
        return False
    mod = path[:-3].replace("/", ".")
    try:
        obj = importlib.import_module(mod)
    except Exception:  # noqa: BLE001
        return False
    for part in sym.split("."):
        if not hasattr(obj, part):
            return False
        obj = getattr(obj, part)
    return True


class ContractAdapter:
    def __init__(self, side: str, model, rank: int = 0, trainer_tp: int | None = None, engine_tp: int | None = None,
                 arch: str | None = None, trainer_pp: int | None = None):
        self.side = side
        self.model = model
        self.rank = rank
        ps = model.ps
        self.trainer_tp = trainer_tp if trainer_tp is not None else ps.tp
        self.engine_tp = engine_tp if engine_tp is not None else ps.tp
        self.trainer_pp = trainer_pp if trainer_pp is not None else ps.pp
        self.arch = arch or detect_arch(model.device_)
        self.fingerprint = Fingerprint()
        self.served: Counter = Counter()
        self.contract: M.ExecutionContract | None = None
        self.ledger: L.Ledger | None = None
        self.selections = None

    # ------------------------------------------------------------------ INSTALL
    def build_contract(self) -> M.ExecutionContract:
        cfg, ps = self.model.cfg, self.model.ps
        profile = profile_from_model_config(cfg, self.trainer_tp, self.engine_tp, self.trainer_pp, ps.cp, ps.ep)
        reg = build_registry()
        self.selections = derive_selections(profile, self.arch)
        return build_execution_contract(profile, reg, self.selections, self.arch)

    def check_all_claims(self) -> None:
        c, lg, ps = self.contract, self.ledger, self.model.ps
        live = {"tp": ps.tp, "pp": ps.pp, "cp": ps.cp, "ep": ps.ep}
        for t in c.claims.topology:
            deg = live.get(t.axis, 1)
            if t.kind == "pinned":
                # a pinned TP names the common degree of both sides
                ok = deg == t.degree
                lg.report("domain_check", f"topology:{t.axis}", ok, "" if ok else f"live degree {deg} != pinned {t.degree}")
            else:
                ok = deg in t.domain and (t.proof is None or resolve_ref(t.proof))
                lg.report("domain_check", f"topology:{t.axis}", ok,
                          "" if ok else f"live degree {deg} outside {t.domain} or proof {t.proof!r} unresolved")
        for s in c.claims.state:
            ok = resolve_ref(s.ref)
            lg.report("hook_exists", f"state:{s.state_id}", ok, "" if ok else f"hook {s.ref!r} does not resolve")

    def install(self) -> None:
        """Record, per (op, site) of this side, what the library on the model's device can really serve: the contract's
        implementation id only if every entry point that implements it resolves in the loaded library of that device
        kind (a CPU model under an sm100 contract, or a library built without a kernel, records a marker instead and
        the comparison with the contract fails). The library's version and export digest are pinned in the record."""
        from ..ops import _cpu, _native
        from . import observe

        gpu = self.model.device_.type == "cuda"
        lib = _native.lib() if gpu else _cpu.lib()     # raises if the library is missing: no silent fallback
        self.library = observe.library_fingerprint(lib, gpu)
        role = {c.id: c.runtime_role for c in self.contract.cases}
        for e in self.contract.composition:
            for cid in e.cases:
                if role[cid] != self.side:
                    continue
                seen = observe.installed_impl(lib, e.impl.id, gpu)
                for op in e.region:             # the ops a fused implementation subsumes are installed with it
                    self.fingerprint.record_install(op, cid, seen, obj=lib, pinned={})
        # pins: what this process would run with, read from the live model configuration
        live = {k: dict(s.pins) for k, s in derive_selections(
            profile_from_model_config(self.model.cfg, self.trainer_tp, self.engine_tp, self.trainer_pp, self.model.ps.cp,
                                      self.model.ps.ep), self.arch).items()}
        for (op, site), pins in live.items():
            rec = self.fingerprint.records.get((op, site))
            if rec is not None:
                rec.pinned = pins

    def run_install(self) -> M.ExecutionContract:
        try:
            self.contract = P.set_process_contract(self.build_contract())
        except (ContractBuildError, Exception) as e:  # noqa: BLE001
            L.refuse(f"contract build failed: {e}")
            raise
        self.ledger = L.Ledger(self.contract, self.side, self.rank)
        self.ledger.report("build_valid", "contract", True)
        self.check_all_claims()
        self.install()
        for key, ok, detail in self.fingerprint.compare(self.contract, self.side):
            self.ledger.report("install_attest", key, ok, detail)
            self.ledger.report("fingerprint", key, ok, detail)
        P.register_contract_extension("install_attestation", self.attestation_digest)
        self.ledger.close_phase("INSTALL")
        return self.contract

    def attestation_digest(self) -> str:
        """Symmetric digest: the contract's own view when the local installs match it, else a marker
        that can never equal the peer's digest."""
        bad = [k for k, ok, _ in self.fingerprint.compare(self.contract, self.side) if not ok]
        if bad:
            return "INSTALL-MISMATCH:" + ",".join(sorted(bad))
        view = {(op, cid): e.impl.id for e in self.contract.composition for cid in e.cases for op in e.region}
        return L.install_attestation_digest(view)

    # ------------------------------------------------------------------ FIRST_FORWARD
    def note_served(self, ops) -> None:
        """Manual credit (tests, external runtimes). The trainer feeds ``on_first_forward`` with an observed census instead."""
        for op in ops:
            self.served[op] += 1

    def expected_impls(self) -> dict[str, set]:
        """{op: implementation ids the contract names for it on this side}; subsumed ops map to their fused entry's id."""
        role = {c.id: c.runtime_role for c in self.contract.cases}
        out: dict[str, set] = {}
        for e in self.contract.composition:
            if any(role[c] == self.side for c in e.cases):
                for op in e.region:
                    out.setdefault(op, set()).add(e.impl.id)
        return out

    def on_first_forward(self, census=None, not_on_this_rank=()) -> None:
        """Close FIRST_FORWARD. ``census``: {(op, impl id): calls} observed by the op layer during the forward being
        judged (``core.observe.diff``). An op is served iff something ran for it and everything that ran for it is an
        implementation the contract names; an op that a fused kernel subsumes is served when its owner is.
        ``not_on_this_rank``: ops that belong to layers another pipeline stage holds."""
        from . import observe

        lg = self.ledger
        want = self.expected_impls()
        primary = {op for (op, site) in (self.selections or {})}
        owner: dict[str, str] = {}
        for e in self.contract.composition:
            own = next((op for op in e.region if op in primary), e.region[0])
            for op in e.region:
                owner.setdefault(op, own)
        for o in [o for o in lg.plan if o.phase == "FIRST_FORWARD" and o.kind == "served"]:
            if census is None:
                n = self.served.get(o.key, 0)
                lg.report("served", o.key, n > 0, "" if n > 0 else "declared but never executed in the first forward")
                continue
            op = owner.get(o.key, o.key)
            if op in not_on_this_rank or o.key in not_on_this_rank:
                # a pipeline stage owns a subset of the layers: ops of layers it does not hold run on another stage
                lg.report("served", o.key, True, "served by another pipeline stage")
                continue
            got = observe.ran(census, op)
            if not got and self.served.get(o.key, 0) > 0:
                got = {next(iter(want.get(op, {"?"}))): self.served[o.key]}
            bad = sorted(set(got) - want.get(op, set()))
            if not got:
                lg.report("served", o.key, False, f"nothing ran for {op!r} during the first forward")
            elif bad:
                lg.report("served", o.key, False, f"{op!r} was served by {bad}, the contract names {sorted(want.get(op, set()))}")
            else:
                lg.report("served", o.key, True, ",".join(f"{k}x{v}" for k, v in sorted(got.items())))
        lg.close_phase("FIRST_FORWARD")

    # ------------------------------------------------------------------ WEIGHT_SYNC / STEP1
    def on_weight_sync(self, peer_hash: str | None, invalidated=None) -> None:
        lg = self.ledger
        mine = P.contract_hash(self.contract)
        ok = peer_hash == mine
        lg.report("handshake", "contract_hash", ok, "" if ok else f"peer {str(peer_hash)[:12]} != local {mine[:12]}")
        # ``invalidated``: {state id: observed} from the invalidation hooks' own counters (a list of ids is read as
        # "the caller vouches", kept for runtimes that cannot observe)
        obs = invalidated if isinstance(invalidated, dict) else {sid: True for sid in (invalidated or [])}
        for sid, seen in obs.items():
            lg.report("installed_backstop", f"invalidate:{sid}", bool(seen),
                      "" if seen else "the state's invalidation hook did not run for this weight sync")
        if "WEIGHT_SYNC" not in lg.closed:
            lg.close_phase("WEIGHT_SYNC")

    def on_gate(self, ok: bool, detail: str = "") -> None:
        self.ledger.report("gate", "forward_gate", ok, detail)
        if "STEP1" not in self.ledger.closed:
            self.ledger.close_phase("STEP1")


def served_ops_of(cfg) -> list[str]:
    """Logical ops one forward of ``cfg`` executes (used to feed the served counters)."""
    ops = ["mm", "attention.varlen", "rope.rope", "norms.rms", "norms.qk", "activation.swiglu", "logprobs.log_softmax",
           "collectives.tree_all_reduce", "collectives.row_parallel"]
    if cfg.attn_output_gate:
        ops.append("activation.attn_gate")
    if cfg.has_gdn:
        ops += ["gdn.core", "gdn.conv", "gdn.gating", "gdn.state", "norms.gated_out"]
    if cfg.has_moe:
        ops += ["moe.router", "moe.dispatch", "moe.experts", "moe.combine"]
    return ops
