"""From a model to its ExecutionContract: profile -> selections -> contract.

* ``ModelProfile`` holds structural facts only (no implementation choices): which op families
  the architecture has, the pinned numerics constants, and the topology / state / tolerance
  facts it claims (reference: ISO/models/profile.py:28-319).
* ``derive_selections`` is the model-independent composition table: which implementation runs
  at each (op, site) with which pins (reference: ISO/models/policy.py:99-257).
* ``build_execution_contract`` freezes the selections into entries (identical selections merge
  into one entry, region = op + subsumed ops, float pins become fp64 bit patterns), validates
  the pins against each implementation's rounding schedule, attaches discharges to asymmetric
  regions and stamps the three identities (reference: ISO/core/contract_build.py:39-51,290-435).
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field

from ..contract import model as M
from ..contract.digest import compute_identities
from ..contract.rules import validate_or_raise
from ..models.config import ModelConfig
from .registry import ENGINE_SITES, SITES, TRAINER_SITES, Registry

CASES = (
    M.ExecutionCase("engine_decode", "engine", "no_grad", "continued", "shape_static",
                    ("cudagraph_capturable", "host_free", "address_stable")),
    M.ExecutionCase("engine_prefill", "engine", "no_grad", "resumable", "variable", ()),
    M.ExecutionCase("trainer_fwd", "trainer", "grad", "checkpoint_recompute", "variable", ("includes_grad_recompute",)),
    M.ExecutionCase("trainer_score", "trainer", "no_grad", "fresh", "variable", ()),
)


class ContractBuildError(Exception):
    pass


@dataclass(frozen=True)
class TopologyAxisFact:
    axis: str
    kind: str                      # "pinned" | "invariant"
    degree: int | None = None
    domain: tuple[int, ...] = ()
    collective_plan: str | None = None
    proof: str | None = None


@dataclass(frozen=True)
class StateFact:
    state_id: str
    invalidated_by: tuple[str, ...]
    replay_safe: bool
    ref: str


@dataclass(frozen=True)
class ToleranceFact:
    case_pair: tuple[str, str]
    bounds: tuple                 # ((name, decimal string), ...)
    attributed_to: tuple[str, ...] = ()


@dataclass(frozen=True)
class ModelProfile:
    family: str
    architectures: tuple[str, ...]
    profile_ref: str
    has_gdn: bool = False
    has_moe: bool = False
    has_qk_norm: bool = True
    attn_output_gate: bool = False
    zero_centered_norms: bool = False
    activation_dtype: str = "bf16"
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_scaling: str = ""           # canonical JSON of the rope_scaling mapping ("" = none): it changes the cos / sin table
    rot_dim: int = 128
    logprob_leaves: int = 8
    pik_leaves: int = 8
    pik_leaf_dtype: str = "fp32"
    router_score: str = "softmax"
    router_topk: int = 0
    router_norm_topk: bool = True
    gdn_kernel: str = "recurrent"
    gdn_chunk_size: int = 64
    gdn_conv_width: int = 4
    topology: tuple[TopologyAxisFact, ...] = ()
    states: tuple[StateFact, ...] = ()
    tolerances: tuple[ToleranceFact, ...] = ()


def profile_from_model_config(cfg: ModelConfig, trainer_tp: int = 1, engine_tp: int = 1, pp: int = 1, cp: int = 1,
                              ep: int = 1) -> ModelProfile:
    """Structural facts of ``cfg`` plus the topology it is deployed with. TP is claimed *invariant*
    over the divisors of ``pik_leaves`` when the two sides differ or ``cfg.tp_invariant`` is set,
    otherwise pinned to the common degree."""
    G = cfg.pik_leaves
    tp_proof = "skyrl_isoexec_b200/parallel/tp.py::tree_all_reduce"
    if cfg.tp_invariant or trainer_tp != engine_tp:
        dom = tuple(d for d in (1, 2, 4, 8, 16, 32, 64) if d <= G and G % d == 0)
        if trainer_tp not in dom or engine_tp not in dom:
            raise ContractBuildError(f"TP degrees {trainer_tp}/{engine_tp} are outside the invariant domain {dom}")
        tp_fact = TopologyAxisFact("tp", "invariant", domain=dom, proof=tp_proof)
    else:
        tp_fact = TopologyAxisFact("tp", "pinned", degree=trainer_tp,
                                   collective_plan=f"pik-tree:G={G}:leaf=fp32" if trainer_tp > 1 else "none")
    topo = [tp_fact,
            # a stage boundary moves the (x, residual) pair as bytes: with a pipelined trainer the engines (pp = 1) and the
            # trainer (pp stages) compute the same function, which the claim states as invariance over both degrees
            (TopologyAxisFact("pp", "pinned", degree=1, collective_plan="nccl-p2p-bytes-only") if pp == 1 else
             TopologyAxisFact("pp", "invariant", domain=(1, pp), proof="skyrl_isoexec_b200/parallel/pp.py::PipelinePolicyWorker")),
            TopologyAxisFact("cp", "pinned", degree=cp, collective_plan="none" if cp == 1 else "ulysses-a2a-bytes-only")]
    if cfg.has_moe:
        topo.append(TopologyAxisFact("ep", "invariant", domain=(1, 2, 4, 8),
                                     proof="skyrl_isoexec_b200/ops/moe.py::combine_fixed_order"))
    states = [StateFact("engine_kv_cache", ("weight_sync", "sleep_wake"), False,
                        "skyrl_isoexec_b200/engine/kv_cache.py::KVCache.sleep")]
    if cfg.has_gdn:
        states.append(StateFact("gdn_recurrent_state", ("weight_sync", "sleep_wake"), False,
                                "skyrl_isoexec_b200/engine/gdn_state.py::GDNStatePool.invalidate"))
    tol = (ToleranceFact(("engine_decode", "trainer_score"), (("max_abs_logprob_diff", "0"), ("mean_abs_logprob_diff", "0")),
                         ("mm", "attention.varlen", "logprobs.log_softmax")),)
    return ModelProfile(
        family=cfg.name, architectures=(cfg.architecture,), profile_ref=f"skyrl_isoexec_b200/models/config.py::{cfg.name}",
        has_gdn=cfg.has_gdn, has_moe=cfg.has_moe, has_qk_norm=cfg.qk_norm, attn_output_gate=cfg.attn_output_gate,
        zero_centered_norms=cfg.zero_centered_norm, activation_dtype="bf16" if cfg.dtype == "bfloat16" else "fp32",
        rms_eps=cfg.rms_eps, rope_theta=cfg.rope_theta,
        rope_scaling=__import__("json").dumps(dict(cfg.rope_scaling), sort_keys=True) if getattr(cfg, "rope_scaling", ()) else "", rot_dim=cfg.rot_dim, logprob_leaves=cfg.logprob_leaves,
        pik_leaves=G, router_score=cfg.router, router_topk=cfg.top_k, router_norm_topk=cfg.norm_topk_prob,
        gdn_kernel="cpr" if getattr(cfg, "gdn_snapshot", False) else "recurrent", gdn_chunk_size=cfg.gdn_chunk, gdn_conv_width=cfg.gdn_conv_kernel, topology=tuple(topo), states=tuple(states),
        tolerances=tol)


@dataclass(frozen=True)
class Selection:
    impl_id: str
    pins: tuple = ()              # sorted ((key, value), ...)

    @staticmethod
    def of(impl_id: str, **pins) -> "Selection":
        return Selection(impl_id, tuple(sorted(pins.items())))


def derive_selections(p: ModelProfile, arch: str) -> dict[tuple[str, str], Selection]:
    """The composition table: {(op, site): Selection}. ``arch`` is "sm100" or "cpu"."""
    gpu = arch != "cpu"
    x = (lambda g, c: g if gpu else c)
    sel: dict[tuple[str, str], Selection] = {}

    def put(op, sites, s):
        for site in sites:
            sel[(op, site)] = s

    put("mm", SITES, Selection.of(x("tcgen05_batch_invariant", "cpu_sequential_k"),
                                  **(dict(block_k=64, mma_k=16, split_k=1, accum="fp32_tmem", tile_m=128, tile_n=256)
                                     if gpu else dict(split_k=1, accum="fp32_sequential"))))
    put("attention.varlen", SITES, Selection.of(x("tcgen05_unified", "cpu_blockwise"), num_splits=1, block_n=128,
                                                window=(-1, 0), softmax_domain="log2", p_dtype=p.activation_dtype))
    put("rope.rope", SITES, Selection.of(x("fused_qknorm_rope_kvwrite", "cpu_fused_qknorm_rope"), rounds=3,
                                         table="fp32_from_fp64", rot_dim=p.rot_dim, theta=p.rope_theta,
                                         **({"scaling": p.rope_scaling} if p.rope_scaling else {})))
    norm_pins = dict(lanes=32, vec=8, eps=p.rms_eps, zero_centered=p.zero_centered_norms, rsqrt="div_sqrt_rn")
    put("norms.rms", SITES, Selection.of(x("fused_add_rmsnorm", "cpu_add_rmsnorm"), **norm_pins))
    put("activation.swiglu", SITES, Selection.of(x("fused_swiglu", "cpu_swiglu"), rounds=2))
    if p.attn_output_gate:
        put("activation.attn_gate", SITES, Selection.of(x("fused_sigmoid_gate", "cpu_sigmoid_gate"), rounds=2))
    put("logprobs.log_softmax", SITES, Selection.of(x("rowinv_leaftree", "cpu_rowinv_leaftree"), leaves=p.logprob_leaves,
                                                    block=4096, threads=256, accum="kahan_fp32"))
    put("logprobs.lm_head_slice", ENGINE_SITES, Selection.of(x("sampled_rows", "cpu_sampled_rows")))
    if p.has_gdn:
        core = dict(kernel=p.gdn_kernel, chunk=p.gdn_chunk_size, state_dtype="fp32", snapshot_dtype=p.activation_dtype)
        put("gdn.core", TRAINER_SITES + ("engine_prefill",), Selection.of("cpr_chunk_scan", **core))
        put("gdn.core", ("engine_decode",), Selection.of("cpr_recurrent_step", **core))
        put("gdn.conv", SITES, Selection.of("shifted_sum_conv", width=p.gdn_conv_width, rounds=1))
        put("gdn.gating", SITES, Selection.of("fp32_gating", l2_eps=1e-6))
        put("gdn.state", ENGINE_SITES, Selection.of("slot_pool", state_dtype="fp32"))
        put("norms.gated_out", SITES, Selection.of(x("fused_gated_outnorm", "cpu_gated_outnorm"), **norm_pins))
    if p.has_moe:
        c = "" if gpu else "cpu_"
        put("moe.router", SITES, Selection.of(c + "deterministic_topk", topk=p.router_topk, tie="lower_index",
                                              score=p.router_score, norm_topk=p.router_norm_topk))
        put("moe.dispatch", SITES, Selection.of(c + "index_build"))
        put("moe.experts", SITES, Selection.of(c + "grouped_gemm", prob_before_fc2=True, fc2_out="fp32"))
        put("moe.combine", SITES, Selection.of(c + "fixed_order", order="ascending_expert", accum="fp32", rounds=1))
    tree = dict(leaves=p.pik_leaves, leaf_dtype=p.pik_leaf_dtype, internal="fp32")
    c = "" if gpu else "cpu_"
    put("collectives.tree_all_reduce", SITES, Selection.of(c + "pik_tree", **tree))
    put("collectives.row_parallel", SITES, Selection.of(c + "pik_tree", **tree))
    put("collectives.nccl_pin", SITES, Selection.of(c + "bytes_only", reductions_on_wire=0))
    return sel


def _const(v):
    if isinstance(v, float):
        return M.BitPattern.of(v, "float64")
    if isinstance(v, (list, tuple)):
        return [_const(x) for x in v]
    return v


def build_execution_contract(profile: ModelProfile, registry: Registry, selections: dict, arch: str) -> M.ExecutionContract:
    if arch not in registry.archs():
        raise ContractBuildError(f"architecture {arch!r} is not declared by any registered implementation "
                                 f"(known: {sorted(registry.archs())})")
    # group identical selections of an op over sites
    groups: dict[tuple, list[str]] = {}
    for (op, site), s in sorted(selections.items()):
        spec = registry.impl(op, s.impl_id)
        opspec = registry.ops[op]
        if site not in opspec.sites:
            raise ContractBuildError(f"op {op!r} is not declared at site {site!r}")
        if spec.sites is not None and site not in spec.sites:
            raise ContractBuildError(f"impl {s.impl_id!r} of {op!r} is not admitted at site {site!r}")
        if arch not in spec.supported_archs:
            raise ContractBuildError(f"impl {s.impl_id!r} of {op!r} is not qualified on {arch!r} "
                                     f"(supported: {sorted(spec.supported_archs)})")
        errs = spec.rounding.check_pin(dict(s.pins))
        if errs:
            raise ContractBuildError(f"{op}@{site} ({s.impl_id}): " + "; ".join(errs))
        groups.setdefault((op, s), []).append(site)
    per_op_impls: dict[str, set] = {}
    for (op, s) in groups:
        per_op_impls.setdefault(op, set()).add(s.impl_id)
    entries = []
    for (op, s), sites in sorted(groups.items(), key=lambda kv: (kv[0][0], kv[0][1].impl_id)):
        spec = registry.impl(op, s.impl_id)
        region = tuple(sorted((op,) + tuple(spec.subsumes)))
        reference = None
        if spec.reference is not None:
            ref_op = op if (op, spec.reference) in registry.impls else next(
                (o for (o, i) in registry.impls if i == spec.reference), op)
            rs = registry.impl(ref_op, spec.reference)
            reference = M.ImplRef(rs.impl_id, rs.version, arch)
        discharge = None
        if len(per_op_impls[op]) > 1:
            discharge = M.EquivalenceProof("bitwise_equal_to", f"skyrl_isoexec_b200/{spec.kernel}::{s.impl_id}")
        entries.append(M.CompositionEntry(
            region=region, cases=tuple(sorted(sites)), impl=M.ImplRef(spec.impl_id, spec.version, arch),
            route=spec.route, constants={k: _const(v) for k, v in s.pins}, artifact=None, reference=reference,
            coverage=M.Coverage("symbolic_domain", spec.rounding.documentary or "row-independent for every shape"),
            discharge=discharge, half="function"))
    claims = M.Claims(
        topology=tuple(M.TopologyClaim(t.axis, t.kind, t.degree, t.collective_plan, tuple(t.domain), t.proof)
                       for t in profile.topology),
        state=tuple(M.StateClaim(s.state_id, tuple(s.invalidated_by), s.replay_safe, s.ref) for s in profile.states),
        tolerances=tuple(M.ToleranceClaim(tuple(t.case_pair), dict(t.bounds), tuple(t.attributed_to))
                         for t in profile.tolerances))
    c = M.ExecutionContract(M.SCHEMA_VERSION, M.ModelRef(profile.family, tuple(profile.architectures), profile.profile_ref),
                            M.Identities("", "", ""), CASES, tuple(entries), claims)
    c = dataclasses.replace(c, identities=compute_identities(c))
    required = {case.id: frozenset(op for (op, site) in selections if site == case.id) for case in CASES}
    validate_or_raise(c, required)
    return c


def contract_for_model(cfg: ModelConfig, arch: str, trainer_tp: int = 1, engine_tp: int = 1, pp: int = 1, cp: int = 1,
                       ep: int = 1, registry: Registry | None = None) -> M.ExecutionContract:
    from .declarations import build_registry

    reg = registry or build_registry()
    prof = profile_from_model_config(cfg, trainer_tp, engine_tp, pp, cp, ep)
    return build_execution_contract(prof, reg, derive_selections(prof, arch), arch)
