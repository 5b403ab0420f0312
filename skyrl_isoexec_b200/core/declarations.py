"""Declarative registry entries for every op family, registered in the fixed order
``mm, attention, rope, norms, activation, logprobs, gdn, moe, collectives`` (the reference keeps
one ``_register.py`` per family and imports them in that order, ISO/core/registry_build.py:18-61).

Each op has one sm_100a implementation (a hand-written kernel in ``csrc/``) shared by all four
sites, and a ``cpu_*`` restatement (``csrc_cpu/ops_cpu.cpp``) with the same reduction order that
serves the CPU/gloo configuration and is the test oracle. Where trainer and engine sites run
different code (GDN chunked scan vs recurrent decode, dense vs sampled-row LM head) the pair is
declared asymmetric and carries a discharge.
"""

from __future__ import annotations

from .registry import ENGINE_SITES, SITES, TRAINER_SITES, ImplSpec, OneOf, OpSpec, PER_MODEL, Registry, RoundingSchedule

BOTH = frozenset({"sm100", "cpu"})
GPU = frozenset({"sm100"})
CPU = frozenset({"cpu"})


def _mm(r: Registry):
    r.add_op(OpSpec("mm", doc="dense x @ w^T on the logprob path (QKV, out-proj, MLP, LM head)"))
    r.add_impl(ImplSpec(
        "mm", "tcgen05_batch_invariant", 1, GPU,
        RoundingSchedule.of("fp32 TMEM accumulation over ascending 64-wide K blocks, four K=16 tcgen05.mma steps per "
                            "block, one bf16 round in the epilogue; no split-K; N tile chosen from (M bucket, N) only",
                            block_k=64, mma_k=16, split_k=1, accum="fp32_tmem", tile_m=128,
                            tile_n=OneOf(32, 64, 128, 256)),
        capabilities=frozenset({"m_invariant", "tile_invariant", "cuda_graph"}),
        hazards=("profiling_shapes", "non_contiguous", "subnormals"), kernel="csrc/gemm_tcgen05.cu"))
    r.add_impl(ImplSpec(
        "mm", "cpu_sequential_k", 1, CPU,
        RoundingSchedule.of("fp32 accumulation over ascending k, separate multiply and add, one round to the "
                            "activation dtype", split_k=1, accum="fp32_sequential"),
        capabilities=frozenset({"m_invariant"}), hazards=("non_contiguous",), kernel="csrc_cpu/ops_cpu.cpp"))


def _attention(r: Registry):
    r.add_op(OpSpec("attention.varlen", doc="causal GQA attention, packed (trainer) or paged (engine) keys"))
    sched = RoundingSchedule.of(
        "keys in 128-wide blocks aligned to position 0, ascending, never split; per block S=QK^T (fp32), t=S*scale*log2e, "
        "row max, alpha=exp2(m_old-m_new), O=O*alpha (+ previous block's PV), p=exp2(t-m) summed left to right, P rounded "
        "to the activation dtype before P@V; final O/l rounded once",
        num_splits=1, block_n=128, window=(-1, 0), softmax_domain="log2", p_dtype=PER_MODEL)
    r.add_impl(ImplSpec("attention.varlen", "tcgen05_unified", 1, GPU, sched,
                        capabilities=frozenset({"paged", "packed", "gqa_packed_rows", "chunked_prefill"}),
                        hazards=("null_lanes", "t_zero", "profiling_shapes"), kernel="csrc/attention_tcgen05.cu"))
    r.add_impl(ImplSpec("attention.varlen", "cpu_blockwise", 1, CPU, sched,
                        capabilities=frozenset({"paged", "packed"}), hazards=("null_lanes", "t_zero"),
                        kernel="csrc_cpu/ops_cpu.cpp"))


def _rope(r: Registry):
    r.add_op(OpSpec("rope.rope", doc="rotate-half RoPE indexed by absolute position, fused with QK-norm and the KV write"))
    sched = RoundingSchedule.of("cos/sin table fp32 from fp64 host math; x*cos, rot(x)*sin and their sum each rounded to the "
                                "activation dtype (three rounds), negation as x*(-1.0)",
                                rounds=3, table="fp32_from_fp64", rot_dim=PER_MODEL, theta=PER_MODEL)
    r.add_impl(ImplSpec("rope.rope", "fused_qknorm_rope_kvwrite", 1, GPU, sched, subsumes=("norms.qk",),
                        hazards=("signed_zero", "non_contiguous"), kernel="csrc/norm_rope.cu"))
    r.add_impl(ImplSpec("rope.rope", "cpu_fused_qknorm_rope", 1, CPU, sched, subsumes=("norms.qk",),
                        hazards=("signed_zero",), kernel="csrc_cpu/ops_cpu.cpp"))


def _norms(r: Registry):
    r.add_op(OpSpec("norms.rms", doc="RMSNorm of the residual stream, optionally fused with the residual add"))
    r.add_op(OpSpec("norms.qk", doc="per-head RMSNorm of q and k"))
    r.add_op(OpSpec("norms.gated_out", doc="GatedDeltaNet output norm: rms_norm(o) * g * silu(z)"))
    chain = ("sum of squares: lane l of 32 takes 8-wide vectors l, l+32, ... ascending, xor butterfly 16,8,4,2,1; "
             "rstd = 1/sqrt(ss/N+eps) with IEEE div and sqrt; x*rstd rounded, gamma (w or round(1+w)) product rounded")
    sched = RoundingSchedule.of(chain, lanes=32, vec=8, eps=PER_MODEL, zero_centered=PER_MODEL, rsqrt="div_sqrt_rn")
    for op, gid, cid, sub in (("norms.rms", "fused_add_rmsnorm", "cpu_add_rmsnorm", ()),
                              ("norms.gated_out", "fused_gated_outnorm", "cpu_gated_outnorm", ())):
        r.add_impl(ImplSpec(op, gid, 1, GPU, sched, subsumes=sub, hazards=("subnormals", "non_contiguous"),
                            kernel="csrc/norm_rope.cu"))
        r.add_impl(ImplSpec(op, cid, 1, CPU, sched, subsumes=sub, hazards=("subnormals",), kernel="csrc_cpu/ops_cpu.cpp"))


def _activation(r: Registry):
    r.add_op(OpSpec("activation.swiglu", doc="silu(gate) * up on the fused gate_up projection"))
    r.add_op(OpSpec("activation.attn_gate", doc="sigmoid output gate of gated attention"))
    sched = RoundingSchedule.of("silu(g) = g / (1 + exp(-g)) in fp32 rounded once, product with up rounded once", rounds=2)
    r.add_impl(ImplSpec("activation.swiglu", "fused_swiglu", 1, GPU, sched, hazards=("subnormals",), kernel="csrc/norm_rope.cu"))
    r.add_impl(ImplSpec("activation.swiglu", "cpu_swiglu", 1, CPU, sched, kernel="csrc_cpu/ops_cpu.cpp"))
    r.add_impl(ImplSpec("activation.attn_gate", "fused_sigmoid_gate", 1, GPU, sched, kernel="csrc/norm_rope.cu"))
    r.add_impl(ImplSpec("activation.attn_gate", "cpu_sigmoid_gate", 1, CPU, sched, kernel="csrc_cpu/ops_cpu.cpp"))


def _logprobs(r: Registry):
    r.add_op(OpSpec("logprobs.log_softmax", doc="sampled-token log-probability, row-count and TP invariant"))
    r.add_op(OpSpec("logprobs.lm_head_slice", sites=ENGINE_SITES, doc="LM head evaluated on the sampled rows only"))
    sched = RoundingSchedule.of(
        "m = exact row max; G equal vocab leaves; per leaf Kahan fp32 sum of exp(x-m) over 4096-column blocks, block sum "
        "= 256 threads x 16 columns, butterfly, 8 warp partials left to right; leaves folded by adjacent pairs; "
        "logprob = (x_t - m) - log(S)", leaves=PER_MODEL, block=4096, threads=256, accum="kahan_fp32")
    r.add_impl(ImplSpec("logprobs.log_softmax", "rowinv_leaftree", 1, GPU, sched,
                        capabilities=frozenset({"tp_invariant", "row_invariant", "fused_single_launch"}),
                        hazards=("tie_boundaries", "subnormals", "null_lanes"), kernel="csrc/logprob.cu"))
    r.add_impl(ImplSpec("logprobs.log_softmax", "cpu_rowinv_leaftree", 1, CPU, sched,
                        capabilities=frozenset({"tp_invariant", "row_invariant"}), hazards=("tie_boundaries",),
                        kernel="csrc_cpu/ops_cpu.cpp"))
    for arch, iid in ((GPU, "sampled_rows"), (CPU, "cpu_sampled_rows")):
        r.add_impl(ImplSpec("logprobs.lm_head_slice", iid, 1, arch,
                            RoundingSchedule.of("row gather before the LM-head GEMM; the GEMM is row-invariant"),
                            route="reference_preserving", reference="tcgen05_batch_invariant" if arch is GPU else "cpu_sequential_k",
                            kernel="engine/llm_engine.py"))


def _gdn(r: Registry):
    r.add_op(OpSpec("gdn.core", doc="gated delta rule: chunked scan (trainer) / recurrent update (engine)"))
    r.add_op(OpSpec("gdn.conv", doc="width-4 causal depthwise conv + SiLU over q|k|v"))
    r.add_op(OpSpec("gdn.gating", doc="g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b), q/k L2 norm"))
    r.add_op(OpSpec("gdn.state", sites=ENGINE_SITES, doc="recurrent + conv state pool keyed by sequence slot"))
    core = RoundingSchedule.of(
        "state fp32 [Hv, V, K]; per token S = S*exp(g); u = beta*(v - S k); S += u k^T; o = S q*K^-0.5, k/q L2-normalised; "
        "chunk boundary states chained in fp32 and snapshotted to the activation dtype every `chunk` tokens; the "
        "within-chunk scan restarts from the snapshot so the chunked scan and token-by-token decode share every "
        "rounding point", kernel=OneOf("cpr", "recurrent"), chunk=PER_MODEL, state_dtype="fp32", snapshot_dtype=PER_MODEL)
    for arch, sfx in ((BOTH, ""),):
        r.add_impl(ImplSpec("gdn.core", "cpr_chunk_scan", 1, arch, core, sites=TRAINER_SITES + ("engine_prefill",),
                            hazards=("t_zero", "null_lanes"), kernel="ops/gdn.py"))
        r.add_impl(ImplSpec("gdn.core", "cpr_recurrent_step", 1, arch, core, sites=("engine_decode",),
                            route="reference_preserving", reference="cpr_chunk_scan", state_invalidation=("weight_sync", "sleep_wake"),
                            hazards=("t_zero", "null_lanes"), kernel="ops/gdn.py"))
        r.add_impl(ImplSpec("gdn.conv", "shifted_sum_conv", 1, arch,
                            RoundingSchedule.of("taps accumulated in fp32 oldest to newest, x*sigmoid(x), one round",
                                                width=PER_MODEL, rounds=1),
                            hazards=("t_zero",), kernel="ops/gdn.py"))
        r.add_impl(ImplSpec("gdn.gating", "fp32_gating", 1, arch,
                            RoundingSchedule.of("softplus, exp and sigmoid in fp32 with IEEE division; L2 norm by the fixed "
                                                "lane order of norms.rms", l2_eps=PER_MODEL), kernel="ops/gdn.py"))
        r.add_impl(ImplSpec("gdn.state", "slot_pool", 1, arch,
                            RoundingSchedule.of("fp32 recurrent state rows + conv tail rows indexed by slot; row 0 is the "
                                                "null lane", state_dtype="fp32"),
                            state_invalidation=("weight_sync", "sleep_wake"), kernel="engine/gdn_state.py"))


def _moe(r: Registry):
    r.add_op(OpSpec("moe.router", doc="fp32 router logits, top-k with lower-index ties, gate weights"))
    r.add_op(OpSpec("moe.dispatch", doc="stable counting-sort permutation of (token, slot) rows by expert"))
    r.add_op(OpSpec("moe.experts", doc="per-expert fc1 -> SwiGLU x gate weight -> fc2"))
    r.add_op(OpSpec("moe.combine", doc="fixed-order top-k sum: ascending expert index, fp32, one final round"))
    for arch, pfx in ((GPU, ""), (CPU, "cpu_")):
        mmref = "tcgen05_batch_invariant" if arch is GPU else "cpu_sequential_k"
        r.add_impl(ImplSpec("moe.router", pfx + "deterministic_topk", 1, arch,
                            RoundingSchedule.of("logits by the batch-invariant GEMM with fp32 output; softmax over E with the "
                                                "norms.rms lane order; k argmax rounds, tie -> lower expert index; optional "
                                                "renormalisation by the sequential sum of the k weights",
                                                topk=PER_MODEL, tie="lower_index", score=OneOf("softmax", "sigmoid_bias"),
                                                norm_topk=PER_MODEL), hazards=("tie_boundaries",), kernel="ops/moe.py"))
        r.add_impl(ImplSpec("moe.dispatch", pfx + "index_build", 1, arch,
                            RoundingSchedule.of("integer only: rows ordered by (expert, token, slot)"), kernel="ops/moe.py"))
        r.add_impl(ImplSpec("moe.experts", pfx + "grouped_gemm", 1, arch,
                            RoundingSchedule.of("fc1 and fc2 by the batch-invariant GEMM per expert row group; gate weight "
                                                "applied to the SwiGLU output before fc2 with one round; fc2 output fp32",
                                                prob_before_fc2=True, fc2_out="fp32"),
                            route="reference_preserving", reference=mmref, hazards=("e_mismatch", "t_zero"), kernel="ops/moe.py"))
        r.add_impl(ImplSpec("moe.combine", pfx + "fixed_order", 1, arch,
                            RoundingSchedule.of("per token: fp32 sum of its k expert rows in ascending expert index, then "
                                                "one round; shared-expert output added after", order="ascending_expert",
                                                accum="fp32", rounds=1), hazards=("tie_boundaries",), kernel="ops/moe.py"))


def _collectives(r: Registry):
    r.add_op(OpSpec("collectives.tree_all_reduce", doc="fixed balanced-tree all-reduce over TP partials"))
    r.add_op(OpSpec("collectives.row_parallel", doc="row-parallel linear = local leaf subtree + tree all-reduce"))
    r.add_op(OpSpec("collectives.nccl_pin", doc="NCCL only moves bytes on the logprob path; no NCCL reduction is used"))
    tree = RoundingSchedule.of("K cut into `leaves` equal leaves; a rank owns leaves/tp consecutive leaves (one subtree); "
                               "fold by stride 1,2,4.. with the lower index on the left; internal nodes fp32; optional "
                               "rounding only at the leaf boundary", leaves=PER_MODEL, leaf_dtype=OneOf("fp32", "bf16"),
                               internal="fp32")
    for arch, pfx in ((GPU, ""), (CPU, "cpu_")):
        r.add_impl(ImplSpec("collectives.tree_all_reduce", pfx + "pik_tree", 1, arch, tree,
                            capabilities=frozenset({"tp_invariant"}), hazards=("signed_zero",), kernel="parallel/tp.py"))
        r.add_impl(ImplSpec("collectives.row_parallel", pfx + "pik_tree", 1, arch, tree,
                            capabilities=frozenset({"tp_invariant"}), kernel="parallel/tp.py"))
        r.add_impl(ImplSpec("collectives.nccl_pin", pfx + "bytes_only", 1, arch,
                            RoundingSchedule.of("all_gather / all_to_all / broadcast only on the forward path; any reduction "
                                                "is a local kernel with the declared tree", reductions_on_wire=0),
                            kernel="parallel/tp.py"))


FAMILIES = {"mm": _mm, "attention": _attention, "rope": _rope, "norms": _norms, "activation": _activation,
            "logprobs": _logprobs, "gdn": _gdn, "moe": _moe, "collectives": _collectives}


def build_registry() -> Registry:
    from .registry import FAMILY_ORDER

    r = Registry()
    for fam in FAMILY_ORDER:
        FAMILIES[fam](r)
    r.check()
    return r
