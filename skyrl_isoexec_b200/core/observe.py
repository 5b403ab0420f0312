"""What actually ran: a process-wide census of (contract op, implementation id) pairs, incremented by the op layer at
the point where it hands a call to a kernel (reference: the served counters that the reference's installers keep inside
the served paths, ISO/core/enforce.py:80-108,808-859, and ``record_install`` with the live object,
ISO/core/fingerprint.py:73-99).

The contract adapter closes its FIRST_FORWARD phase from the DIFFERENCE of two snapshots taken around the forward it
judges, so an op that was served by another path than the contract names (the per-expert loop instead of the grouped
kernel, a library GEMM instead of the batch-invariant one, the torch sampler instead of the kernel) shows up under a
different implementation id and the ledger refuses.

``IMPL_SYMBOLS`` names, per implementation id, the entry points of the native library that implement it; the install
fingerprint is taken from which of those the loaded library really exports on the device the model lives on.
"""

from __future__ import annotations

import hashlib
from collections import Counter

_CENSUS: Counter = Counter()


def note(op: str, impl: str, n: int = 1) -> None:
    _CENSUS[(op, impl)] += n


def snapshot() -> Counter:
    return Counter(_CENSUS)


def diff(before: Counter) -> Counter:
    """Calls made since ``before`` was taken."""
    out = Counter()
    for k, v in _CENSUS.items():
        d = v - before.get(k, 0)
        if d > 0:
            out[k] = d
    return out


def ran(census: Counter, op: str) -> dict[str, int]:
    return {impl: n for (o, impl), n in census.items() if o == op}


# implementation id -> native entry points that must exist for it to be "installed"
IMPL_SYMBOLS: dict[str, tuple[str, ...]] = {
    # sm_100a library (lib/libisoexec_b200.so)
    "tcgen05_batch_invariant": ("ix_gemm_bf16_nt",),
    "tcgen05_unified": ("ix_attention_fwd",),
    "fused_qknorm_rope_kvwrite": ("ix_qk_norm_rope",),
    "fused_add_rmsnorm": ("ix_rmsnorm",),
    "fused_swiglu": ("ix_swiglu",),
    "fused_sigmoid_gate": ("ix_sigmoid_gate",),
    "fused_gated_outnorm": ("ix_gated_outnorm",),
    "rowinv_leaftree": ("ix_logprob_fused", "ix_logprob_rowmax", "ix_logprob_leafsum", "ix_logprob_finalize"),
    "sampled_rows": ("ix_gemm_bf16_nt",),
    "cpr_chunk_scan": ("ix_gdn_scan", "ix_gdn_chunk_fwd"),
    "cpr_recurrent_step": ("ix_gdn_scan",),
    "shifted_sum_conv": ("ix_gdn_conv",),
    "fp32_gating": ("ix_gdn_gate", "ix_gdn_l2norm"),
    "slot_pool": ("ix_gdn_conv_state",),
    "deterministic_topk": ("ix_router_topk",),
    "index_build": ("ix_moe_dispatch_plan", "ix_moe_gather_rows"),
    "grouped_gemm": ("ix_moe_grouped_gemm",),
    "fixed_order": ("ix_moe_combine",),
    "pik_tree": ("ix_tp_gemm_fused", "ix_peer_tree_reduce", "ix_leaf_split_gemm", "ix_leaftree_gemm_add"),
    "bytes_only": (),
    # C++ CPU library (lib/libisoexec_cpu.so)
    "cpu_sequential_k": ("ixc_gemm_nt",),
    "cpu_blockwise": ("ixc_attention_fwd",),
    "cpu_fused_qknorm_rope": ("ixc_qk_norm_rope",),
    "cpu_add_rmsnorm": ("ixc_rmsnorm",),
    "cpu_swiglu": ("ixc_swiglu",),
    "cpu_sigmoid_gate": ("ixc_sigmoid_gate",),
    "cpu_gated_outnorm": ("ixc_gated_outnorm",),
    "cpu_rowinv_leaftree": ("ixc_logprob_fused", "ixc_logprob_rowmax", "ixc_logprob_leafsum", "ixc_logprob_finalize"),
    "cpu_sampled_rows": ("ixc_gemm_nt",),
    "cpu_deterministic_topk": ("ixc_router_topk",),
    "cpu_index_build": (),
    "cpu_grouped_gemm": ("ixc_gemm_nt",),
    "cpu_fixed_order": (),
    "cpu_pik_tree": ("ixc_leaftree_gemm",),
    "cpu_bytes_only": (),
}


def _names(is_gpu: bool) -> list[str]:
    pre = "ix_" if is_gpu else "ixc_"
    return sorted({n for syms in IMPL_SYMBOLS.values() for n in syms if n.startswith(pre) and n.startswith("ixc_") != is_gpu})


def library_fingerprint(lib, is_gpu: bool) -> dict:
    """Version symbol and a digest over which of the known entry points the loaded library exports."""
    present = [(n, hasattr(lib, n)) for n in _names(is_gpu)]
    ver = getattr(lib, "ix_version" if is_gpu else "ixc_version")()
    h = hashlib.sha256(repr((int(ver), present)).encode()).hexdigest()[:24]
    return {"version": int(ver), "exports_digest": h, "missing": [n for n, ok in present if not ok]}


# implementations whose id is the same on both kinds of device (their kernels exist in both libraries)
_BOTH = {"cpr_chunk_scan": "gdn_scan", "cpr_recurrent_step": "gdn_scan", "shifted_sum_conv": "gdn_conv",
         "fp32_gating": "gdn_gate", "slot_pool": "gdn_conv_state"}


def installed_impl(lib, impl_id: str, is_gpu: bool) -> str:
    """The id under which ``impl_id`` is recorded as installed: itself when the library of the device the model lives
    on exports every entry point it needs; otherwise a marker that can never equal a contract entry."""
    if impl_id in _BOTH:
        sym = ("ix_" if is_gpu else "ixc_") + _BOTH[impl_id]
        return impl_id if hasattr(lib, sym) else f"missing:{impl_id}:{sym}"
    syms = IMPL_SYMBOLS.get(impl_id)
    if syms is None:
        return f"unknown:{impl_id}"
    if impl_id.startswith("cpu_") == is_gpu:
        return f"wrong-device:{impl_id}"
    missing = [n for n in syms if not hasattr(lib, n)]
    return impl_id if not missing else f"missing:{impl_id}:{','.join(missing)}"
