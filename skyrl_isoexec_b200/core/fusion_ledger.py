"""Ledger of hand-fused kernels and their bit-equality evidence (the role of the reference's autofuse package:
ISO/autofuse/region_gate.py admission, fusion_ledger.py:44-182 digest folded into the handshake, pair.py PAIR_EQUALITY).

The reference admits ``torch.compile`` regions only after proving the fused code bitwise equal to the eager chain on
hazard populations. Here no compiler fuses anything: each fusion is a kernel written by hand, but the obligation is
the same. Every fused kernel is listed with (a) the unfused chain it must reproduce, (b) a checker that runs both on
hazard inputs (denormals, large magnitudes, exact ties, negative zeros, ragged shapes) and compares bits. The digest of
the ledger (names + chains) is part of the process contract's extensions, so a trainer and an engine built with
different fusion sets refuse to sync.
"""

from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from typing import Callable


@dataclass(frozen=True)
class FusedRegion:
    name: str                    # kernel / entry point
    replaces: tuple              # the unfused op chain it must equal bit for bit
    equality: str                # "bitwise" | "pair" (two fused sites must equal each other, not an eager chain) | "close"
    note: str = ""


REGIONS: tuple[FusedRegion, ...] = (
    FusedRegion("rmsnorm+residual", ("add(bf16)", "rmsnorm"), "bitwise", "h = bf16(x + r) is formed in the kernel and returned"),
    FusedRegion("qk_norm+rope+kv_write", ("rmsnorm(head)", "rope", "scatter(kv)"), "bitwise"),
    FusedRegion("gemm+swiglu (EPI_GLU)", ("gemm_nt -> bf16", "swiglu", "scale_rows"), "bitwise",
                "the epilogue repeats the three roundings of the separate kernels"),
    FusedRegion("grouped_gemm(experts)", ("loop over experts: gemm_nt",), "bitwise"),
    FusedRegion("leaftree_gemm (LOCAL)", ("per-leaf gemm_nt fp32", "tree_fold"), "bitwise"),
    FusedRegion("leaftree_gemm (one CTA per leaf | two 4-leaf launches | one CTA)", ("leaftree_gemm (LOCAL)",), "pair",
                "the decode-sized cluster form and the split 8-leaf training form equal the single-CTA form"),
    FusedRegion("tp_gemm_fused (AR1/AR2/RS)", ("leaftree_gemm", "tree_all_reduce"), "bitwise"),
    FusedRegion("tp_gemm_fused (AG)", ("all_gather", "gemm_nt"), "bitwise"),
    FusedRegion("logprob_fused", ("rowmax", "leafsum", "finalize", "gather_target"), "bitwise"),
    FusedRegion("attention (prefill | decode | chunk)", ("attention(prefill)",), "pair", "decode and chunked prefill equal full prefill"),
    FusedRegion("rmsnorm (cta-per-row | warp-per-row)", ("rmsnorm",), "pair", "two launch geometries, one reduction order"),
    FusedRegion("gdn_scan (chunked | recurrent)", ("gdn_scan(sequential)",), "pair"),
    FusedRegion("ppo_loss_fused", ("ratio", "clip", "min", "mask", "sum"), "close",
                "outside the logprob path: equal to the torch chain up to fp32 summation order, bit-identical run to run"),
)


def ledger_digest(regions=REGIONS) -> str:
    doc = [{"name": r.name, "replaces": list(r.replaces), "equality": r.equality} for r in regions]
    return hashlib.sha256(json.dumps(doc, sort_keys=True, separators=(",", ":")).encode()).hexdigest()[:24]


def hazard_population(shape, dtype, device, seed: int = 0):
    """Inputs on which a wrong fusion shows: normal draws plus denormals, +-0, huge and tiny magnitudes, exact ties."""
    import torch

    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(shape, generator=g)
    flat = x.view(-1)
    n = flat.numel()
    specials = torch.tensor([0.0, -0.0, 1e-40, -1e-40, 65504.0, -65504.0, 3.0e38, 1e-30, 1.0, 1.0, -1.0, 0.5, 2.0 ** -126])
    idx = torch.randperm(n, generator=g)[: min(n, 4 * specials.numel())]
    flat[idx] = specials.repeat(4)[: idx.numel()]
    return x.to(dtype).to(device)


_CHECKERS: dict[str, Callable[[str], bool]] = {}


def checker(name: str):
    def deco(fn):
        _CHECKERS[name] = fn
        return fn
    return deco


def run_checkers(device: str) -> dict[str, bool | None]:
    """Run every region's checker on ``device``: True / False, or None when the comparison needs another device
    (deferred, not proven). A region WITHOUT a checker raises: an unproven fusion must not pass silently."""
    from . import fusion_checks  # noqa: F401  (registers the checkers)

    missing = [r.name for r in REGIONS if r.name not in _CHECKERS]
    if missing:
        raise LookupError(f"fused regions without a bit-equality checker: {missing}")
    return {r.name: _CHECKERS[r.name](device) for r in REGIONS}


@checker("rmsnorm+residual")
def _chk_rmsnorm(device: str) -> bool:
    import torch

    from ..ops import functional as F

    dt = torch.bfloat16 if device != "cpu" else torch.float32
    x, r = hazard_population((33, 512), dt, device, 1), hazard_population((33, 512), dt, device, 2)
    w = hazard_population((512,), dt, device, 3)
    y1, h1, _ = F.rmsnorm_fwd(x, w, 1e-6, False, r)
    h = (x.float() + r.float()).to(dt)
    y2, _, _ = F.rmsnorm_fwd(h, w, 1e-6, False, None)
    return bool(torch.equal(h1, h) and torch.equal(y1.view(torch.int16 if dt == torch.bfloat16 else torch.int32),
                                                    y2.view(torch.int16 if dt == torch.bfloat16 else torch.int32)))


@checker("logprob_fused")
def _chk_logprob(device: str) -> bool:
    import torch

    from ..ops import functional as F

    dt = torch.bfloat16 if device != "cpu" else torch.float32
    lg = hazard_population((9, 4096), dt, device, 4).clamp(-60000, 60000)
    tg = torch.arange(9, device=device) * 37
    a = F.logprob_fused_fwd(lg, tg, 8)[0]
    b = F.token_logprobs(lg, tg, 8)[0]
    return bool(torch.equal(a.view(torch.int32), b.view(torch.int32)))
