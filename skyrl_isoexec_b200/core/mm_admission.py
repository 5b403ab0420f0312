"""Per-shape admission of the GEMM provider on the shapes a model really runs (the reference proves, at install time and
for every (K, N) of its census, that two M buckets of its pinned cuBLASLt algorithm agree before it lets the provider
serve that shape: ISO/ops/mm/mm_cublaslt.py, ISO/ops/mm/csrc/cublaslt_pinned.cpp:58-118).

Here the provider is the framework's own tcgen05 GEMM, whose K order is fixed by construction; the admission is the
self-check that the construction holds on THIS build and THIS device for every shape of the model's census:

* a row of the output is the same bits whether it is computed alone, inside a decode-sized batch or inside a
  training-sized one (three different tile choices of the kernel), and
* for row-parallel sites under the TP-invariant leaf tree, the form that gives every leaf its own CTA (decode) and the
  form that keeps all leaves in one CTA (training) agree as well.

``admit(cfg, device)`` returns {site: True | False | None}; None means the site cannot be checked here (no GPU, or a
shape the kernel does not serve). ``refused(report)`` lists the sites that failed; the trainer refuses to start on one.
"""

from __future__ import annotations

import torch

_REPORTS: dict = {}


def _rows_agree(fn, x: torch.Tensor, buckets=(1, 64, 320)) -> bool:
    """fn(x[:m]) row 0 and row m-1 equal the rows of the largest bucket."""
    big = fn(x[:buckets[-1]].contiguous())
    for m in buckets[:-1]:
        got = fn(x[:m].contiguous())
        if not torch.equal(got.view(torch.int16 if got.dtype == torch.bfloat16 else torch.int32),
                           big[:m].contiguous().view(torch.int16 if big.dtype == torch.bfloat16 else torch.int32)):
            return False
    return True


def admit(cfg, device: str = "cuda", tp: int = 1, ep: int = 1) -> dict:
    """Run the self-check for every GEMM site of ``cfg`` at tensor-parallel degree ``tp``. Cached per (model shape, tp)."""
    from ..models.census import gemm_census
    from ..ops import functional as F

    key = (cfg.name, cfg.hidden_size, cfg.num_layers, tp, ep, getattr(cfg, "pik_leaves", 0), bool(getattr(cfg, "tp_invariant", False)), str(device))
    if key in _REPORTS:
        return _REPORTS[key]
    report: dict = {}
    on_gpu = str(device).startswith("cuda") and torch.cuda.is_available()
    g = torch.Generator(device=device if on_gpu else "cpu").manual_seed(17)
    seen: dict = {}
    for site in gemm_census(cfg, tp, ep):
        shape = (site.k, site.n, "row" if site.sharding == "row" else "plain", site.out_dtype)
        if shape in seen:                     # several sites share a shape: one check
            report[site.name] = seen[shape]
            continue
        if not on_gpu or cfg.dtype != "bfloat16" or site.grouped or site.k % 8 or site.n % 8:
            report[site.name] = seen[shape] = None      # expert matrices are covered by the grouped-GEMM region check
            continue
        # drawn in bf16 and scaled in place: the LM head's probe weight is 1.2 GB, an fp32 detour would hold 6 GB for a moment
        x = torch.randn(320, site.k, generator=g, device=device, dtype=torch.bfloat16).mul_(0.5)
        w = torch.randn(site.n, site.k, generator=g, device=device, dtype=torch.bfloat16).mul_(0.05)
        f32 = site.out_dtype == "fp32"
        ok = _rows_agree(lambda a: F.gemm_nt(a, w, out_f32=f32), x)
        leaves = getattr(cfg, "pik_leaves", 0) // max(1, tp) if getattr(cfg, "tp_invariant", False) else 0
        if ok and site.sharding == "row" and leaves >= 2:
            from ..parallel import tp_fused

            if tp_fused.fused_ok(320, site.n, site.k, leaves):
                ok = _rows_agree(lambda a: tp_fused.leaftree_gemm_fused(a, w, leaves, out_f32=True), x)
                one = tp_fused.leaftree_gemm_fused(x[:64].contiguous(), w, leaves, out_f32=True, split=False)
                ok = ok and torch.equal(one, tp_fused.leaftree_gemm_fused(x[:64].contiguous(), w, leaves, out_f32=True))
        report[site.name] = seen[shape] = bool(ok)
        del x, w
    _REPORTS[key] = report
    return report


def refused(report: dict) -> list[str]:
    return sorted(k for k, v in report.items() if v is False)
