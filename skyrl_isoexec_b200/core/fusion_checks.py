"""Bit-equality checkers of the hand-fused kernels listed in ``fusion_ledger.REGIONS`` (the reference proves each
``torch.compile`` region equal to its eager chain before admitting it, ISO/autofuse/region_gate.py, pair.py).

Every region has a checker. A checker runs the fused kernel and the chain it replaces (or the two members of a pair)
on hazard inputs and returns True / False, or None when the comparison cannot be made on the given device (a kernel
that exists on the GPU only, or one that needs several GPUs); None is reported as "deferred", never as proven.
Importing this module registers the checkers.
"""

from __future__ import annotations

import math

import torch

from .fusion_ledger import checker, hazard_population


def _bits(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.int16 if t.dtype == torch.bfloat16 else torch.int32)


def _same(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.shape == b.shape and a.dtype == b.dtype and bool(torch.equal(_bits(a), _bits(b)))


def _dt(device: str):
    return torch.bfloat16 if device != "cpu" else torch.float32


@checker("qk_norm+rope+kv_write")
def _chk_rope(device: str):
    """The engine form (K/V scattered into slot pools) against the trainer form (fresh packed K/V): same bits."""
    from ..ops import functional as F

    dt = _dt(device)
    Hq, Hkv, D, T = 4, 2, 64, 37
    qkv = hazard_population((T, (Hq + 2 * Hkv) * D), dt, device, 5).clamp(-100, 100)
    qw, kw = hazard_population((D,), dt, device, 6).clamp(-4, 4), hazard_population((D,), dt, device, 7).clamp(-4, 4)
    pos = torch.arange(T, dtype=torch.int32, device=device) * 3 % 50
    rope = F.RopeTable(D, 64, 1e6, torch.device(device))
    slots = torch.randperm(2 * T)[:T].to(device)
    kp, vp = torch.zeros(2 * T, Hkv, D, dtype=dt, device=device), torch.zeros(2 * T, Hkv, D, dtype=dt, device=device)
    q1 = F.qk_norm_rope_fwd(qkv, pos, slots, rope, qw, kw, kp, vp, Hq, Hkv, D, 1e-6)
    k2, v2 = torch.zeros(T, Hkv, D, dtype=dt, device=device), torch.zeros(T, Hkv, D, dtype=dt, device=device)
    q2 = F.qk_norm_rope_fwd(qkv, pos, None, rope, qw, kw, k2, v2, Hq, Hkv, D, 1e-6)
    return _same(q1, q2) and _same(kp[slots], k2) and _same(vp[slots], v2)


@checker("gemm+swiglu (EPI_GLU)")
def _chk_glu(device: str):
    if device == "cpu":
        return None
    from ..ops import functional as F
    from ..ops import moe

    x = hazard_population((70, 256), torch.bfloat16, device, 8).clamp(-8, 8)
    w = (hazard_population((2 * 128, 256), torch.bfloat16, device, 9).clamp(-1, 1) * 0.1).bfloat16()
    fused = moe.grouped_gemm(x, w.unsqueeze(0), None, moe.EPI_GLU)
    return _same(fused, F.swiglu_fwd(F.gemm_nt(x, w)))


@checker("grouped_gemm(experts)")
def _chk_grouped(device: str):
    if device == "cpu":
        return None
    from ..ops import moe

    g = torch.Generator().manual_seed(3)
    T, E, k, H, Fd = 150, 8, 2, 256, 128
    y = hazard_population((T, H), torch.bfloat16, device, 10).clamp(-8, 8)
    gu = (torch.randn(E, 2 * Fd, H, generator=g) * 0.05).bfloat16().to(device)
    dn = (torch.randn(E, H, Fd, generator=g) * 0.05).bfloat16().to(device)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).int().to(device)
    w = torch.rand(T, k, generator=g).to(device)
    plan = moe.DispatchPlan(idx, E, 1)
    xr, wr = plan.gather(y, w.reshape(-1).contiguous())
    counts = (plan.offs[1:] - plan.offs[:-1]).tolist()
    return _same(moe.expert_rows_grouped(xr, wr, plan.offs, gu, dn), moe._expert_rows(xr, wr, counts, gu, dn))


@checker("leaftree_gemm (LOCAL)")
def _chk_leaftree(device: str):
    """One kernel holding G leaf accumulators against G separate fp32 GEMMs folded by the balanced tree."""
    from ..ops import functional as F
    from ..parallel import tp

    dt = _dt(device)
    x = hazard_population((45, 512), dt, device, 11).clamp(-8, 8)
    w = hazard_population((96, 512), dt, device, 12).clamp(-1, 1)
    G, LK = 8, 512 // 8
    parts = torch.stack([F.gemm_nt(x[:, j * LK:(j + 1) * LK].contiguous(), w[:, j * LK:(j + 1) * LK].contiguous(), out_f32=True)
                         for j in range(G)])
    want = tp.tree_fold(parts)
    if device == "cpu":
        got = tp.leaftree_gemm(x, w, G)
    else:
        from ..parallel import tp_fused

        got = tp_fused.leaftree_gemm_fused(x, w, G, out_f32=True)
    return _same(got, want)


@checker("leaftree_gemm (one CTA per leaf | two 4-leaf launches | one CTA)")
def _chk_leaf_forms(device: str):
    """The three schedules of the single-rank leaf-tree GEMM give one set of bits: a cluster with one CTA per leaf
    (decode sizes), two launches of four leaves joined by the addend epilogue (8 leaves at training sizes), and all
    leaves in one CTA's TMEM."""
    if device == "cpu":
        return None             # one schedule on the CPU
    from ..parallel import tp_fused

    w = hazard_population((256, 1024), torch.bfloat16, device, 21).clamp(-1, 1)
    ok = True
    for M in (40, 300):
        x = hazard_population((M, 1024), torch.bfloat16, device, 22 + M).clamp(-8, 8)
        for L in (2, 8):
            one = tp_fused.leaftree_gemm_fused(x, w, L, out_f32=True, bn=32, split=False)       # every leaf in one CTA
            ok = ok and _same(tp_fused.leaftree_gemm_fused(x, w, L, out_f32=True), one)           # the form the size selects
            if M <= 256:
                ok = ok and _same(tp_fused.leaftree_gemm_fused(x, w, L, out_f32=True, split=True), one)
    return ok


def _admitted(kind: str):
    """The fused GEMM+collective kernels are compared with their unfused chain by the admission probe that runs on the
    first call of every shape (parallel/tp.py::admit_fused_row_parallel). Without a multi-GPU job there is nothing to
    read: deferred."""
    from ..parallel import tp

    shapes = tp.admitted_shapes()
    if not shapes:
        return None
    return all(shapes.values())


@checker("tp_gemm_fused (AR1/AR2/RS)")
def _chk_tp_ar(device: str):
    return _admitted("ar")


@checker("tp_gemm_fused (AG)")
def _chk_tp_ag(device: str):
    return _admitted("ag")


@checker("attention (prefill | decode | chunk)")
def _chk_attention(device: str):
    """One query token against a paged cache, and a chunk of queries, equal the rows of the full prefill."""
    from ..ops import functional as F

    dt = _dt(device)
    Hq, Hkv, D, S = 4, 2, 64, 300
    q = hazard_population((S, Hq, D), dt, device, 13).clamp(-6, 6)
    k = hazard_population((S, Hkv, D), dt, device, 14).clamp(-6, 6)
    v = hazard_population((S, Hkv, D), dt, device, 15).clamp(-6, 6)
    scale = 1 / math.sqrt(D)
    full, _ = F.attention_fwd(q, k, v, F.AttnMeta.packed([S], Hq, Hkv, device), scale)
    pages = [4, 0, 2]
    kc, vc = torch.zeros(5 * 128, Hkv, D, dtype=dt, device=device), torch.zeros(5 * 128, Hkv, D, dtype=dt, device=device)
    for b, p in enumerate(pages):
        lo, hi = b * 128, min(S, b * 128 + 128)
        kc[p * 128:p * 128 + hi - lo], vc[p * 128:p * 128 + hi - lo] = k[lo:hi], v[lo:hi]
    bt = torch.tensor([pages], dtype=torch.int32, device=device)
    ok = True
    for t in (0, 127, 128, 299):
        items = torch.tensor([[0, 1, t, t + 1, 0, 0, 0, 0]], dtype=torch.int32, device=device)
        o, _ = F.attention_fwd(q[t:t + 1].contiguous(), kc, vc, F.AttnMeta(items, bt), scale)
        ok = ok and _same(o[0], full[t])
    tq = 128 // (Hq // Hkv)
    lo = 130
    n = min(tq, S - lo)
    items = torch.tensor([[0, n, lo, lo + n, 0, 0, 0, 0]], dtype=torch.int32, device=device)
    o, _ = F.attention_fwd(q[lo:lo + n].contiguous(), kc, vc, F.AttnMeta(items, bt), scale)
    return ok and _same(o, full[lo:lo + n])


@checker("rmsnorm (cta-per-row | warp-per-row)")
def _chk_rms_geometry(device: str):
    if device == "cpu":
        return None             # one geometry on the CPU
    from ..ops import functional as F

    x = hazard_population((1500, 1024), torch.bfloat16, device, 16)
    r = hazard_population((1500, 1024), torch.bfloat16, device, 17)
    w = hazard_population((1024,), torch.bfloat16, device, 18)
    big = F.rmsnorm_fwd(x, w, 1e-6, False, r)
    small = F.rmsnorm_fwd(x[:64].contiguous(), w, 1e-6, False, r[:64].contiguous())
    return _same(small[0], big[0][:64]) and _same(small[1], big[1][:64])


@checker("gdn_scan (chunked | recurrent)")
def _chk_gdn(device: str):
    """A sequence scanned whole equals the same sequence fed as a prefill chunk, single decode steps and further chunks
    through the state pool."""
    from ..models.config import get_config
    from ..ops import gdn

    cfg = get_config("tiny-hybrid", dtype="bfloat16" if device != "cpu" else "float32")
    dt = cfg.torch_dtype
    hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
    C = (2 * hk + hv) * d
    T = 140
    g = torch.Generator().manual_seed(12)
    proj = (torch.randn(T, C + hv * d + 2 * hv, generator=g) * 0.5).to(dt).to(device)
    conv_w = (torch.randn(C, cfg.gdn_conv_kernel, generator=g) * 0.3).to(dt).to(device)
    A_log, dtb = (torch.randn(hv, generator=g) * 0.1).to(dt).to(device), (torch.randn(hv, generator=g) * 0.1).to(dt).to(device)
    whole = gdn.gdn_core_fwd(proj, conv_w, A_log, dtb, gdn.GDNMeta.packed([T], device), cfg, 1)
    conv_state = torch.zeros(3, C, cfg.gdn_conv_kernel - 1, dtype=dt, device=device)
    ssm = torch.zeros(3, hv, d, d, dtype=torch.float32, device=device)
    open_chunk = gdn.new_chunk_buffers(3, hk, hv, d, dt, device) if gdn.chunked_ok(proj, d) else None
    outs, pos = [], 0
    for n in (70, 1, 1, 64, 1, 3):
        meta = gdn.GDNMeta.build([(0, n, pos, 2 if pos > 0 else -1, 2)], device)
        outs.append(gdn.gdn_core_fwd(proj[pos:pos + n].contiguous(), conv_w, A_log, dtb, meta, cfg, 1, conv_state, ssm, open_chunk))
        pos += n
    return _same(torch.cat(outs, 0), whole)


@checker("ppo_loss_fused")
def _chk_ppo(device: str):
    """The fused loss kernel against the torch chain: same loss and gradient up to fp32 summation order (1e-4), and
    bit-identical from run to run. The loss is outside the logprob path, so closeness, not bit equality, is the claim."""
    if device == "cpu":
        return None
    from ..train import algorithms as alg

    g = torch.Generator().manual_seed(10)
    cfg = alg.AlgorithmConfig()
    lp = torch.randn(6, 40, generator=g) * 0.3 - 2
    old = lp + torch.randn(6, 40, generator=g) * 0.2
    adv, mask = torch.randn(6, 40, generator=g), (torch.rand(6, 40, generator=g) > 0.2).float()
    fn = alg.get_policy_loss("regular")
    a = lp.clone().requires_grad_()
    l0, _ = fn(a, old, adv, cfg, loss_mask=mask)
    (g0,) = torch.autograd.grad(l0, a)
    res = []
    for _ in range(2):
        b = lp.to(device).requires_grad_()
        l1, _ = fn(b, old.to(device), adv.to(device), cfg, loss_mask=mask.to(device))
        (g1,) = torch.autograd.grad(l1, b)
        res.append((l1.detach().cpu(), g1.cpu()))
    close = abs(float(l0) - float(res[0][0])) < 1e-3 * max(1.0, abs(float(l0))) and float((g0 - res[0][1]).abs().max()) < 1e-4
    return close and _same(res[0][1], res[1][1]) and _same(res[0][0].reshape(1), res[1][0].reshape(1))
