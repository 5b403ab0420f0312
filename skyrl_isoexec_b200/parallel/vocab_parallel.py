"""Token log-probabilities with the vocabulary sharded over tensor-parallel ranks.

Each rank holds V/tp columns of the LM head = G/tp whole leaves of the fixed-leaf log-softmax
(csrc/logprob.cu). The exchange moves only exact, order-free quantities (reference:
ISO/ops/logprobs/rowinv.py:481-508): the row maximum (max is exact in any order), the per-leaf
exp-sums (gathered, then folded locally by the fixed pairwise tree) and the target logit (owned
by one rank, the others contribute +0.0). Every rank ends with the same bits as a TP=1 run.
The backward is rank-local except for the sum of d(hidden) over vocabulary shards.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..core import observe as _obs
from ..ops import _cpu, _native
from ..ops import functional as F


def _staged_forward(logits, targets, G, tp, tp_rank, group, want_entropy):
    rows, vloc = logits.shape
    dev = logits.device
    lpl = G // tp                                    # leaves per rank
    is_f32 = int(logits.dtype == torch.float32)
    rmax = torch.empty(rows, dtype=torch.float32, device=dev)
    leaf = torch.zeros(rows, G, dtype=torch.float32, device=dev)
    leafpx = torch.zeros(rows, G, dtype=torch.float32, device=dev) if want_entropy else None
    tl = torch.empty(rows, dtype=torch.float32, device=dev)
    targets = targets.to(torch.int64).contiguous()
    _obs.note("logprobs.log_softmax", "rowinv_leaftree" if logits.is_cuda else "cpu_rowinv_leaftree")
    if logits.is_cuda:
        L, s, ck = _native.lib(), _native.stream(), _native.check
        ck(L.ix_logprob_rowmax(logits.data_ptr(), logits.stride(0), rows, vloc, rmax.data_ptr(), is_f32, s), "rowmax")
        dist.all_reduce(rmax, op=dist.ReduceOp.MAX, group=group)
        ck(L.ix_logprob_leafsum(logits.data_ptr(), logits.stride(0), rows, vloc, lpl, G, tp_rank * lpl, rmax.data_ptr(),
                                leaf.data_ptr(), _native.ptr(leafpx), is_f32, s), "leafsum")
        ck(L.ix_logprob_gather_target(logits.data_ptr(), logits.stride(0), rows, vloc, tp_rank * vloc, targets.data_ptr(),
                                      tl.data_ptr(), is_f32, s), "gather_target")
    else:
        L, dt = _cpu.lib(), _cpu.dt(logits)
        L.ixc_logprob_rowmax(logits.data_ptr(), logits.stride(0), rows, vloc, rmax.data_ptr(), dt)
        dist.all_reduce(rmax, op=dist.ReduceOp.MAX, group=group)
        L.ixc_logprob_leafsum(logits.data_ptr(), logits.stride(0), rows, vloc, lpl, G, tp_rank * lpl, rmax.data_ptr(),
                              leaf.data_ptr(), _cpu.ptr(leafpx), dt)
        t = targets - tp_rank * vloc
        ok = (t >= 0) & (t < vloc)
        tl = torch.where(ok, logits.float().gather(1, t.clamp(0, vloc - 1)[:, None])[:, 0], torch.zeros_like(tl))
    # leaf sums: every rank filled its own columns, the others are zero -> a sum is a gather
    dist.all_reduce(leaf, group=group)
    dist.all_reduce(tl, group=group)
    if want_entropy:
        dist.all_reduce(leafpx, group=group)
    lp = torch.empty(rows, dtype=torch.float32, device=dev)
    lse = torch.empty_like(lp)
    ent = torch.empty_like(lp) if want_entropy else None
    if logits.is_cuda:
        _native.check(_native.lib().ix_logprob_finalize(leaf.data_ptr(), _native.ptr(leafpx), rmax.data_ptr(), tl.data_ptr(),
                                                        targets.data_ptr(), lp.data_ptr(), lse.data_ptr(), _native.ptr(ent), rows, G,
                                                        _native.stream()), "finalize")
    else:
        _cpu.lib().ixc_logprob_finalize(leaf.data_ptr(), _cpu.ptr(leafpx), rmax.data_ptr(), tl.data_ptr(), targets.data_ptr(),
                                        lp.data_ptr(), lse.data_ptr(), _cpu.ptr(ent), rows, G)
    return lp, lse, ent


class _VocabParallelLogprob(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, G, ps, chunk, want_entropy):
        n = hidden.shape[0]
        lp = torch.empty(n, device=hidden.device, dtype=torch.float32)
        lse = torch.empty_like(lp)
        ent = torch.empty_like(lp) if want_entropy else torch.zeros_like(lp)
        for lo in range(0, n, chunk):
            hi = min(n, lo + chunk)
            logits = F.gemm_nt(hidden[lo:hi], weight)
            a, b, c = _staged_forward(logits, targets[lo:hi], G, ps.tp, ps.tp_rank, ps.tp_group, want_entropy)
            lp[lo:hi], lse[lo:hi] = a, b
            if want_entropy:
                ent[lo:hi] = c
        ctx.save_for_backward(hidden, weight, targets, lse, ent)
        ctx.cfg = (ps, chunk, want_entropy)
        if not want_entropy:
            ctx.mark_non_differentiable(ent)
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        hidden, weight, targets, lse, ent = ctx.saved_tensors
        ps, chunk, want_entropy = ctx.cfg
        n, vloc = hidden.shape[0], weight.shape[0]
        g_lp = g_lp.contiguous().float()
        ge = g_ent.contiguous().float() if want_entropy and g_ent is not None else None
        dh = torch.empty_like(hidden)
        own = hidden.is_cuda and hidden.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0
        dwf = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device) if own else None
        dw = None if own else torch.zeros_like(weight)
        for lo in range(0, n, chunk):
            hi = min(n, lo + chunk)
            logits = F.gemm_nt(hidden[lo:hi], weight)
            d = F.logprob_bwd(logits, targets[lo:hi].to(torch.int64).contiguous(), lse[lo:hi], g_lp[lo:hi],
                              None if ge is None else ge[lo:hi], ent[lo:hi] if ge is not None else None,
                              col_base=ps.tp_rank * vloc, inplace=True)
            dh[lo:hi] = F.gemm_nn(d, weight)
            if dwf is not None:
                F.gemm_tn(d, hidden[lo:hi], out=dwf, accumulate=True)
            else:
                dw.addmm_(d.t(), hidden[lo:hi])
        dist.all_reduce(dh, group=ps.tp_group)       # sum of the vocabulary shards' contributions
        return dh, (dwf.to(weight.dtype) if dwf is not None else dw), None, None, None, None, None


def vocab_parallel_logprobs(model, hidden_rows, targets, chunk: int, want_entropy: bool = False):
    w = model.lm_head_weight()
    G = model.cfg.logprob_leaves
    if G % model.ps.tp:
        raise ValueError(f"TP degree {model.ps.tp} does not divide the {G} vocabulary leaves")
    if torch.is_grad_enabled() and (hidden_rows.requires_grad or w.requires_grad):
        return _VocabParallelLogprob.apply(hidden_rows, w, targets, G, model.ps, chunk, want_entropy)
    n = hidden_rows.shape[0]
    lp = torch.empty(n, device=hidden_rows.device, dtype=torch.float32)
    ent = torch.zeros_like(lp)
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        a, _, c = _staged_forward(F.gemm_nt(hidden_rows[lo:hi], w), targets[lo:hi], G, model.ps.tp, model.ps.tp_rank,
                                  model.ps.tp_group, want_entropy)
        lp[lo:hi] = a
        if want_entropy:
            ent[lo:hi] = c
    return lp, ent
