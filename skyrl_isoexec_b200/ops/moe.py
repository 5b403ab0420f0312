"""Mixture-of-experts block with batch-, EP- and order-invariant numerics.

Recipe (the reference's deterministic MoE, ISO/ops/moe/moe_batch_invariant.py:276-321,744-887 and
moe_batched_experts.py:152-298, restated without Megatron):
  router   fp32 logits from the batch-invariant GEMM; per-token top-k with lower-index ties;
           gate weights optionally renormalised over the k picks (csrc/moe.cu)
  dispatch (token, slot) rows ordered by (expert, token, slot): a stable counting sort, integers only
  experts  per expert row group: fc1 -> SwiGLU -> x gate weight (one round) -> fc2 with fp32 output,
           each through the batch-invariant GEMM, so a row's value does not depend on its group size
  combine  per token: fp32 sum of its k expert rows in ASCENDING EXPERT INDEX, one round, then the
           shared expert (if any) is added
With expert parallelism the rows travel to the expert's owner and back by all-to-all (bytes only);
the sum order is a property of the token, not of where its experts live, so EP never changes bits.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from collections import Counter

from ..core import observe as _obs
from . import _cpu, _native
from . import functional as F

_SERVED: Counter = Counter()       # which expert path served how many MoE blocks (read by the contract ledger)


# ------------------------------------------------------------------------------------ router
def router_topk_fwd(logits: torch.Tensor, k: int, bias: torch.Tensor | None, sigmoid_bias: bool, norm_topk: bool,
                    want_probs: bool = False):
    """logits fp32 [T, E] -> (idx int32 [T, k], weights fp32 [T, k], probs [T, E] | None)."""
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    probs = torch.empty(T, E, dtype=torch.float32, device=logits.device) if want_probs else None
    if T == 0:
        return idx, w, probs
    _obs.note("moe.router", "deterministic_topk" if logits.is_cuda else "cpu_deterministic_topk")
    if logits.is_cuda:
        _native.check(_native.lib().ix_router_topk(logits.data_ptr(), logits.stride(0), _native.ptr(bias), T, E, k,
                                                   int(sigmoid_bias), int(norm_topk), idx.data_ptr(), w.data_ptr(),
                                                   _native.ptr(probs), _native.stream()), "ix_router_topk")
    else:
        _cpu.lib().ixc_router_topk(logits.data_ptr(), logits.stride(0), _cpu.ptr(bias), T, E, k, int(sigmoid_bias),
                                   int(norm_topk), idx.data_ptr(), w.data_ptr(), _cpu.ptr(probs))
    return idx, w, probs


class _RouterTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, bias, sigmoid_bias, norm_topk):
        idx, w, _ = router_topk_fwd(logits, k, bias, sigmoid_bias, norm_topk)
        ctx.save_for_backward(logits, idx)
        ctx.cfg = (sigmoid_bias, norm_topk)
        ctx.mark_non_differentiable(idx)
        return idx, w

    @staticmethod
    def backward(ctx, _g_idx, g_w):
        logits, idx = ctx.saved_tensors
        sigmoid_bias, norm_topk = ctx.cfg
        with torch.enable_grad():
            x = logits.detach().requires_grad_(True)
            p = torch.sigmoid(x) if sigmoid_bias else torch.softmax(x, -1)
            w = p.gather(1, idx.long())
            if norm_topk:
                w = w / w.sum(-1, keepdim=True)
            (gx,) = torch.autograd.grad(w, x, g_w)
        return gx, None, None, None, None


def route(logits, k, bias=None, sigmoid_bias=False, norm_topk=True):
    if torch.is_grad_enabled() and logits.requires_grad:
        return _RouterTopK.apply(logits, k, bias, sigmoid_bias, norm_topk)
    idx, w, _ = router_topk_fwd(logits, k, bias, sigmoid_bias, norm_topk)
    return idx, w


# ------------------------------------------------------------------------------------ auxiliary load-balancing loss
# Switch-style balance term of a MoE layer, aux = E * sum_e f_e * P_e (f_e: share of the routed (token, slot) pairs that
# went to expert e; P_e: mean router probability of e), as in the reference's Megatron path (``moe_aux_loss_coeff``). It is
# not added to the policy loss: its gradient is INJECTED where the routing weights enter the block (``_AuxGrad``), which is
# what survives activation recomputation (the recomputed layer rebuilds the injection). The trainer sets ``coeff`` and,
# per micro-batch, ``scale`` (the micro-batch's share of the global loss normalisation); ``sum`` / ``layers`` feed a metric.
AUX_LOSS = {"coeff": 0.0, "scale": 1.0, "sum": 0.0, "layers": 0}


class _AuxGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, aux, scale):
        ctx.scale = scale
        ctx.aux_shape = aux.shape
        return w.view_as(w)

    @staticmethod
    def backward(ctx, g):
        return g, torch.full(ctx.aux_shape, ctx.scale, dtype=g.dtype, device=g.device), None


def _with_aux_loss(logits: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, cfg) -> torch.Tensor:
    if AUX_LOSS["coeff"] <= 0 or not (torch.is_grad_enabled() and logits.requires_grad and w.requires_grad) or logits.shape[0] == 0:
        return w
    T, E = logits.shape
    if cfg.router == "sigmoid_bias":
        s = torch.sigmoid(logits)
        probs = s / s.sum(-1, keepdim=True).clamp_min(1e-20)
    else:
        probs = torch.softmax(logits, -1)
    with torch.no_grad():
        f = torch.zeros(E, dtype=torch.float32, device=logits.device)
        f.index_add_(0, idx.reshape(-1).long(), torch.ones(idx.numel(), dtype=torch.float32, device=logits.device))
        f /= float(idx.numel())
    aux = E * (f * probs.mean(0)).sum()
    AUX_LOSS["sum"] += float(aux.detach())
    AUX_LOSS["layers"] += 1
    return _AuxGrad.apply(w, aux, AUX_LOSS["coeff"] * AUX_LOSS["scale"])


# ------------------------------------------------------------------------------------ dispatch / combine
def build_dispatch(idx: torch.Tensor, num_experts: int):
    """Integer routing mechanics. idx int32 [T, k]. Returns
    order   int64 [T*k]  flat (token*k + slot) ids sorted by (expert, token, slot),
    counts  int64 [E]    rows per expert,
    pos     int64 [T, k] for each token, the dispatch row of its experts in ASCENDING expert index."""
    T, k = idx.shape
    if idx.is_cuda and idx.dtype == torch.int32 and k <= 16:
        # the counting-sort kernels (csrc/moe_dispatch.cu): same tables, no sort, no host round trip
        plan = DispatchPlan(idx, num_experts, 1)
        return plan.src_of_row[:T * k].long(), (plan.offs[1:] - plan.offs[:-1]).long(), plan.pos
    _obs.note("moe.dispatch", "cpu_index_build" if not idx.is_cuda else "torch_sort_index_build")
    flat = idx.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices            # stable: ties keep (token, slot) order
    counts = torch.bincount(flat, minlength=num_experts)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=idx.device)
    by_expert = torch.sort(idx.long(), dim=1, stable=True).indices   # slots of a token by ascending expert
    pos = inv.view(T, k).gather(1, by_expert)
    return order, counts, pos


def combine_fixed_order(rows: torch.Tensor, pos: torch.Tensor, out_dtype, shared: torch.Tensor | None = None):
    """out[t] = round(sum_j rows[pos[t, j]]) with j over ascending expert index (fp32), + shared after the round."""
    T, k = pos.shape
    H = rows.shape[1]
    _obs.note("moe.combine", "fixed_order" if rows.is_cuda else "cpu_fixed_order")
    if rows.is_cuda and out_dtype in (torch.bfloat16, torch.float32) and not (torch.is_grad_enabled() and rows.requires_grad):
        out = torch.empty(T, H, dtype=out_dtype, device=rows.device)
        if T:
            _native.check(_native.lib().ix_moe_combine(rows.data_ptr(), pos.data_ptr(), _native.ptr(shared), out.data_ptr(), T, H,
                                                       k, int(out_dtype == torch.bfloat16), _native.stream()), "ix_moe_combine")
        return out
    acc = rows.index_select(0, pos[:, 0])
    for j in range(1, k):
        acc = acc + rows.index_select(0, pos[:, j])
    out = acc.to(out_dtype)
    if shared is not None:
        out = (out.float() + shared.float()).to(out_dtype)
    return out


class _AllToAll(torch.autograd.Function):
    """Variable-split all-to-all of rows over the EP group (bytes only); backward is the reverse exchange. The forward
    payload keeps its dtype (the returned expert rows must reach the source unrounded: fp32). ``grad_wire``: dtype the
    GRADIENT rows travel in; bf16 halves the backward exchange of the fp32 rows and is outside the bitwise contract
    (reference: the bf16 all-to-all wire of the MoE backward, ISO/ops/moe/moe_combine_backward.py)."""

    @staticmethod
    def forward(ctx, x, send_counts, recv_counts, group, grad_wire=None):
        ctx.cfg = (send_counts, recv_counts, group, grad_wire)
        out = x.new_empty((sum(recv_counts),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        send_counts, recv_counts, group, grad_wire = ctx.cfg
        wire = g.to(grad_wire) if grad_wire is not None and g.dtype != grad_wire else g
        out = wire.new_empty((sum(send_counts),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, wire.contiguous(), output_split_sizes=send_counts, input_split_sizes=recv_counts, group=group)
        return out.to(g.dtype), None, None, None, None


# ------------------------------------------------------------------------------------ experts
def _expert_rows(x_rows, w_rows, counts, gate_up, down):
    """Rows grouped by local expert -> fp32 expert outputs, one GEMM pair per non-empty group."""
    _obs.note("moe.experts", "cpu_grouped_gemm" if not x_rows.is_cuda else "looped_experts")
    outs = []
    lo = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        xe = x_rows[lo:lo + n]
        h1 = F.linear(xe, gate_up[e])
        a = F.swiglu(h1)
        if a.is_cuda and a.dtype == torch.bfloat16 and not (torch.is_grad_enabled() and a.requires_grad):
            _native.check(_native.lib().ix_scale_rows(a.data_ptr(), w_rows[lo:lo + n].contiguous().data_ptr(), n, a.shape[1],
                                                      _native.stream()), "ix_scale_rows")
        else:
            a = (a.float() * w_rows[lo:lo + n, None]).to(a.dtype)
        outs.append(F.linear(a, down[e], out_f32=True))
        lo += n
    if not outs:
        return x_rows.new_zeros((0, down.shape[1]), dtype=torch.float32)
    return torch.cat(outs, 0)


EPI_BF16, EPI_F32, EPI_GLU = 0, 1, 2


def grouped_gemm(x_rows: torch.Tensor, w: torch.Tensor, offs: torch.Tensor, epi: int, w_rows: torch.Tensor | None = None,
                 row_dst: torch.Tensor | None = None, out: torch.Tensor | None = None, bn: int = 0) -> torch.Tensor:
    """One launch over all experts (csrc/moe_grouped_gemm.cu). x_rows [R, K] bf16 sorted by expert, offs int32 [E+1]
    on the device, w [E, N or 2N, K]. epi: EPI_BF16 | EPI_F32 plain output, EPI_GLU = SwiGLU x gate weight.
    ``row_dst`` (int64 [R] device addresses) scatters the output rows, possibly into peer memory."""
    R, K = x_rows.shape
    E = w.shape[0]
    N = w.shape[1] // 2 if epi == EPI_GLU else w.shape[1]
    assert x_rows.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and x_rows.stride(1) == 1
    assert offs is None or (offs.dtype == torch.int32 and offs.numel() == E + 1)
    if out is None and row_dst is None:
        out = torch.empty(R, N, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16, device=x_rows.device)
    _native.check(_native.lib().ix_moe_grouped_gemm(x_rows.data_ptr(), w.data_ptr(), _native.ptr(out), _native.ptr(offs),
                                                    _native.ptr(w_rows), _native.ptr(row_dst), R, E, N, K, x_rows.stride(0), N,
                                                    epi, bn, _native.stream()), "ix_moe_grouped_gemm")
    return out


def expert_rows_grouped(x_rows, w_rows, offs, gate_up, down, row_dst=None):
    """fc1 + SwiGLU + gate weight in one grouped launch, fc2 (fp32 out) in a second; no host round trip."""
    _obs.note("moe.experts", "grouped_gemm")
    _obs.note("activation.swiglu", "fused_swiglu")          # applied in the fc1 epilogue
    a = grouped_gemm(x_rows, gate_up, offs, EPI_GLU, w_rows=w_rows.contiguous())
    return grouped_gemm(a, down, offs, EPI_F32, row_dst=row_dst)


def _grouped_ok(x_rows, gate_up, down) -> bool:
    return (x_rows.is_cuda and x_rows.dtype == torch.bfloat16 and not torch.is_grad_enabled() and gate_up.shape[2] % 64 == 0
            and down.shape[2] % 64 == 0 and down.shape[1] % 32 == 0 and (gate_up.shape[1] // 2) % 32 == 0 and gate_up.shape[0] <= 512)


# ------------------------------------------------------------------------------------ device-side routing plan + expert VJP
class DispatchPlan:
    """Routing tables built on the device without a host round trip (csrc/moe_dispatch.cu): rows ordered by (expert,
    token, slot); every expert's group padded to a multiple of ``pad`` rows (zero rows)."""

    def __init__(self, idx: torch.Tensor, num_experts: int, pad: int):
        import ctypes as C

        T, k = idx.shape
        _obs.note("moe.dispatch", "index_build")
        self.T, self.k, self.E, self.pad = T, k, num_experts, pad
        dev = idx.device
        self.r_cap = ((T * k + num_experts * (pad - 1)) + 63) // 64 * 64 if pad > 1 else max(1, T * k)
        self.offs = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
        self.row_of = torch.empty(max(1, T * k), dtype=torch.int32, device=dev)
        self.src_of_row = torch.empty(self.r_cap, dtype=torch.int32, device=dev)
        self.pos = torch.empty(T, k, dtype=torch.int64, device=dev)
        scratch = torch.empty(T * k + num_experts, dtype=torch.int32, device=dev)
        lib = _native.lib()
        if not getattr(lib, "_moe_plan_sig", False):
            P, I, L = C.c_void_p, C.c_int, C.c_longlong
            lib.ix_moe_dispatch_plan.argtypes = [P, I, I, I, I, P, P, P, I, P, P, P]
            lib.ix_moe_gather_rows.argtypes = [P, L, P, P, P, I, I, I, P, P, P]
            lib.ix_moe_scatter_rows.argtypes = [P, L, P, P, I, I, I, P, P]
            lib.ix_moe_glu_scale_bwd.argtypes = [P, P, P, P, I, I, P, P, P]
            lib.ix_moe_grouped_gemm_nn.argtypes = [P, P, P, P, I, I, I, I, I, I, I, P]
            lib.ix_moe_grouped_gemm_tn.argtypes = [P, P, P, P, I, I, I, I, I, I, I, P]
            lib._moe_plan_sig = True
        self.lib = lib
        _native.check(lib.ix_moe_dispatch_plan(idx.contiguous().data_ptr(), T, k, num_experts, pad, self.offs.data_ptr(),
                                               self.row_of.data_ptr(), self.src_of_row.data_ptr(), self.r_cap, self.pos.data_ptr(),
                                               scratch.data_ptr(), _native.stream()), "ix_moe_dispatch_plan")

    def gather(self, y: torch.Tensor, w_flat: torch.Tensor | None):
        """(x_rows bf16 [r_cap, H], w_rows fp32 [r_cap]) in dispatch order; padding rows are zero."""
        H = y.shape[1]
        x_rows = torch.empty(self.r_cap, H, dtype=y.dtype, device=y.device)
        w_rows = torch.empty(self.r_cap, dtype=torch.float32, device=y.device)
        _native.check(self.lib.ix_moe_gather_rows(y.data_ptr(), y.stride(0), _native.ptr(w_flat), self.src_of_row.data_ptr(),
                                                  self.offs.data_ptr(), self.E, self.k, H, x_rows.data_ptr(), w_rows.data_ptr(),
                                                  _native.stream()), "ix_moe_gather_rows")
        return x_rows, w_rows

    def scatter(self, g: torch.Tensor) -> torch.Tensor:
        """d_rows[r] = g[token of r] (zero for padding): backward of the combine."""
        H = g.shape[1]
        out = torch.empty(self.r_cap, H, dtype=g.dtype, device=g.device)
        _native.check(self.lib.ix_moe_scatter_rows(g.data_ptr(), g.stride(0), self.src_of_row.data_ptr(), self.offs.data_ptr(), self.E,
                                                   self.k, H, out.data_ptr(), _native.stream()), "ix_moe_scatter_rows")
        return out


def grouped_gemm_nn(a: torch.Tensor, w: torch.Tensor, plan: DispatchPlan, out_f32: bool = False) -> torch.Tensor:
    """out[r] = a[r] @ w[e(r)] for w [E, Kred, N] (the input gradient of a grouped linear)."""
    R, Kred = a.shape
    E, _, N = w.shape
    out = torch.empty(R, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
    _native.check(plan.lib.ix_moe_grouped_gemm_nn(a.data_ptr(), w.data_ptr(), out.data_ptr(), plan.offs.data_ptr(), R, E, N, Kred,
                                                  a.stride(0), N, int(out_f32), _native.stream()), "ix_moe_grouped_gemm_nn")
    return out


def grouped_gemm_tn(a: torch.Tensor, b: torch.Tensor, plan: DispatchPlan, out: torch.Tensor | None = None,
                    accumulate: bool = False) -> torch.Tensor:
    """out[e] (+)= a[rows of e]^T @ b[rows of e] -> [E, M, N] (the weight gradient of a grouped linear)."""
    R, M = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(plan.E, M, N, dtype=torch.bfloat16, device=a.device)
        mode = 0
    else:
        assert out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (plan.E, M, N)
        mode = 2 if accumulate else 1
    _native.check(plan.lib.ix_moe_grouped_gemm_tn(a.data_ptr(), b.data_ptr(), out.data_ptr(), plan.offs.data_ptr(), R, plan.E, M, N,
                                                  a.stride(0), b.stride(0), mode, _native.stream()), "ix_moe_grouped_gemm_tn")
    return out


def _glu_scale(h: torch.Tensor, w_rows: torch.Tensor) -> torch.Tensor:
    """a2 = bf16(bf16(bf16(silu(g)) * u) * w_row): the two kernels whose roundings the fused GLU epilogue repeats."""
    a = F.swiglu_fwd(h)
    _native.check(_native.lib().ix_scale_rows(a.data_ptr(), w_rows.data_ptr(), a.shape[0], a.shape[1], _native.stream()), "ix_scale_rows")
    return a


class _ExpertsFn(torch.autograd.Function):
    """All experts of one layer, differentiable, as grouped tcgen05 launches with no host synchronisation:
    forward = plan, gather, grouped fc1, GLU x gate weight, grouped fc2 (fp32), fixed-order combine;
    backward = scatter of the output gradient, grouped NN / TN GEMMs for both linears, the GLU x weight VJP, and the
    fixed-order sum of the k row gradients of every token (no atomics)
    (reference: ISO/ops/moe/moe_batched_experts.py:301-400, moe_backward_kernel.py:254-401, moe_combine_backward.py:80-231).

    ``raw=True`` is the form the expert-parallel owner runs on the rows it received: one expert per input row (k = 1),
    the result stays fp32 and unrounded so that the SOURCE rank does the fixed-order sum and the single rounding."""

    @staticmethod
    def forward(ctx, y, w, gate_up, down, idx, shared, raw=False):
        E = gate_up.shape[0]
        _obs.note("moe.experts", "grouped_gemm")
        _obs.note("moe.combine", "fixed_order")
        plan = DispatchPlan(idx, E, 64)
        x_rows, w_rows = plan.gather(y, w.reshape(-1).contiguous())
        h = grouped_gemm(x_rows, gate_up, plan.offs, EPI_BF16)
        a2 = _glu_scale(h, w_rows)
        rows = grouped_gemm(a2, down, plan.offs, EPI_F32)
        out = torch.empty(y.shape[0], down.shape[1], dtype=torch.float32 if raw else y.dtype, device=y.device)
        if y.shape[0]:
            _native.check(_native.lib().ix_moe_combine(rows.data_ptr(), plan.pos.data_ptr(), _native.ptr(shared), out.data_ptr(),
                                                       y.shape[0], out.shape[1], plan.k, int(out.dtype == torch.bfloat16),
                                                       _native.stream()), "ix_moe_combine")
        ctx.plan = plan
        ctx.has_shared = shared is not None
        ctx.save_for_backward(y, h, w_rows, gate_up, down)
        ctx.mark_non_differentiable(idx)
        return out

    @staticmethod
    def backward(ctx, g):
        y, h, w_rows, gate_up, down = ctx.saved_tensors
        plan: DispatchPlan = ctx.plan
        g = g.to(y.dtype).contiguous()
        d_rows = plan.scatter(g)                                    # [R, H]
        a2 = _glu_scale(h, w_rows)                                  # recomputed (an elementwise pass) instead of kept
        d_a2 = grouped_gemm_nn(d_rows, down, plan)                  # [R, F]      down [E, H, F]
        d_down = grouped_gemm_tn(d_rows, a2, plan)                  # [E, H, F]
        del a2
        d_h = torch.empty_like(h)
        d_w_rows = torch.empty_like(w_rows)
        _native.check(plan.lib.ix_moe_glu_scale_bwd(h.data_ptr(), w_rows.data_ptr(), d_a2.data_ptr(), plan.offs.data_ptr(), plan.E,
                                                    h.shape[1] // 2, d_h.data_ptr(), d_w_rows.data_ptr(), _native.stream()),
                      "ix_moe_glu_scale_bwd")
        del d_a2
        x_rows, _ = plan.gather(y, None)
        d_gate_up = grouped_gemm_tn(d_h, x_rows, plan)              # [E, 2F, H]
        del x_rows
        d_x_rows = grouped_gemm_nn(d_h, gate_up, plan, out_f32=True)     # [R, H] fp32
        d_y = torch.empty_like(y)
        if y.shape[0]:
            _native.check(_native.lib().ix_moe_combine(d_x_rows.data_ptr(), plan.pos.data_ptr(), None, d_y.data_ptr(), y.shape[0],
                                                       y.shape[1], plan.k, int(y.dtype == torch.bfloat16), _native.stream()),
                          "ix_moe_combine")
        d_w = d_w_rows.index_select(0, plan.row_of[:plan.T * plan.k].long()).view(plan.T, plan.k)
        return d_y, d_w, d_gate_up, d_down, None, (g if ctx.has_shared else None), None


def _experts_fn_ok(y, gate_up, down) -> bool:
    return (y.is_cuda and y.dtype == torch.bfloat16 and gate_up.shape[2] % 64 == 0 and down.shape[2] % 64 == 0
            and down.shape[1] % 64 == 0 and (gate_up.shape[1] // 2) % 32 == 0 and gate_up.shape[0] <= 512)


def counts_to_offsets(counts: torch.Tensor) -> torch.Tensor:
    offs = torch.zeros(counts.numel() + 1, dtype=torch.int32, device=counts.device)
    offs[1:] = torch.cumsum(counts, 0)
    return offs


def moe_block(y: torch.Tensor, model, i: int) -> torch.Tensor:
    cfg, ps = model.cfg, model.ps
    pfx = f"layers.{i}.moe."
    T, h = y.shape
    E, k = cfg.num_experts, cfg.top_k
    logits = F.linear(y, model.p(pfx + "router.weight"), out_f32=True).float()
    bias = model.p(pfx + "router.expert_bias").float() if cfg.router == "sigmoid_bias" else None
    idx, w = route(logits, k, bias, cfg.router == "sigmoid_bias", cfg.norm_topk_prob)
    w = _with_aux_loss(logits, idx, w, cfg)
    gate_up, down = model.p(pfx + "experts.gate_up"), model.p(pfx + "experts.down")
    if ps.ep == 1 and _experts_fn_ok(y, gate_up, down):
        # single-rank experts on a GPU: routing tables, expert GEMMs and (with autograd) their VJPs are all kernels,
        # and nothing in the block reads a value back to the host
        shared = _shared_expert(y, model, pfx) if cfg.shared_expert_ffn else None
        if torch.is_grad_enabled() and (y.requires_grad or gate_up.requires_grad):
            _SERVED["moe.experts/grouped_autograd"] += 1
            return _ExpertsFn.apply(y, w, gate_up, down, idx, shared)
        _SERVED["moe.experts/grouped"] += 1
        plan = DispatchPlan(idx, E, 1)
        x_rows, w_rows = plan.gather(y, w.reshape(-1).contiguous())
        rows = expert_rows_grouped(x_rows, w_rows, plan.offs, gate_up, down)
        return combine_fixed_order(rows, plan.pos, y.dtype, shared)
    order, counts, pos = build_dispatch(idx, E)
    tok_of_row = torch.div(order, k, rounding_mode="floor")
    x_rows = y.index_select(0, tok_of_row)
    w_rows = w.reshape(-1).index_select(0, order)
    peer = None
    if ps.ep > 1 and y.is_cuda and not torch.is_grad_enabled():
        from . import moe_ep

        peer = moe_ep.get(ps.ep_group)
    if peer is not None:
        # dispatch, expert GEMMs and the return of the rows as our own kernels over peer memory
        rows, pos = peer.forward(y, idx, w, gate_up, down)
    elif ps.ep > 1:
        e_loc = E // ps.ep
        counts_l = counts.tolist()
        send = [sum(counts_l[r * e_loc:(r + 1) * e_loc]) for r in range(ps.ep)]
        # exchange per-expert counts so every owner knows its incoming group sizes
        cnt_in = torch.empty(ps.ep * e_loc, dtype=counts.dtype, device=counts.device)
        dist.all_to_all_single(cnt_in, counts.contiguous(), group=ps.ep_group)
        cnt_in_l = cnt_in.view(ps.ep, e_loc).tolist()
        recv = [sum(c) for c in cnt_in_l]
        xr = _AllToAll.apply(x_rows, send, recv, ps.ep_group)
        wr = _AllToAll.apply(w_rows, send, recv, ps.ep_group)
        if torch.is_grad_enabled() and xr.shape[0] and _experts_fn_ok(xr, gate_up, down):
            # under autograd on a GPU the owner runs its experts and their VJPs as grouped launches: the device plan sorts
            # the received rows by expert (stable, so source order is kept inside an expert) and pads every group
            _SERVED["moe.experts/nccl_grouped_autograd"] += 1
            own = torch.repeat_interleave(torch.arange(e_loc, device=y.device, dtype=torch.int32).repeat(ps.ep), cnt_in.view(-1),
                                          output_size=xr.shape[0])
            out_rows = _ExpertsFn.apply(xr, wr.view(-1, 1), gate_up, down, own.view(-1, 1), None, True)
            rows = _AllToAll.apply(out_rows, recv, send, ps.ep_group, torch.bfloat16 if y.dtype == torch.bfloat16 else None)
            shared = _shared_expert(y, model, pfx) if cfg.shared_expert_ffn else None
            return combine_fixed_order(rows, pos, y.dtype, shared)
        # received rows are grouped by (source rank, expert); regroup by expert, keeping source order
        segs, base = [], 0
        for r in range(ps.ep):
            for e in range(e_loc):
                segs.append((e, r, base, cnt_in_l[r][e]))
                base += cnt_in_l[r][e]
        perm = torch.cat([torch.arange(b, b + n, device=y.device) for e, r, b, n in sorted(segs) if n] or
                         [torch.zeros(0, dtype=torch.long, device=y.device)])
        loc_counts = [sum(cnt_in_l[r][e] for r in range(ps.ep)) for e in range(e_loc)]
        xs, wsr = xr.index_select(0, perm), wr.index_select(0, perm)
        if _grouped_ok(xs, gate_up, down):
            offs = counts_to_offsets(torch.tensor(loc_counts, dtype=torch.int64, device=y.device))
            out_rows = expert_rows_grouped(xs, wsr, offs, gate_up, down)
        else:
            out_rows = _expert_rows(xs, wsr, loc_counts, gate_up, down)
        back = torch.empty_like(out_rows)
        back[perm] = out_rows
        rows = _AllToAll.apply(back, recv, send, ps.ep_group, torch.bfloat16 if y.dtype == torch.bfloat16 else None)
    elif _grouped_ok(x_rows, gate_up, down):
        rows = expert_rows_grouped(x_rows, w_rows, counts_to_offsets(counts), gate_up, down)
    else:
        rows = _expert_rows(x_rows, w_rows, counts.tolist(), gate_up, down)
    _SERVED["moe.experts/" + ("peer" if peer is not None else "looped_or_nccl")] += 1
    shared = _shared_expert(y, model, pfx) if cfg.shared_expert_ffn else None
    return combine_fixed_order(rows, pos, y.dtype, shared)


def _shared_expert(y, model, pfx):
    from ..parallel import tp as tp_ops

    cfg, ps = model.cfg, model.ps
    gu = F.linear(tp_ops.copy_to_tp(y, ps), model.p(pfx + "shared.gate_up.weight"))   # column-parallel: sum the input grads
    shared = tp_ops.row_parallel_linear(F.swiglu(gu), model.p(pfx + "shared.down.weight"), ps, cfg)
    if cfg.shared_expert_gate:        # one scalar per token: sigmoid(y . w_gate), applied in fp32, one round
        gl = F.linear(y, model.p(pfx + "shared.gate.weight"), out_f32=True).float()
        if not gl.is_cuda:
            # the CPU sigmoid rounds a vector lane and a scalar tail differently, so a [T, 1] tensor's values would depend
            # on T; at full row width every element sits in a whole vector and a token's value is the same in any batch
            gl = gl.expand(-1, shared.shape[-1]).contiguous()
        shared = (shared.float() * torch.sigmoid(gl)).to(y.dtype)
    return shared
