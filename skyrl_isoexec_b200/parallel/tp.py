"""Tensor-parallel linears with a TP-invariant reduction ("pik" in the reference,
ISO/ops/collectives/pik/plan.py:20-36,104-119 and pik/allreduce.py:1018-1168).

The K reduction of a row-parallel linear is fixed as G equal leaves folded by a balanced
binary fp32 tree (left operand = lower leaf index). A rank at TP degree C owns the G/C
consecutive leaves of its K slice, i.e. one whole subtree; the cross-rank step is the upper
levels of the SAME tree. Any C dividing G therefore yields identical bits, and C == G costs
nothing extra (one leaf per rank = a plain GEMM).

Transports for the upper levels:
  * ``symm``  - peer-memory kernel (csrc/tree_allreduce.cu): every rank stores its partial in
                symmetric memory, then reads all peers and folds in tree order (one launch);
  * ``nccl``  - all_gather of the fp32 partials + local fold (the baseline / fallback);
  * CPU/gloo  - all_gather + the same fold in torch.
"""

from __future__ import annotations

import os
from collections import Counter
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..core import observe as _obs
from ..ops import functional as F
from ..ops import _cpu, _native


@dataclass(frozen=True)
class ReductionPlan:
    num_leaves: int = 8
    leaf_dtype: str = "fp32"  # "fp32" | "bf16": optional rounding at the leaf boundary only

    def validate(self, K: int, tp: int) -> None:
        G = self.num_leaves
        if G < 1 or G & (G - 1):
            raise ValueError(f"num_leaves={G} must be a power of two")
        if G % tp:
            raise ValueError(f"TP degree {tp} does not divide the {G} leaves")
        if K % G:
            raise ValueError(f"K={K} is not divisible into {G} leaves")

    def leaves_per_rank(self, tp: int) -> int:
        return self.num_leaves // tp

    def contract_string(self, arch: str) -> str:
        return f"pik-tree:G={self.num_leaves}:leaf={self.leaf_dtype}:arch={arch}"


def combine_order(n: int) -> list[tuple[int, int]]:
    """(dst, src) pairs of the balanced tree over n slots: stride 1, 2, 4, ...; slot[i] += slot[i+stride]."""
    out, stride = [], 1
    while stride < n:
        out += [(i, i + stride) for i in range(0, n, 2 * stride)]
        stride *= 2
    return out


def tree_fold(parts: torch.Tensor) -> torch.Tensor:
    """Fold ``parts[n, ...]`` (fp32) along dim 0 in tree order. n must be a power of two."""
    n = parts.shape[0]
    buf = [parts[i] for i in range(n)]
    for dst, src in combine_order(n):
        buf[dst] = buf[dst] + buf[src]
    return buf[0]


def leaftree_gemm(x: torch.Tensor, w: torch.Tensor, leaves: int, round_leaf: bool = False) -> torch.Tensor:
    """fp32 [M,N] = tree over ``leaves`` K-slices of x[M,K] @ w[N,K]^T (local subtree of one rank)."""
    M, K = x.shape
    N = w.shape[0]
    assert K % leaves == 0
    if leaves == 1 and not round_leaf:
        return F.gemm_nt(x, w, out_f32=True)
    if x.is_cuda:
        LK = K // leaves
        parts = torch.stack([F.gemm_nt(x[:, j * LK:(j + 1) * LK], w[:, j * LK:(j + 1) * LK], out_f32=True)
                             for j in range(leaves)])
        if round_leaf:
            parts = parts.bfloat16().float()
        return tree_fold(parts)
    out = torch.empty(M, N, dtype=torch.float32)
    if M:
        _cpu.lib().ixc_leaftree_gemm(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, leaves, int(round_leaf),
                                     x.stride(0), w.stride(0), N, _cpu.dt(x))
    return out


def tree_all_reduce(partial: torch.Tensor, group, tp: int) -> torch.Tensor:
    """Upper levels of the tree across the TP group: gather every rank's fp32 partial (rank order =
    leaf order) and fold. All ranks end with identical bits."""
    if tp == 1:
        return partial
    from . import symm

    if partial.is_cuda and symm.enabled(group):
        return symm.tree_all_reduce(partial, group)
    part = partial.contiguous().view(-1)
    gathered = torch.empty(tp * part.numel(), dtype=partial.dtype, device=partial.device)
    dist.all_gather_into_tensor(gathered, part, group=group)
    return tree_fold(gathered.view((tp,) + tuple(partial.shape)))


# ------------------------------------------------------------------------------------ census and admission
# Which transport served how many calls (reference: the pik transport census, ISO/ops/collectives/pik/allreduce.py:213-226,
# 719-808), and the per-shape admission of the fused kernel (reference: pik/allreduce.py:476-486,1018-1068): the first
# call of a shape runs BOTH the fused kernel and the plain path (leaf-tree GEMM, then the tree all-reduce), compares the
# bits, and every rank of the group takes the worst answer (MIN all-reduce). A shape that is not admitted stays on
# the plain path for the life of the process.
_CENSUS: Counter = Counter()
_ADMITTED: dict = {}


def transport_census(reset: bool = False) -> dict:
    """{(operation, transport): calls served}. Transports: ``fused_peer`` (GEMM + collective in one kernel),
    ``peer_tree`` (stand-alone tree all-reduce over peer memory), ``nccl`` / ``gloo`` (all-gather + local fold),
    ``local`` (tp = 1), ``refused`` (a shape whose probe failed, served by the plain path)."""
    out = {f"{op}/{tr}": n for (op, tr), n in sorted(_CENSUS.items())}
    if reset:
        _CENSUS.clear()
    return out


def admitted_shapes() -> dict:
    return dict(_ADMITTED)


def _plain_row_parallel(x, w, ps, leaves_local, round_leaf):
    part = leaftree_gemm(x, w, leaves_local, round_leaf)
    return tree_all_reduce(part, ps.tp_group, ps.tp)


def admit_fused_row_parallel(rt, ps, x, w, leaves_local, fused_dtype):
    """Returns (admitted, result of THIS call or None). The probe runs once per (group, size class, N, K, leaves,
    dtype); ``ISOEXEC_B200_TP_ADMISSION=0`` admits without probing."""
    from ..core.testing import bitwise_equal

    M = x.shape[0]
    key = (id(ps.tp_group), "small" if M <= 256 else "large", w.shape[0], x.shape[1], leaves_local, str(fused_dtype))
    if key in _ADMITTED:
        return _ADMITTED[key], None
    if os.environ.get("ISOEXEC_B200_TP_ADMISSION", "1") == "0":
        _ADMITTED[key] = True
        return True, None
    want = _plain_row_parallel(x, w, ps, leaves_local, False).to(fused_dtype)
    ok = True
    try:
        got = rt.row_parallel(x, w, leaves_local, out_dtype=fused_dtype)
        rt.check()
        ok = bool(bitwise_equal(got, want))
    except Exception:  # noqa: BLE001 - a probe that cannot run is a refusal, not a crash
        ok = False
    if ps.tp > 1 and dist.is_initialized():
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=x.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=ps.tp_group)
        ok = bool(int(flag.item()))
    _ADMITTED[key] = ok
    return ok, want       # the plain result has the same bits when admitted and is the fallback when not


class _RowParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, ps, leaves_local, round_leaf, out_dtype):
        ctx.save_for_backward(x, w)
        if x.is_cuda and not round_leaf and x.dtype == torch.bfloat16 and x.stride(-1) == 1 and x.stride(0) % 8 == 0:
            from . import tp_fused

            if tp_fused.fused_ok(x.shape[0], w.shape[0], x.shape[1], leaves_local):
                # one kernel: leaf accumulators in TMEM, leaf tree in the epilogue, rank tree over peer memory
                if ps.tp == 1:
                    _CENSUS[("row_parallel", "local")] += 1
                    return tp_fused.leaftree_gemm_fused(x, w, leaves_local, out_f32=out_dtype == torch.float32).to(out_dtype)
                rt = tp_fused.get(ps.tp_group)
                if rt is not None:
                    fdt = out_dtype if out_dtype == torch.float32 else torch.bfloat16
                    ok, first = admit_fused_row_parallel(rt, ps, x, w, leaves_local, fdt)
                    _CENSUS[("row_parallel", "fused_peer" if ok else "refused")] += 1
                    if first is None:
                        first = rt.row_parallel(x, w, leaves_local, out_dtype=fdt) if ok else _plain_row_parallel(x, w, ps, leaves_local, False)
                    return first.to(out_dtype)
        full = _plain_row_parallel(x, w, ps, leaves_local, round_leaf)
        if ps.tp > 1:
            from . import symm

            _CENSUS[("row_parallel", "peer_tree" if (x.is_cuda and symm.enabled(ps.tp_group)) else str(dist.get_backend(ps.tp_group)))] += 1
        else:
            _CENSUS[("row_parallel", "local")] += 1
        return full.to(out_dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.to(w.dtype)
        return F.gemm_nn(dy, w), F.gemm_tn(dy, x), None, None, None, None


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, ps, cfg, sp: bool = False) -> torch.Tensor:
    """y = x_full @ w_full^T where this rank holds the K slice x[:, K/tp], w[:, K/tp].

    With ``cfg.pik_leaves == 0`` (TP pinned, same degree on both sides) and tp == 1 this is the
    plain batch-invariant GEMM. Otherwise the leaf tree runs so that every TP degree dividing
    ``cfg.pik_leaves`` produces the same bits."""
    G = getattr(cfg, "pik_leaves", 0)
    # one op in the contract's eyes whatever the degree: a tree whose cross-rank levels are empty at tp = 1
    impl = "pik_tree" if x.is_cuda else "cpu_pik_tree"
    _obs.note("collectives.row_parallel", impl)
    _obs.note("collectives.tree_all_reduce", impl)
    if ps.tp == 1 and (G <= 1 or not cfg.tp_invariant):
        return F.linear(x, w)
    plan = ReductionPlan(G)
    plan.validate(w.shape[1] * ps.tp, ps.tp)
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    y = _RowParallel.apply(x2, w, ps, plan.leaves_per_rank(ps.tp), plan.leaf_dtype == "bf16", x.dtype)
    if ps.tp > 1 and sp:
        # sequence parallelism: this rank continues with its rows of the tree sum (the same bits as the all-reduced rows)
        return _KeepRows.apply(y, ps)
    return y.reshape(*shp[:-1], w.shape[0])


def column_parallel_gather(y_local: torch.Tensor, ps) -> torch.Tensor:
    """All-gather the column shards of a column-parallel output along the last dim (byte movement only)."""
    if ps.tp == 1:
        return y_local
    parts = [torch.empty_like(y_local) for _ in range(ps.tp)]
    dist.all_gather(parts, y_local.contiguous(), group=ps.tp_group)
    return torch.cat(parts, dim=-1)


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward: input of a column-parallel region."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def copy_to_tp(x, ps, sp_T: int | None = None):
    """Input of a column-parallel region. ``sp_T``: sequence parallelism is on, ``x`` holds this rank's rows of ``sp_T``
    and is gathered (backward: the ranks' partial input gradients are summed and this rank's rows are kept)."""
    if ps.tp > 1 and sp_T is not None:
        return _GatherRows.apply(x, sp_T, ps, True)
    if ps.tp == 1 or not (torch.is_grad_enabled() and x.requires_grad):
        return x
    return _CopyToTP.apply(x, ps.tp_group)


# ------------------------------------------------------------------------------------ sequence parallelism
# Megatron-style sequence parallelism for the differentiable trainer forward: between the tensor-parallel regions the
# residual stream, the norms and the residual adds live on T / tp rows per rank instead of being repeated on every rank.
# A column-parallel region is entered by gathering the rows (backward: the partial input gradients of the ranks are
# summed and scattered), a row-parallel region is left by keeping this rank's rows of the tree sum (backward: the row
# gradients of all ranks are gathered). Every row is computed by the same kernels from the same inputs as without it,
# so the forward bits do not change (reference: B/workers/megatron sequence_parallel; ISO/ops/collectives/pik tree
# reduce-scatter, pik/allreduce.py:476-486).
def sp_rows(T: int, ps) -> tuple[int, int]:
    """[lo, hi) of the T rows that tensor-parallel rank ``ps.tp_rank`` keeps: equal shares, the remainder on the last ranks."""
    base, rem = divmod(T, ps.tp)
    start = lambda r: r * base + max(0, r - (ps.tp - rem))
    return start(ps.tp_rank), start(ps.tp_rank + 1)


def _gather_rows(x_loc: torch.Tensor, T: int, ps) -> torch.Tensor:
    base, rem = divmod(T, ps.tp)
    sizes = [base + (1 if r >= ps.tp - rem else 0) for r in range(ps.tp)]
    mx = max(sizes)
    pad = x_loc if x_loc.shape[0] == mx else torch.cat([x_loc, x_loc.new_zeros((mx - x_loc.shape[0],) + tuple(x_loc.shape[1:]))])
    parts = [torch.empty_like(pad) for _ in range(ps.tp)]
    dist.all_gather(parts, pad.contiguous(), group=ps.tp_group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], 0)


class _GatherRows(torch.autograd.Function):
    """Rows of every rank -> all T rows. ``summed``: the incoming gradient is a per-rank PARTIAL (input of a
    column-parallel region): sum over ranks, keep this rank's rows. Otherwise it is already the same on every rank
    (output of the final norm): keep this rank's rows."""

    @staticmethod
    def forward(ctx, x_loc, T, ps, summed):
        ctx.cfg = (T, ps, summed)
        return _gather_rows(x_loc, T, ps)

    @staticmethod
    def backward(ctx, g):
        T, ps, summed = ctx.cfg
        if summed:
            g = g.clone()
            dist.all_reduce(g, group=ps.tp_group)
        lo, hi = sp_rows(T, ps)
        return g[lo:hi], None, None, None


class _KeepRows(torch.autograd.Function):
    """All T rows (the same on every rank) -> this rank's rows; backward gathers the row gradients of all ranks, which is
    the full gradient every rank would have had without sequence parallelism."""

    @staticmethod
    def forward(ctx, x, ps):
        ctx.cfg = (x.shape[0], ps)
        lo, hi = sp_rows(x.shape[0], ps)
        return x[lo:hi]

    @staticmethod
    def backward(ctx, g):
        T, ps = ctx.cfg
        return _gather_rows(g.contiguous(), T, ps), None


def sp_scatter(x: torch.Tensor, ps) -> torch.Tensor:
    """Replicated rows -> this rank's share (entering the sequence-parallel stream, e.g. after the embedding)."""
    return _KeepRows.apply(x, ps)


def sp_gather(x_loc: torch.Tensor, T: int, ps, summed: bool) -> torch.Tensor:
    return _GatherRows.apply(x_loc, T, ps, summed)


class _TiedHeadSlice(torch.autograd.Function):
    """Vocabulary shard of a replicated (tied) embedding used as the LM head. Backward returns the
    full-size gradient with every rank's shard filled in (sum over TP), so the replicated parameter
    receives the same gradient on every rank."""

    @staticmethod
    def forward(ctx, w, ps):
        ctx.ps = ps
        n = w.shape[0] // ps.tp
        return w[ps.tp_rank * n:(ps.tp_rank + 1) * n]

    @staticmethod
    def backward(ctx, g):
        ps = ctx.ps
        n = g.shape[0]
        full = g.new_zeros((n * ps.tp,) + tuple(g.shape[1:]))
        full[ps.tp_rank * n:(ps.tp_rank + 1) * n] = g
        dist.all_reduce(full, group=ps.tp_group)
        return full, None


def tied_head_slice(w, ps):
    if torch.is_grad_enabled() and w.requires_grad:
        return _TiedHeadSlice.apply(w, ps)
    n = w.shape[0] // ps.tp
    return w[ps.tp_rank * n:(ps.tp_rank + 1) * n]
