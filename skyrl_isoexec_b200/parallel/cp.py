"""Long-context sequence parallelism for attention: Ulysses-style head/sequence all-to-all and an all-gather
form (reference: B/distributed/ulysses/utils.py:66-240 ``SeqAllToAll`` / gather helpers; the context-parallel
all-gather autograd of B/distributed/megatron/model_utils.py:1438-1540). No ring or blockwise attention
exists in the reference either; both forms below move bytes only, so the attention kernel sees complete
sequences and the single-split, fixed-block numerics are untouched.

Layout: the packed token dimension is cut into ``cp`` contiguous, equal chunks (pad the micro-batch to a
multiple of ``cp`` tokens); rank r holds chunk r of every per-token tensor.

  * ``ulysses_attention``  before attention, an all-to-all turns [T/cp, H, D] into [T, H/cp, D] (every rank: the
                           whole sequence for a slice of the heads); after it, the inverse. Needs cp | Hkv.
  * ``gather_sequence`` / ``scatter_sequence``  all-gather of a sequence-sharded tensor with the matching
                           backward (slice of the gradient), for K/V when the head count does not divide.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_sequence(x: torch.Tensor, cp_rank: int, cp: int) -> torch.Tensor:
    """This rank's contiguous chunk along dim 0 (length must divide)."""
    T = x.shape[0]
    assert T % cp == 0, f"{T} tokens do not split over cp={cp}; pad the micro-batch"
    n = T // cp
    return x[cp_rank * n:(cp_rank + 1) * n]


def pad_to_multiple(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def _all_to_all(x: torch.Tensor, group) -> torch.Tensor:
    """x [cp, ...] -> out [cp, ...] with out[j] = rank j's x[my_rank]."""
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x.contiguous(), group=group)     # equal splits along dim 0 (NCCL and gloo both have it)
    return out


class _SeqToHeads(torch.autograd.Function):
    """[T/cp, H, D] (my tokens, all heads) -> [T, H/cp, D] (all tokens, my heads)."""

    @staticmethod
    def forward(ctx, x, group, cp):
        ctx.group, ctx.cp = group, cp
        t, H, D = x.shape
        send = x.view(t, cp, H // cp, D).permute(1, 0, 2, 3).contiguous()       # [cp(dst), t, H/cp, D]
        recv = _all_to_all(send, group)                                          # [cp(src), t, H/cp, D]
        return recv.reshape(cp * t, H // cp, D)

    @staticmethod
    def backward(ctx, g):
        return _HeadsToSeq.apply(g, ctx.group, ctx.cp), None, None


class _HeadsToSeq(torch.autograd.Function):
    """[T, H/cp, D] -> [T/cp, H, D], the inverse of ``_SeqToHeads``."""

    @staticmethod
    def forward(ctx, x, group, cp):
        ctx.group, ctx.cp = group, cp
        T, h, D = x.shape
        t = T // cp
        send = x.view(cp, t, h, D).contiguous()                                  # [cp(dst = owner of the token chunk), t, h, D]
        recv = _all_to_all(send, group)                                          # [cp(src = owner of a head slice), t, h, D]
        return recv.permute(1, 0, 2, 3).reshape(t, cp * h, D)

    @staticmethod
    def backward(ctx, g):
        return _SeqToHeads.apply(g.contiguous(), ctx.group, ctx.cp), None, None


def ulysses_attention(q, k, v, meta_full, scale: float, ps, attention_fn=None):
    """q [T/cp, Hq, D], k/v [T/cp, Hkv, D] sequence-sharded; ``meta_full`` describes the FULL packed micro-batch.
    Returns [T/cp, Hq, D]."""
    from ..ops import functional as F

    cp = ps.cp
    attention_fn = attention_fn or F.attention
    if cp == 1:
        return attention_fn(q, k, v, meta_full, scale)
    assert q.shape[1] % cp == 0 and k.shape[1] % cp == 0, "Ulysses needs cp to divide the query and KV head counts"
    qf = _SeqToHeads.apply(q, ps.cp_group, cp)
    kf = _SeqToHeads.apply(k, ps.cp_group, cp)
    vf = _SeqToHeads.apply(v, ps.cp_group, cp)
    o = attention_fn(qf.contiguous(), kf.contiguous(), vf.contiguous(), meta_full, scale)
    return _HeadsToSeq.apply(o, ps.cp_group, cp)


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, cp, rank):
        ctx.group, ctx.cp, ctx.rank = group, cp, rank
        parts = [torch.empty_like(x) for _ in range(cp)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, 0)

    @staticmethod
    def backward(ctx, g):
        # every rank used the gathered tensor: the gradient of my chunk is the SUM over ranks of their slice for it
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        n = g.shape[0] // ctx.cp
        return g[ctx.rank * n:(ctx.rank + 1) * n], None, None, None


def gather_sequence(x, ps):
    """All-gather a sequence-sharded tensor along dim 0 (differentiable)."""
    if ps.cp == 1:
        return x
    return _GatherSeq.apply(x, ps.cp_group, ps.cp, ps.cp_rank)


def scatter_sequence(x, ps):
    return shard_sequence(x, ps.cp_rank, ps.cp) if ps.cp > 1 else x
