"""Long-context sequence parallelism for attention: Ulysses-style head/sequence all-to-all and an all-gather
form (reference: B/distributed/ulysses/utils.py:66-240 ``SeqAllToAll`` / gather helpers; the context-parallel
all-gather autograd of B/distributed/megatron/model_utils.py:1438-1540). Those two forms move bytes only, so the
attention kernel sees complete sequences and the single-split, fixed-block numerics are untouched. A ring /
blockwise variant (absent from the reference) is at the end of the file: chunks of K/V travel around the ranks and
the per-chunk results are folded in one fixed order; it is outside the bitwise contract.

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


# ------------------------------------------------------------------------------------ ring / blockwise attention
# The K/V chunks travel around the ring of context-parallel ranks; every rank attends its local queries to one chunk
# per step. The per-chunk results (o_b, lse_b) are kept and folded at the end in ASCENDING chunk order, whatever order
# they arrived in, so the block-combine order is one fixed function of the layout. This variant is outside the bitwise
# contract (the contract's attention consumes keys in 128-wide blocks with one running state); it exists for
# sequences whose K/V do not fit one GPU and whose head count does not divide for the all-to-all form.
class _RingShift(torch.autograd.Function):
    """Forward: pass ``x`` to the next rank of the ring and return what the previous rank passed. Backward: the
    gradient travels the other way."""

    @staticmethod
    def forward(ctx, x, ranks, me, group):
        ctx.ranks, ctx.me, ctx.group = ranks, me, group
        return _ring_exchange(x, ranks[(me + 1) % len(ranks)], ranks[(me - 1) % len(ranks)], group, me)

    @staticmethod
    def backward(ctx, g):
        ranks, me = ctx.ranks, ctx.me
        return _ring_exchange(g.contiguous(), ranks[(me - 1) % len(ranks)], ranks[(me + 1) % len(ranks)], ctx.group, me), None, None, None


def _ring_exchange(x, dst, src, group, me):
    x = x.contiguous()
    out = torch.empty_like(x)
    if dst == src and len({dst}) == 1 and dst == dist.get_rank():      # ring of one
        return x.clone()
    # even positions send first, odd positions receive first: no rank waits on a peer that is also waiting to send
    if me % 2 == 0:
        dist.send(x, dst, group=group)
        dist.recv(out, src, group=group)
    else:
        dist.recv(out, src, group=group)
        dist.send(x, dst, group=group)
    return out


def _chunk_attention(q, k, v, scale, q_off: int, k_off: int, causal: bool):
    """Local queries against ONE chunk of keys. q [n, Hq, D], k/v [m, Hkv, D]. Returns (o [n, Hq, D] fp32 normalised
    inside the chunk, lse [n, Hq] fp32; rows that see no key of the chunk get lse = -inf and o = 0)."""
    n, Hq, _ = q.shape
    m, Hkv, _ = k.shape
    G = Hq // Hkv
    qf = q.float().transpose(0, 1)                                   # [Hq, n, D]
    kf = k.float().repeat_interleave(G, 1).transpose(0, 1)           # [Hq, m, D]
    vf = v.float().repeat_interleave(G, 1).transpose(0, 1)
    s = (qf @ kf.transpose(1, 2)) * scale                            # [Hq, n, m]
    if causal:
        qi = torch.arange(q_off, q_off + n, device=q.device)[:, None]
        ki = torch.arange(k_off, k_off + m, device=q.device)[None, :]
        s = s.masked_fill((ki > qi)[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                                 # -inf where the whole row is masked
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
    return (p @ vf).transpose(0, 1), lse.transpose(0, 1)


def ring_attention(q, k, v, scale: float, ps, causal: bool = True):
    """Blockwise attention over ONE sequence cut into ``cp`` equal contiguous chunks; this rank holds chunk
    ``ps.cp_rank`` of q [n, Hq, D] and k, v [n, Hkv, D]. Differentiable (the ring shift carries gradients back).
    Returns this rank's [n, Hq, D] in q's dtype."""
    cp, r = ps.cp, ps.cp_rank
    n = q.shape[0]
    if cp == 1:
        o, _ = _chunk_attention(q, k, v, scale, 0, 0, causal)
        return o.to(q.dtype)
    parts = {}
    kv = torch.stack([k, v])                                          # one tensor, one shift per step: the backward
    for step in range(cp):                                            # of the ring is then a single chain on every rank
        src = (r - step) % cp                                         # whose chunk this rank holds at this step
        if not causal or src <= r:
            parts[src] = _chunk_attention(q, kv[0], kv[1], scale, r * n, src * n, causal)
        if step + 1 < cp:                                             # every rank shifts, also those that skipped
            kv = _RingShift.apply(kv, tuple(ps.cp_ranks), r, ps.cp_group)
    # fold in ascending chunk order: out = sum_b exp(lse_b - lse) o_b
    order = sorted(parts)
    lse = parts[order[0]][1]
    for b in order[1:]:
        lse = torch.logaddexp(lse, parts[b][1])
    out = None
    for b in order:
        o_b, lse_b = parts[b]
        w = torch.exp(lse_b - lse)
        w = torch.where(torch.isinf(lse_b), torch.zeros_like(w), w)
        term = o_b * w[..., None]
        out = term if out is None else out + term
    # A rank that skipped the later chunks (causal) still has to take part in the backward of every shift: tie the last
    # shifted tensor to the output with weight zero so that autograd walks the whole chain everywhere.
    out = out + kv.sum() * 0.0
    return out.to(q.dtype)
