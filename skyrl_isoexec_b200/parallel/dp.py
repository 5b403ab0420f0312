"""Data-parallel gradient reduction over the flat fp32 main-gradient buffer.

The buffer is cut into fixed-size buckets in storage order and the buckets are reduced in that
order, so the association of the sum does not depend on timing. Transport: the peer-memory
reduce-scatter kernel when symmetric memory is registered for the DP group
(``parallel/symm_runtime.py``), else NCCL all-reduce (gloo on CPU). Gradients are summed, not
averaged: the controller has already normalised the advantages by the GLOBAL mini-batch size.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

BUCKET_ELEMS = 64 << 20  # 256 MiB of fp32 per bucket: large enough that launch latency is noise


def reduce_main_grads(main_grad: torch.Tensor, ps, bucket_elems: int = BUCKET_ELEMS, ranges=None, group=None) -> None:
    """Sum ``main_grad`` (or only its ``ranges`` = [(lo, hi), ...] of elements) over ``group`` (default: the DP group)."""
    group = group if group is not None else ps.dp_group
    if group is None or dist.get_world_size(group) == 1:
        return
    from . import symm

    pieces = [main_grad] if ranges is None else [main_grad[lo:hi] for lo, hi in ranges if hi > lo]
    for piece in pieces:
        if piece.is_cuda and symm.enabled(group):
            symm.get(group).all_reduce_sum_(piece)
            continue
        n = piece.numel()
        for lo in range(0, n, bucket_elems):
            dist.all_reduce(piece[lo:min(n, lo + bucket_elems)], group=group)


def split_ranges_by_expert_sharding(store) -> tuple[list, list]:
    """(ranges of parameters replicated over the data-parallel group, ranges of expert-parallel shards), merged into
    maximal contiguous runs in storage order."""
    import math

    dense, expert = [], []
    for name in store.order:
        s = store.specs[name]
        lo, hi = s.offset, s.offset + math.prod(s.shape)
        tgt = expert if s.ep_sharded else dense
        if tgt and tgt[-1][1] >= lo - store.ALIGN and (not (expert if tgt is dense else dense) or (expert if tgt is dense else dense)[-1][1] <= tgt[-1][1]):
            tgt[-1] = (tgt[-1][0], hi)
        else:
            tgt.append((lo, hi))
    return dense, expert
