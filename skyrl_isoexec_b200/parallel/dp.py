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


def reduce_main_grads(main_grad: torch.Tensor, ps, bucket_elems: int = BUCKET_ELEMS) -> None:
    if ps.dp == 1:
        return
    from . import symm

    if main_grad.is_cuda and symm.enabled(ps.dp_group):
        symm.get(ps.dp_group).all_reduce_sum_(main_grad)
        return
    n = main_grad.numel()
    for lo in range(0, n, bucket_elems):
        dist.all_reduce(main_grad[lo:min(n, lo + bucket_elems)], group=ps.dp_group)
