"""Batch dispatch over the data-parallel ranks (reference: B/distributed/dispatch.py:87-195 ``MeshDispatch``,
B/workers/worker_dispatch.py). In the reference a controller process slices a batch, ships the slices to Ray actors
and concatenates what comes back; here every rank runs the same program, so dispatch is arithmetic: which rows of a
global batch are mine, and how per-rank results are put back in global order.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist


def dp_slice(n_rows: int, dp_rank: int, dp: int) -> slice:
    """Contiguous, equal shares (the batch size must divide: pad first with ``pad_training_input_batch``)."""
    if n_rows % dp:
        raise ValueError(f"{n_rows} rows do not split over {dp} data-parallel ranks; pad the batch")
    per = n_rows // dp
    return slice(dp_rank * per, (dp_rank + 1) * per)


def shard_batch(batch, ps):
    """This rank's rows of a global ``TensorBatch`` (identical on every rank)."""
    if ps.dp == 1:
        return batch
    s = dp_slice(batch.batch_size, ps.dp_rank, ps.dp)
    return batch.slice(s.start, s.stop)


def gather_rows(local: torch.Tensor, ps) -> torch.Tensor:
    """Concatenate per-rank row blocks in data-parallel rank order (inverse of ``shard_batch`` for one tensor)."""
    if ps.dp == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(ps.dp)]
    dist.all_gather(parts, local.contiguous(), group=ps.dp_group)
    return torch.cat(parts, 0)


def reduce_metrics(metrics: dict, ps, how: str = "mean") -> dict:
    """mean / min / max / sum of scalar metrics over the data-parallel group (reference: B/workers/worker_utils.py:102-128)."""
    if ps.dp == 1 or not metrics:
        return dict(metrics)
    keys = sorted(k for k, v in metrics.items() if isinstance(v, (int, float)))
    t = torch.tensor([float(metrics[k]) for k in keys], dtype=torch.float64)
    if dist.get_backend(ps.dp_group) == "nccl":
        t = t.cuda()
    op = {"mean": dist.ReduceOp.SUM, "sum": dist.ReduceOp.SUM, "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX}[how]
    dist.all_reduce(t, op=op, group=ps.dp_group)
    if how == "mean":
        t = t / ps.dp
    out = dict(metrics)
    out.update({k: float(v) for k, v in zip(keys, t.tolist())})
    return out


def set_numa_affinity(local_rank: int, gpus_per_node: int = 8) -> list[int] | None:
    """Pin this process to the CPU cores nearest its GPU, assuming cores are split evenly over the GPUs of a node
    (reference: NUMA affinity in B/workers/worker.py:236). Returns the core list, or None where not supported."""
    if not hasattr(os, "sched_setaffinity"):
        return None
    try:
        cores = sorted(os.sched_getaffinity(0))
        per = max(1, len(cores) // gpus_per_node)
        mine = cores[local_rank * per:(local_rank + 1) * per] or cores
        os.sched_setaffinity(0, mine)
        return mine
    except OSError:
        return None
