"""NCCL housekeeping: communicator pre-warm and the transport capability record (reference:
ISO/runtimes/megatron/nccl_prewarm.py:215-259 six collectives per process group;
nccl_transport_capabilities.py:138-425 capability registry + guards).

NCCL builds a communicator's channels lazily, at the first collective of each kind; in a colocated RL job that
first call would otherwise land inside a timed step, or worse, while the rollout engine holds all spare memory.
``prewarm`` issues one small collective of every kind the framework uses on every group, once, at start-up.
``capabilities`` records which transports are usable (peer access, symmetric memory, NVLS as reported by the
environment) and is folded into the deployment identity; a kernel path asks it before choosing peer memory.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

_warmed: set = set()


def prewarm(groups: list, device=None) -> int:
    """all_reduce (sum, max), all_gather, reduce_scatter, all_to_all, broadcast, barrier on each group. Returns the
    number of collectives issued."""
    n = 0
    for g in groups:
        if g is None or id(g) in _warmed:
            continue
        w = dist.get_world_size(g)
        dev = device or ("cuda" if torch.cuda.is_available() and dist.get_backend(g) != "gloo" else "cpu")
        x = torch.ones(w * 4, device=dev)
        dist.all_reduce(x, group=g)
        dist.all_reduce(x, op=dist.ReduceOp.MAX, group=g)
        out = torch.empty(w * x.numel(), device=dev)
        dist.all_gather_into_tensor(out, x, group=g)
        n += 3
        if dev != "cpu":
            rs = torch.empty(x.numel() // w, device=dev)
            dist.reduce_scatter_tensor(rs, x, group=g)
            n += 1
        a2a = torch.empty_like(x)
        dist.all_to_all_single(a2a, x, group=g)
        dist.broadcast(x, src=dist.get_global_rank(g, 0), group=g)
        dist.barrier(group=g)
        n += 3
        _warmed.add(id(g))
    return n


def capabilities(group=None) -> dict:
    """What the fused kernels may use on this process. Read-only: nothing on the GPU is changed."""
    caps = {"backend": dist.get_backend(group) if dist.is_initialized() else "none", "peer_access": False,
            "symmetric_memory": False, "nvls_requested": os.environ.get("NCCL_NVLS_ENABLE", "") not in ("0",),
            "cuda": torch.cuda.is_available()}
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        cur = torch.cuda.current_device()
        caps["peer_access"] = all(torch.cuda.can_device_access_peer(cur, j) for j in range(n) if j != cur) if n > 1 else False
        import importlib.util

        caps["symmetric_memory"] = caps["peer_access"] and importlib.util.find_spec("torch.distributed._symmetric_memory") is not None
    return caps


def require(caps: dict, what: str) -> None:
    if not caps.get(what):
        raise RuntimeError(f"transport capability {what!r} is not available here ({caps}); use the NCCL transport")
