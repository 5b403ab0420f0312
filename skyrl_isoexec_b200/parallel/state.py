"""Process topology: one process per GPU, ranks laid out TP-fastest, then EP/DP, then PP.

The reference obtains these groups from Megatron's mpu (B/distributed/megatron/megatron_strategy.py:281-323);
here they are plain ``torch.distributed`` groups (NCCL on GPUs, gloo on CPU) created once.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class ParallelState:
    world_size: int = 1
    rank: int = 0
    tp: int = 1
    pp: int = 1
    dp: int = 1
    ep: int = 1
    cp: int = 1
    tp_rank: int = 0
    pp_rank: int = 0
    dp_rank: int = 0
    ep_rank: int = 0
    cp_rank: int = 0
    tp_group: object = None
    pp_group: object = None
    dp_group: object = None
    ep_group: object = None
    edp_group: object = None      # ranks that hold the SAME expert shard (expert data parallel)
    kvr_group: object = None      # consecutive TP ranks that share one (replicated) KV head, when tp > num_kv_heads
    kvr_ranks: list = field(default_factory=lambda: [0])
    kvr_rank: int = 0
    cp_group: object = None
    tp_ranks: list = field(default_factory=lambda: [0])
    dp_ranks: list = field(default_factory=lambda: [0])
    ep_ranks: list = field(default_factory=lambda: [0])
    edp_ranks: list = field(default_factory=lambda: [0])
    edp_rank: int = 0
    pp_ranks: list = field(default_factory=lambda: [0])
    cp_ranks: list = field(default_factory=lambda: [0])

    @staticmethod
    def single() -> "ParallelState":
        return ParallelState()

    @property
    def is_first_pp(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_pp(self) -> bool:
        return self.pp_rank == self.pp - 1

    @staticmethod
    def build(tp: int = 1, pp: int = 1, ep: int = 1, cp: int = 1, ranks: list[int] | None = None, kv_rep: int = 1) -> "ParallelState":
        """Create the groups for a job (or for the sub-job made of ``ranks``). Every process of the
        default group must call this with the same arguments (``new_group`` is collective)."""
        if not dist.is_initialized():
            assert tp == pp == ep == cp == 1, "parallel degrees > 1 need torch.distributed"
            return ParallelState.single()
        me = dist.get_rank()
        ranks = list(range(dist.get_world_size())) if ranks is None else list(ranks)
        n = len(ranks)
        assert n % (tp * pp * cp) == 0, f"{n} ranks not divisible by tp*pp*cp={tp * pp * cp}"
        dp = n // (tp * pp * cp)
        assert dp % ep == 0 or ep % dp == 0 or ep == 1, (dp, ep)
        st = ParallelState(world_size=n, rank=me, tp=tp, pp=pp, dp=dp, ep=ep, cp=cp)
        # index = ((pp_i * dp + dp_i) * cp + cp_i) * tp + tp_i
        def idx(pp_i, dp_i, cp_i, tp_i):
            return ranks[((pp_i * dp + dp_i) * cp + cp_i) * tp + tp_i]

        def mk(members_lists, attr_group, attr_ranks, attr_rank):
            for members in members_lists:
                g = dist.new_group(members) if len(members) > 1 else None
                if me in members:
                    setattr(st, attr_group, g)
                    setattr(st, attr_ranks, members)
                    setattr(st, attr_rank, members.index(me))

        mk([[idx(p, d, c, t) for t in range(tp)] for p in range(pp) for d in range(dp) for c in range(cp)],
           "tp_group", "tp_ranks", "tp_rank")
        mk([[idx(p, d, c, t) for d in range(dp)] for p in range(pp) for c in range(cp) for t in range(tp)],
           "dp_group", "dp_ranks", "dp_rank")
        mk([[idx(p, d, c, t) for p in range(pp)] for d in range(dp) for c in range(cp) for t in range(tp)],
           "pp_group", "pp_ranks", "pp_rank")
        mk([[idx(p, d, c, t) for c in range(cp)] for p in range(pp) for d in range(dp) for t in range(tp)],
           "cp_group", "cp_ranks", "cp_rank")
        if kv_rep > 1:
            # tp > num_kv_heads: kv_rep consecutive TP ranks hold copies of one KV head (models/decoder.py)
            assert tp % kv_rep == 0, (tp, kv_rep)
            mk([[idx(p, d, c, t0 + t) for t in range(kv_rep)] for p in range(pp) for d in range(dp) for c in range(cp)
                for t0 in range(0, tp, kv_rep)], "kvr_group", "kvr_ranks", "kvr_rank")
        if ep > 1:
            # expert parallel spans (dp x tp) ranks of one pipeline stage, ep consecutive ranks per group
            stage = lambda p: [idx(p, d, c, t) for d in range(dp) for c in range(cp) for t in range(tp)]
            groups = []
            for p in range(pp):
                s = stage(p)
                assert len(s) % ep == 0, f"stage size {len(s)} not divisible by ep={ep}"
                groups += [s[i:i + ep] for i in range(0, len(s), ep)]
            mk(groups, "ep_group", "ep_ranks", "ep_rank")
            # ranks with the same position in their EP group hold the same experts: their expert gradients are summed
            edp = []
            for p in range(pp):
                s = stage(p)
                edp += [[s[i + r] for i in range(0, len(s), ep)] for r in range(ep)]
            mk(edp, "edp_group", "edp_ranks", "edp_rank")
        return st


def init_distributed(backend: str | None = None, timeout_s: int | None = None) -> tuple[int, int, int]:
    """Initialise the default process group from the torchrun environment. Returns
    (rank, world_size, local_rank). A no-op for a single process without RANK set. The collective timeout is
    ``timeout_s``, else ``SKYRL_WORKER_NCCL_TIMEOUT_IN_S`` (reference: R/env_vars.py:22), else 600 s."""
    import datetime

    if timeout_s is None:
        timeout_s = int(os.environ.get("SKYRL_WORKER_NCCL_TIMEOUT_IN_S", "600"))

    if "RANK" not in os.environ or int(os.environ.get("WORLD_SIZE", "1")) == 1:
        return 0, 1, int(os.environ.get("LOCAL_RANK", "0"))
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    if not dist.is_initialized():
        if backend is None:
            backend = "cpu:gloo,cuda:nccl" if torch.cuda.is_available() else "gloo"
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
        kw = {}
        if torch.cuda.is_available():
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, local
