"""Expert parallelism over NVLink peer memory for inference-mode MoE layers (engine decode/prefill and the
trainer's no-grad scoring pass): counts exchange, row dispatch, grouped expert GEMMs and the return of the
expert outputs all run as our own kernels on symmetric memory (csrc/moe_ep_peer.cu,
csrc/moe_grouped_gemm.cu); nothing goes through NCCL and nothing returns to the host between them.

The gradient-carrying training pass keeps the autograd all-to-all in ``ops/moe.py``.

Order of one layer on every rank (all ranks call ``forward`` for the same layers in the same order):
  counts -> dispatch push -> handshake -> resolve return addresses -> grouped fc1(+SwiGLU, gate weight)
  -> grouped fc2 with rows scattered to their source rank -> handshake -> local fixed-order combine.
The two handshakes are what make single buffering safe: a rank can only write into a peer's receive
buffers (or result rows) after that peer has passed the previous layer's second (first) handshake.
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..core import observe as _obs
from . import _native
from . import moe as M

_P, _I, _L = C.c_void_p, C.c_int, C.c_longlong


class EPPeer:
    def __init__(self, group, hidden: int, num_experts: int, max_rows_local: int, capacity_rows: int | None = None, device=None):
        """``max_rows_local``: most dispatch rows (tokens x top_k) this rank sends in one layer call;
        ``capacity_rows``: most rows this rank may RECEIVE (default: every rank's rows, the worst case)."""
        import torch.distributed._symmetric_memory as sm

        self.group = group
        self.rank, self.W = dist.get_rank(group), dist.get_world_size(group)
        self.E, self.H = num_experts, hidden
        assert num_experts % self.W == 0
        self.e_loc = num_experts // self.W
        self.max_rows = max_rows_local
        self.cap = capacity_rows or max_rows_local * self.W
        dev = torch.device(device or f"cuda:{torch.cuda.current_device()}")
        self.xbuf = sm.empty(self.cap * hidden, dtype=torch.bfloat16, device=dev)
        self.wbuf = sm.empty(self.cap, dtype=torch.float32, device=dev)
        self.dstbuf = sm.empty(self.cap, dtype=torch.int64, device=dev)
        self.rows = sm.empty(max_rows_local * hidden, dtype=torch.float32, device=dev)
        self.cnt = sm.empty(self.W * num_experts, dtype=torch.int32, device=dev)
        self.flags = sm.empty(64, dtype=torch.int32, device=dev)
        self.flags.zero_()
        self.cnt.zero_()
        torch.cuda.synchronize()
        name = group.group_name if group is not None else dist.group.WORLD.group_name
        hs = [sm.rendezvous(t, group=name) for t in (self.xbuf, self.wbuf, self.dstbuf, self.rows, self.cnt, self.flags)]
        dist.barrier(group=group)
        self._handles = hs
        arr = lambda h: (C.c_longlong * self.W)(*[int(p) for p in h.buffer_ptrs])  # noqa: E731
        self.p_x, self.p_w, self.p_dst, self.p_rows, self.p_cnt, self.p_flags = (arr(h) for h in hs)
        # flag slots: [0, W) counts exchange; [16, 16+W) handshakes
        self.p_flags_hs = (C.c_longlong * self.W)(*[int(p) + 64 for p in hs[5].buffer_ptrs])
        self.send_base = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.local_off = torch.zeros(num_experts + 1, dtype=torch.int32, device=dev)
        self.own_offs = torch.zeros(self.e_loc + 1, dtype=torch.int32, device=dev)
        self.epoch = 0
        lib = _native.lib()
        lib.ix_ep_counts.argtypes = [_P, _P, _P, _I, _I, _I, C.c_uint, _I, _I, _P, _P, _P, _P]
        lib.ix_ep_dispatch.argtypes = [_P, _P, _P, _P, _P, _P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]
        lib.ix_ep_resolve_dst.argtypes = [_P, _P, _P, _I, _I, _L, _I, _P]
        lib.ix_peer_handshake.argtypes = [_P, _I, _I, C.c_uint, _P]
        self.lib = lib

    def _handshake(self) -> None:
        self.epoch += 1
        _native.check(self.lib.ix_peer_handshake(self.p_flags_hs, self.rank, self.W, self.epoch, _native.stream()), "ix_peer_handshake")

    def forward(self, y: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor) -> tuple:
        """y [T, H] bf16 local tokens, idx int32 [T, k] global expert ids, w fp32 [T, k] gate weights; gate_up/down:
        this rank's experts. Returns (rows fp32 [T*k, H] in local dispatch order, pos [T, k]) for the fixed-order combine."""
        T, k = idx.shape
        R = T * k
        if R > self.max_rows:
            raise ValueError(f"{R} dispatch rows exceed the {self.max_rows} the peer buffers were sized for")
        st = _native.stream()
        _obs.note("moe.experts", "grouped_gemm")                # the owner's fc1 (SwiGLU x gate weight epilogue) and fc2
        _obs.note("activation.swiglu", "fused_swiglu")
        order, counts, pos = M.build_dispatch(idx, self.E)
        tok_of_row = torch.div(order, k, rounding_mode="floor")
        expert_of_row = idx.reshape(-1).index_select(0, order).contiguous()
        w_rows = w.reshape(-1).index_select(0, order).contiguous()
        self.epoch += 1
        _native.check(self.lib.ix_ep_counts(self.p_cnt, self.p_flags, counts.data_ptr(), self.rank, self.W, self.E, self.epoch, 0, self.cap,
                                            self.send_base.data_ptr(), self.local_off.data_ptr(), self.own_offs.data_ptr(), st), "ix_ep_counts")
        _native.check(self.lib.ix_ep_dispatch(self.p_cnt, self.p_flags, self.p_x, self.p_w, self.p_dst, y.data_ptr(), y.stride(0),
                                              tok_of_row.data_ptr(), expert_of_row.data_ptr(), w_rows.data_ptr(), self.send_base.data_ptr(),
                                              self.local_off.data_ptr(), self.rank, R, self.H, self.E, self.W, self.cap, st), "ix_ep_dispatch")
        self._handshake()                      # every source's rows for my experts have landed
        _native.check(self.lib.ix_ep_resolve_dst(self.dstbuf.data_ptr(), self.p_rows, self.own_offs.data_ptr(), self.e_loc, self.W,
                                                 self.H * 4, self.cap, st), "ix_ep_resolve_dst")
        xb = self.xbuf.view(self.cap, self.H)
        a = M.grouped_gemm(xb, gate_up, self.own_offs, M.EPI_GLU, w_rows=self.wbuf)
        M.grouped_gemm(a, down, self.own_offs, M.EPI_F32, row_dst=self.dstbuf)
        self._handshake()                      # every owner has written my rows back
        return self.rows[:R * self.H].view(R, self.H), pos


_registry: dict = {}


def register(group, rt: EPPeer) -> None:
    _registry[group] = rt


def get(group):
    return _registry.get(group)
