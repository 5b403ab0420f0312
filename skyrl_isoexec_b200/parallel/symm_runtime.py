"""Symmetric-memory runtime for the peer-memory collectives (csrc/peer_collectives.cu).

``SymmGroup`` owns, for one process group, a double-buffered staging area and a flag array in
symmetric memory (allocated and exchanged through ``torch.distributed._symmetric_memory``: CUDA VMM
allocations mapped into every rank of the group) and exposes:

  * ``tree_all_reduce(partial)``  one-shot all-reduce of an fp32 tensor in the fixed balanced-tree
                                  order over ranks (the TP reduction of row-parallel linears);
  * ``all_reduce_sum_(flat)``     two-shot (reduce-scatter + all-gather) in-place sum of a large
                                  fp32 buffer in fixed-size buckets (the DP gradient reduction);
  * ``push(descs)``               descriptor-driven copy/cast into peer memory (weight sync).

Every rank of the group must call the same methods in the same order (each call advances a
shared epoch counter). Waits inside the kernels are bounded; ``check()`` turns a timed-out wait
into a Python exception on the host instead of a hang on the device.
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _native
from . import symm


class PeerTimeout(RuntimeError):
    pass


def _rendezvous(t: torch.Tensor, group):
    import torch.distributed._symmetric_memory as sm

    name = group.group_name if group is not None else dist.group.WORLD.group_name
    return sm.rendezvous(t, group=name)


class SymmGroup:
    def __init__(self, group, staging_bytes: int = 256 << 20, device=None):
        import torch.distributed._symmetric_memory as sm

        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        assert self.world & (self.world - 1) == 0 and self.world <= 16, "peer collectives need a power-of-two group size <= 16"
        self.device = torch.device(device or f"cuda:{torch.cuda.current_device()}")
        self.half = staging_bytes // 4 // 4 * 4               # fp32 elements per staging half (multiple of 4)
        self.staging = sm.empty(2 * self.half, dtype=torch.float32, device=self.device)
        self.flags = sm.empty(64, dtype=torch.int32, device=self.device)
        self.staging.zero_()
        self.flags.zero_()
        torch.cuda.synchronize()
        self.h_staging = _rendezvous(self.staging, group)
        self.h_flags = _rendezvous(self.flags, group)
        dist.barrier(group=group)
        self.buf_ptrs = [int(p) for p in self.h_staging.buffer_ptrs]
        self.flag_ptrs = (C.c_longlong * self.world)(*[int(p) for p in self.h_flags.buffer_ptrs])
        self.epoch = 0
        self.calls = 0
        self.lib = _native.lib()
        self.lib.ix_peer_tree_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_uint, C.c_longlong, C.c_longlong,
                                                 C.c_void_p, C.c_longlong, C.c_int, C.c_void_p]
        self.lib.ix_peer_gather_slices.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_uint, C.c_longlong, C.c_longlong,
                                                   C.c_void_p, C.c_void_p]
        self.lib.ix_peer_handshake.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_uint, C.c_void_p]
        self.lib.ix_push_copy.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        symm.register(group, self)

    # ------------------------------------------------------------------ helpers
    def _half_ptrs(self, parity: int):
        off = parity * self.half * 4
        return (C.c_longlong * self.world)(*[p + off for p in self.buf_ptrs])

    def _my_half(self, parity: int) -> torch.Tensor:
        return self.staging[parity * self.half:(parity + 1) * self.half]

    def check(self) -> None:
        st = _native.read_status()
        if st != 0:
            raise PeerTimeout(f"a peer-memory wait ran out (kernel status {st}): a rank of the group did not arrive")

    # ------------------------------------------------------------------ collectives
    def tree_all_reduce(self, partial: torch.Tensor, out_dtype=None) -> torch.Tensor:
        """All ranks pass their fp32 partial [.., N]; all get the tree-ordered sum (fp32 or ``out_dtype``=bf16)."""
        assert partial.dtype == torch.float32
        n = partial.numel()
        n4 = (n + 3) // 4 * 4
        if n4 > self.half:
            raise ValueError(f"tree_all_reduce of {n} elements exceeds the staging half ({self.half})")
        parity = self.calls & 1
        self.calls += 1
        self.epoch += 1
        stage = self._my_half(parity)
        stage[:n].copy_(partial.reshape(-1))
        out_bf16 = out_dtype == torch.bfloat16
        out = torch.empty(n4, dtype=torch.bfloat16 if out_bf16 else torch.float32, device=partial.device)
        _native.check(self.lib.ix_peer_tree_reduce(self._half_ptrs(parity), self.flag_ptrs, self.rank, self.world, self.epoch, 0, n4,
                                                   out.data_ptr(), 0, int(out_bf16), _native.stream()), "ix_peer_tree_reduce")
        return out[:n].view(partial.shape)

    def all_reduce_sum_(self, flat: torch.Tensor) -> torch.Tensor:
        """In-place sum of a flat fp32 buffer over the group, bucket by bucket (two-shot per bucket)."""
        assert flat.dtype == torch.float32 and flat.dim() == 1
        W = self.world
        unit = 4 * W
        n = flat.numel()
        bucket = self.half // unit * unit
        for lo in range(0, n, bucket):
            m = min(bucket, n - lo)
            m_pad = (m + unit - 1) // unit * unit
            parity = self.calls & 1
            self.calls += 1
            stage = self._my_half(parity)
            stage[:m].copy_(flat[lo:lo + m])
            if m_pad > m:
                stage[m:m_pad].zero_()
            slice_n = m_pad // W
            ptrs = self._half_ptrs(parity)
            self.epoch += 1
            _native.check(self.lib.ix_peer_tree_reduce(ptrs, self.flag_ptrs, self.rank, W, self.epoch, self.rank * slice_n,
                                                       (self.rank + 1) * slice_n, stage.data_ptr(), self.rank * slice_n, 0,
                                                       _native.stream()), "ix_peer_tree_reduce")
            self.epoch += 1
            if m_pad == m:
                _native.check(self.lib.ix_peer_gather_slices(ptrs, self.flag_ptrs, self.rank, W, self.epoch, slice_n, m_pad,
                                                             flat[lo:lo + m].data_ptr(), _native.stream()), "ix_peer_gather_slices")
            else:
                tmp = torch.empty(m_pad, dtype=torch.float32, device=flat.device)
                _native.check(self.lib.ix_peer_gather_slices(ptrs, self.flag_ptrs, self.rank, W, self.epoch, slice_n, m_pad,
                                                             tmp.data_ptr(), _native.stream()), "ix_peer_gather_slices")
                flat[lo:lo + m].copy_(tmp[:m])
        return flat

    def barrier(self) -> None:
        self.epoch += 1
        _native.check(self.lib.ix_peer_handshake(self.flag_ptrs, self.rank, self.world, self.epoch, _native.stream()), "ix_peer_handshake")

    def peer_view(self, rank: int, numel: int, dtype, offset_bytes: int = 0) -> int:
        """Device address, in this process, of ``rank``'s staging buffer (+offset)."""
        return self.buf_ptrs[rank] + offset_bytes
