"""Weight sync by GPU peer-memory push (the reference's CUDA-IPC strategy, B/weight_sync/cuda_ipc_strategy.py:242-354,
plus the layout/cast repack that the reference does on the host side of the transfer).

The engine rank exports a CUDA IPC handle of its flat parameter buffer; the trainer rank maps it and, at every sync,
launches ONE descriptor-driven kernel (csrc/peer_collectives.cu ``push_copy_kernel``) that reads its own parameters
(bf16, or the fp32 master copy, rounded on the way) and stores them straight into the engine's buffer over NVLink.
No staging bucket, no NCCL, no host copy. Both models must have the same parameter layout (same TP/EP degrees and
storage order); a different engine TP goes through the ``broadcast`` strategy, which reshards.

Handshake: the init message carries the trainer's contract hash; ``PeerPushReceiver`` refuses a different one. The
transfer is ordered by a host-side barrier on the pair's process group after the sender's stream has drained, so the
engine never computes with half-written weights.
"""

from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..core import process as P
from ..ops import _native


_OPENED: dict = {}     # IPC handle bytes -> base address of the mapping in this process


@dataclass
class PeerPushInitInfo:
    contract_hash: str | None
    numel: int
    dtype: str
    ipc_handle: tuple | None = None      # what ``UntypedStorage._share_cuda_()`` returned on the engine rank

    def strategy_type(self) -> str:
        return "peer"


def export_engine_buffer(model, contract_hash: str | None = None) -> PeerPushInitInfo:
    """Engine side: describe the flat parameter buffer so that a trainer process on the same node can map it."""
    flat = model.store.flat
    assert flat.is_cuda, "peer push needs the engine's parameters on a GPU"
    handle = flat.untyped_storage()._share_cuda_()
    return PeerPushInitInfo(contract_hash if contract_hash is not None else P.contract_hash_or_none(), flat.numel(),
                            str(flat.dtype).replace("torch.", ""), handle)


class PeerPushSender:
    def __init__(self, info: PeerPushInitInfo, model, from_master: torch.Tensor | None = None):
        """``from_master``: the optimizer's fp32 master buffer; if given, the push rounds fp32 -> bf16 in flight
        instead of reading the trainer's bf16 copy."""
        self.model, self.info = model, info
        mine = model.store.flat
        if info.numel != mine.numel() or info.dtype != str(mine.dtype).replace("torch.", ""):
            raise ValueError(f"engine buffer ({info.numel} x {info.dtype}) does not match the trainer's layout "
                             f"({mine.numel()} x {mine.dtype}); use the broadcast strategy to reshard")
        # The handle is opened HERE, natively, with the trainer's device current and lazy peer access: a mapping made
        # in the context of the device that owns the memory (what torch's own importer does) cannot be dereferenced by
        # kernels of another device. A handle can be opened once per process, so mappings are cached.
        lib = _native.lib()
        owner_device, handle, _size_bytes, offset_bytes = info.ipc_handle[:4]
        key = bytes(handle)
        if key not in _OPENED:
            base = C.c_void_p()
            with torch.cuda.device(mine.device):
                if owner_device != mine.device.index:
                    _native.check(lib.ix_enable_peer_access(int(owner_device)), "ix_enable_peer_access")
                _native.check(lib.ix_ipc_open(C.c_char_p(key), C.byref(base)), "ix_ipc_open")
            _OPENED[key] = base.value
        self.remote_ptr = _OPENED[key] + int(offset_bytes)
        where = lib.ix_pointer_device(C.c_void_p(self.remote_ptr))
        if where != int(owner_device):
            raise RuntimeError(f"the engine's buffer is not a device allocation on GPU {owner_device} (got {where})")
        self.src = from_master if from_master is not None else mine
        self.src_f32 = self.src.dtype == torch.float32
        if self.src_f32 and mine.dtype != torch.bfloat16:
            raise ValueError("the casting push writes bf16")
        # one descriptor per parameter (16-byte aligned by construction of the flat layout)
        recs = []
        esz_src = 4 if self.src_f32 else mine.element_size()
        for name in model.store.order:
            s = model.store.specs[name]
            n = 1
            for d in s.shape:
                n *= d
            n_al = (n + 7) // 8 * 8
            recs.append(struct.pack("<QQqii", self.src.data_ptr() + s.offset * esz_src, self.remote_ptr + s.offset * mine.element_size(),
                                    n_al, int(self.src_f32), 0))
        self.n_desc = len(recs)
        self.descs = torch.frombuffer(bytearray(b"".join(recs)), dtype=torch.uint8).to(mine.device)
        lib = _native.lib()
        lib.ix_push_copy.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        self.lib = lib

    def send(self, group=None) -> int:
        """Push every parameter; returns the bytes written to the peer."""
        _native.check(self.lib.ix_push_copy(self.descs.data_ptr(), self.n_desc, _native.stream()), "ix_push_copy")
        torch.cuda.current_stream().synchronize()
        if group is not None or dist.is_initialized():
            dist.barrier(group=group)
        return self.info.numel * self.model.store.flat.element_size()


class PeerPushReceiver:
    def __init__(self, info: PeerPushInitInfo, model):
        mine = P.contract_hash_or_none()
        if info.contract_hash is not None and mine is not None and info.contract_hash != mine:
            raise RuntimeError(f"weight sync refused: trainer contract {info.contract_hash} != engine contract {mine}")
        self.model = model

    def receive(self, group=None) -> None:
        """Wait until the sender's push has landed (its stream drained before the barrier)."""
        dist.barrier(group=group)
        torch.cuda.current_stream().synchronize()
