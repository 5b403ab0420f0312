"""Trainer -> rollout weight synchronisation.

Data structures and the strategy protocol follow the reference (B/weight_sync/base.py:10-106,
transfer_strategy.py:26-186): ``WeightChunk``, ``WeightUpdateRequest``, an init-info object that
carries the trainer's **contract hash**, and ``create_sender`` / ``create_receiver``; the receiver
refuses to be built if the hash differs from its own (B/weight_sync/cuda_ipc_strategy.py:537-547).

Weights travel in the model's native layout (no HF renaming, like ISO/sync/native_weight_sync.py):
the unit is the flat parameter buffer. Strategies:
  * ``shared``     trainer and engine live in one process with the same TP layout and alias one
                   flat buffer: the sync is the handshake, the state invalidation and an epoch bump;
  * ``broadcast``  packed buckets over a ``torch.distributed`` group (NCCL on GPUs, gloo on CPU);
                   when the engine's TP differs, each bucket is resharded on the fly;
  * ``peer``       GPU peer-memory push (``sync/peer_push.py``): one kernel casts/repacks a trainer
                   shard straight into every engine rank's flat buffer over NVLink.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Iterator

import torch
import torch.distributed as dist

from ..core import process as P
from ..models.decoder import DecoderLM, shard_of


# ------------------------------------------------------------------------------------ data
@dataclass
class WeightChunk:
    names: list[str]
    dtypes: list[str]
    shapes: list[list[int]]
    tensors: list[torch.Tensor]

    def __post_init__(self):
        n = len(self.names)
        if not (len(self.dtypes) == len(self.shapes) == len(self.tensors) == n):
            raise ValueError("WeightChunk fields must have equal lengths")

    @property
    def total_numel(self) -> int:
        return sum(t.numel() for t in self.tensors)

    @property
    def total_size_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors)


@dataclass
class WeightUpdateRequest:
    names: list[str]
    dtypes: list[str]
    shapes: list[list[int]]

    def to_json_dict(self) -> dict:
        return {"names": self.names, "dtypes": self.dtypes, "shapes": self.shapes}

    @staticmethod
    def from_json_dict(d: dict) -> "WeightUpdateRequest":
        return WeightUpdateRequest(list(d["names"]), list(d["dtypes"]), [list(s) for s in d["shapes"]])


@dataclass
class LoraLoadRequest:
    lora_path: str
    lora_name: str = "default"


@dataclass
class WeightSyncInitInfo:
    contract_hash: str | None = None
    override_existing_receiver: bool = False
    engine_tp: int = 1

    def strategy_type(self) -> str:
        raise NotImplementedError

    def for_engine(self, engine_index: int, tp: int, pp: int, dp: int) -> "WeightSyncInitInfo":
        return self


@dataclass
class SharedInitInfo(WeightSyncInitInfo):
    def strategy_type(self) -> str:
        return "shared"


@dataclass
class ReshardInitInfo(WeightSyncInitInfo):
    """Colocated engines at another tensor-parallel degree than the trainer (``sync/reshard.py``)."""
    trainer_tp: int = 1

    def strategy_type(self) -> str:
        return "reshard"


@dataclass
class BroadcastInitInfo(WeightSyncInitInfo):
    group_ranks: list[int] = field(default_factory=list)   # global ranks: [trainer src] + engine ranks
    src_rank: int = 0
    bucket_bytes: int = 1 << 30

    def strategy_type(self) -> str:
        return "broadcast"


# ------------------------------------------------------------------------------------ extraction / loading
def extract_native_weights(model: DecoderLM, engine_tp: int | None = None, bucket_bytes: int = 1 << 30) -> Iterator[WeightChunk]:
    """Yield buckets of (name, local tensor) in storage order. If the engine runs another TP degree,
    sharded tensors are first gathered to full shape over the trainer's TP group (every trainer TP
    rank must iterate in lock step) and the engine slices what it needs on arrival."""
    ps = model.ps
    reshard = engine_tp is not None and engine_tp != ps.tp
    names, dtypes, shapes, tensors, size = [], [], [], [], 0
    for name, t in model.named_weights():
        spec = model.store.specs[name]
        if reshard and spec.shard_dim is not None and ps.tp > 1:
            t = gather_full(t, spec, ps)
        names.append(name)
        dtypes.append(str(t.dtype).replace("torch.", ""))
        shapes.append(list(t.shape))
        tensors.append(t)
        size += t.numel() * t.element_size()
        if size >= bucket_bytes:
            yield WeightChunk(names, dtypes, shapes, tensors)
            names, dtypes, shapes, tensors, size = [], [], [], [], 0
    if names:
        yield WeightChunk(names, dtypes, shapes, tensors)


def gather_full(t: torch.Tensor, spec, ps) -> torch.Tensor:
    """All-gather a TP-sharded tensor to its full shape, undoing the per-section split."""
    parts = [torch.empty_like(t) for _ in range(ps.tp)]
    dist.all_gather(parts, t.contiguous(), group=ps.tp_group)
    if getattr(spec, "kv_rep", 1) > 1:
        from ..models.decoder import unshard_kv_rep

        return unshard_kv_rep(parts, spec)
    if not spec.sections:
        return torch.cat(parts, dim=spec.shard_dim)
    secs = [s // ps.tp for s in spec.sections]
    cols = []
    for si, sz in enumerate(secs):
        lo = sum(secs[:si])
        cols += [p.narrow(spec.shard_dim, lo, sz) for p in parts]
    return torch.cat(cols, dim=spec.shard_dim)


def load_weights(model: DecoderLM, named: Iterator[tuple[str, torch.Tensor]]) -> int:
    """In-place load into the model's flat buffer; full-shape tensors are sliced to the local shard."""
    n = 0
    ps = model.ps
    with torch.no_grad():
        for name, t in named:
            if name not in model.store.views:
                raise KeyError(f"weight sync delivered unknown parameter {name!r}")
            dst = model.store.views[name]
            spec = model.store.specs[name]
            if tuple(t.shape) != tuple(dst.shape):
                if tuple(t.shape) == tuple(spec.full_shape):
                    t = shard_of(t, spec, ps.tp_rank, ps.tp, ps.ep_rank, ps.ep)
                else:
                    raise ValueError(f"{name}: got shape {tuple(t.shape)}, want {tuple(dst.shape)} or {spec.full_shape}")
            dst.copy_(t.to(dst.dtype))
            n += 1
    return n


# ------------------------------------------------------------------------------------ shared (same process)
class SharedSender:
    def __init__(self, init_info, model):
        self.model = model

    def send_chunks(self, chunks, weight_metadata=None) -> WeightUpdateRequest:
        names, dtypes, shapes = [], [], []
        for c in chunks:
            names += c.names
            dtypes += c.dtypes
            shapes += c.shapes
        return WeightUpdateRequest(names, dtypes, shapes)


class SharedReceiver:
    """Engine model aliases the trainer's flat buffer; receiving checks that this is still true."""

    def __init__(self, init_info, model):
        P.assert_init_info_contract(init_info)
        self.model = model

    def receive_weights(self, request: WeightUpdateRequest) -> Iterator[tuple[str, torch.Tensor]]:
        for name in request.names:
            yield name, self.model.store.views[name]


# ------------------------------------------------------------------------------------ broadcast
_groups: dict[tuple, object] = {}


def _group_for(ranks: list[int]):
    key = tuple(ranks)
    if key not in _groups:
        world = list(range(dist.get_world_size()))
        _groups[key] = None if list(ranks) == world else dist.new_group(list(ranks))
    return _groups[key]


class BroadcastSender:
    def __init__(self, init_info: BroadcastInitInfo, model):
        self.info = init_info
        self.group = _group_for(init_info.group_ranks)
        self.device = model.device_

    def send_chunks(self, chunks, weight_metadata=None) -> WeightUpdateRequest:
        names, dtypes, shapes = [], [], []
        for c in chunks:
            meta = [{"names": c.names, "dtypes": c.dtypes, "shapes": c.shapes}]
            dist.broadcast_object_list(meta, src=self.info.src_rank, group=self.group)
            packed = torch.cat([t.reshape(-1) for t in c.tensors]) if len(c.tensors) > 1 else c.tensors[0].reshape(-1).contiguous()
            dist.broadcast(packed, src=self.info.src_rank, group=self.group)
            names += c.names
            dtypes += c.dtypes
            shapes += c.shapes
        dist.broadcast_object_list([None], src=self.info.src_rank, group=self.group)
        return WeightUpdateRequest(names, dtypes, shapes)


class BroadcastReceiver:
    def __init__(self, init_info: BroadcastInitInfo, model):
        P.assert_init_info_contract(init_info)
        self.info = init_info
        self.group = _group_for(init_info.group_ranks)
        self.device = model.device_

    def receive_weights(self, request: WeightUpdateRequest | None = None) -> Iterator[tuple[str, torch.Tensor]]:
        while True:
            meta = [None]
            dist.broadcast_object_list(meta, src=self.info.src_rank, group=self.group)
            if meta[0] is None:
                return
            m = meta[0]
            dts = [getattr(torch, d) for d in m["dtypes"]]
            numels = [math.prod(s) for s in m["shapes"]]
            packed = torch.empty(sum(numels), dtype=dts[0], device=self.device)
            dist.broadcast(packed, src=self.info.src_rank, group=self.group)
            off = 0
            for name, shape, n in zip(m["names"], m["shapes"], numels):
                yield name, packed[off:off + n].view(shape)
                off += n


# ------------------------------------------------------------------------------------ factory
def create_init_info(strategy: str, **kw) -> WeightSyncInitInfo:
    """``peer`` (CUDA-IPC push) is built on the ENGINE rank from its model: ``create_init_info("peer", model=m)``."""
    if strategy == "peer":
        from .peer_push import export_engine_buffer

        return export_engine_buffer(kw["model"], kw.get("contract_hash"))
    if "contract_hash" not in kw:
        kw["contract_hash"] = P.contract_hash()
    if strategy == "shared":
        return SharedInitInfo(**kw)
    if strategy in ("broadcast", "nccl", "gloo"):
        return BroadcastInitInfo(**kw)
    raise ValueError(f"unknown weight sync strategy {strategy!r}")


def _peer_classes():
    from .peer_push import PeerPushReceiver, PeerPushSender

    return PeerPushSender, PeerPushReceiver


def create_sender(init_info: WeightSyncInitInfo, model, **kw):
    kind = init_info.strategy_type()
    if kind == "peer":
        return _peer_classes()[0](init_info, model, **kw)
    return {"shared": SharedSender, "broadcast": BroadcastSender}[kind](init_info, model)


def create_receiver(init_info: WeightSyncInitInfo, model):
    kind = init_info.strategy_type()
    if kind == "peer":
        return _peer_classes()[1](init_info, model)
    return {"shared": SharedReceiver, "broadcast": BroadcastReceiver}[kind](init_info, model)
