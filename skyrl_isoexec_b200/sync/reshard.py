"""Weight delivery between DIFFERENT layouts: a trainer at tensor-parallel degree Tt feeds colocated rollout engines at
degree Te (reference: ISO/sync/native_weight_sync.py:64-125,237-298, which gathers every sharded tensor to full shape
on the trainer and lets the engine slice it; B/weight_sync/cuda_ipc_strategy.py:242-264 for the transfer).

Here the layout change is planned once and executed as rectangular copies:

  * ``shard_ranges``   the intervals of the FULL tensor (along the shard dim) that a rank's local shard consists of, in
                       local order: per-section slices of gate|up style weights, per-KV-group slices when KV heads are
                       replicated, the whole dim for replicated parameters;
  * ``plan_pieces``    for one engine rank: every engine interval is cut against the trainer ranks' intervals, which
                       gives pieces ``(trainer tp rank, source offset, destination offset, rows, row width, pitches)``;
  * ``PeerPullResharder``  GPUs: the trainer's flat buffer lives in symmetric memory; ONE kernel launch
                       (csrc/reshard.cu) reads each piece from its owner over NVLink (or locally) and stores it into
                       the engine's flat buffer, so only the engine shard's own bytes move;
  * ``CollectiveResharder``  CPU / no peer access: all-gather of the trainer group's flat buffers in buckets, then the
                       same pieces are copied out of the gathered buckets (gloo or NCCL).

Both executors run the same plan, so the CPU tests of the plan cover the GPU path's index arithmetic.
Engines must nest inside trainer tensor-parallel groups (Tt a multiple of Te) or be the trainer's own size; expert-
and pipeline-parallel layouts must agree on both sides.
"""

from __future__ import annotations

import ctypes as C
import math
import struct
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Piece:
    name: str
    src_rank: int        # trainer tensor-parallel rank that owns the source
    src_off: int         # element offset inside the trainer's flat buffer
    dst_off: int         # element offset inside the engine's flat buffer
    rows: int
    row_elems: int
    src_pitch: int       # elements between rows
    dst_pitch: int


def shard_ranges(spec, tp_rank: int, tp: int) -> list[tuple[int, int]]:
    """[(first index in the full tensor, count)] along ``spec.shard_dim`` that make up the local shard, in local order."""
    if spec.shard_dim is None or tp == 1:
        d = spec.shard_dim if spec.shard_dim is not None else 0
        return [(0, spec.full_shape[d] if spec.full_shape else 1)]
    if spec.kv_rep > 1:
        Hkv, G, qs, D = spec.kv_layout
        rep = spec.kv_rep
        g, j, gl = tp_rank // rep, tp_rank % rep, G // rep
        base = g * (G * qs + 2 * D)
        return [(base + j * gl * qs, gl * qs), (base + G * qs, 2 * D)]
    full = spec.full_shape[spec.shard_dim]
    secs = spec.sections or (full,)
    out, lo = [], 0
    for sz in secs:
        out.append((lo + tp_rank * (sz // tp), sz // tp))
        lo += sz
    return out


def _dims(spec, local_shape):
    d = spec.shard_dim if spec.shard_dim is not None else 0
    outer = math.prod(local_shape[:d])
    inner = math.prod(local_shape[d + 1:])
    return d, outer, inner


def plan_pieces(trainer_specs: dict, engine_specs: dict, order: list[str], t_tp: int, e_tp: int, e_tp_rank: int,
                prefer_rank: int = 0) -> list[Piece]:
    """Pieces that build engine rank ``e_tp_rank``'s shard of every parameter out of the trainer ranks' shards.
    ``prefer_rank``: the trainer tensor-parallel rank living on the same GPU; replicated data is taken from it."""
    pieces: list[Piece] = []
    cand = [prefer_rank] + [r for r in range(t_tp) if r != prefer_rank]
    for name in order:
        es, ts = engine_specs[name], trainer_specs[name]
        if tuple(es.full_shape) != tuple(ts.full_shape):
            raise ValueError(f"{name}: full shape {tuple(ts.full_shape)} on the trainer, {tuple(es.full_shape)} on the engine")
        if not es.full_shape or math.prod(es.full_shape) == 0:
            continue
        if es.ep_sharded and tuple(es.shape[:1]) != tuple(ts.shape[:1]):
            raise ValueError(f"{name}: expert-parallel layouts differ between trainer and engine; resharding covers tensor parallelism")
        d, outer, inner = _dims(es, es.shape)
        if es.shard_dim is None and ts.shard_dim is not None or (es.shard_dim is not None and ts.shard_dim is not None and es.shard_dim != ts.shard_dim):
            raise ValueError(f"{name}: shard dim differs between trainer ({ts.shard_dim}) and engine ({es.shard_dim})")
        e_local_dim = es.shape[d] if es.shape else 1
        t_local_dim = ts.shape[d] if ts.shape else 1
        if es.shard_dim is None:
            # replicated on both sides: one copy from the colocated trainer rank
            n = math.prod(es.shape)
            pieces.append(Piece(name, prefer_rank, ts.offset, es.offset, 1, n, n, n))
            continue
        src_ranges = {r: shard_ranges(ts, r, t_tp) for r in range(t_tp)}
        dst_local = 0
        for lo, n in shard_ranges(es, e_tp_rank, e_tp):
            todo = [(lo, lo + n)]
            for r in cand:
                if not todo:
                    break
                s_local = 0
                for slo, sn in src_ranges[r]:
                    nxt = []
                    for a, b in todo:
                        x, y = max(a, slo), min(b, slo + sn)
                        if x >= y:
                            nxt.append((a, b))
                            continue
                        pieces.append(Piece(name, r,
                                            ts.offset + (s_local + x - slo) * inner,
                                            es.offset + (dst_local + x - lo) * inner,
                                            outer, (y - x) * inner, t_local_dim * inner, e_local_dim * inner))
                        if a < x:
                            nxt.append((a, x))
                        if y < b:
                            nxt.append((y, b))
                    todo = nxt
                    s_local += sn
            if todo:
                raise ValueError(f"{name}: engine rows {todo} are held by no trainer rank")
            dst_local += n
    return pieces


def bytes_moved(pieces: list[Piece], elem_size: int, my_rank: int) -> tuple[int, int]:
    """(bytes copied in total, bytes that come from another rank)."""
    tot = sum(p.rows * p.row_elems for p in pieces) * elem_size
    far = sum(p.rows * p.row_elems for p in pieces if p.src_rank != my_rank) * elem_size
    return tot, far


class _Base:
    def __init__(self, trainer_model, engine_model, group, t_rank: int):
        self.t, self.e = trainer_model, engine_model
        self.group = group
        self.t_tp = trainer_model.ps.tp
        self.t_rank = t_rank
        if trainer_model.ps.ep != engine_model.ps.ep or trainer_model.ps.pp != 1 or engine_model.ps.pp != 1:
            raise ValueError("resharding weight sync needs equal expert parallelism and no pipeline parallelism on both sides")
        if self.t.store.flat.dtype != self.e.store.flat.dtype:
            raise ValueError("trainer and engine parameter dtypes differ")
        self.pieces = plan_pieces(self.t.store.specs, self.e.store.specs, self.e.store.order, self.t_tp,
                                  engine_model.ps.tp, engine_model.ps.tp_rank, prefer_rank=t_rank)
        self.total_bytes, self.remote_bytes = bytes_moved(self.pieces, self.e.store.flat.element_size(), t_rank)

    def _barrier(self):
        if self.group is not None and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.barrier(group=self.group)


class CollectiveResharder(_Base):
    """All-gather of the trainer group's flat buffers (bucketed), pieces copied out of the gathered buckets."""

    def __init__(self, trainer_model, engine_model, group, t_rank: int, bucket_elems: int = 64 << 20):
        super().__init__(trainer_model, engine_model, group, t_rank)
        self.bucket = bucket_elems
        n = self.t.store.numel
        if self.t_tp > 1:
            dev = self.t.store.flat.device
            mine = torch.tensor([n], dtype=torch.int64, device=dev)
            got = [torch.zeros_like(mine) for _ in range(self.t_tp)]
            dist.all_gather(got, mine, group=group)
            if any(int(g) != n for g in got):
                raise ValueError("trainer ranks have flat buffers of different sizes; the bucketed gather needs equal sizes")

    @torch.no_grad()
    def sync(self) -> int:
        src, dst = self.t.store.flat.detach(), self.e.store.flat.detach()
        n = src.numel()
        for lo in range(0, n, self.bucket):
            hi = min(n, lo + self.bucket)
            if self.t_tp > 1:
                parts = [torch.empty(hi - lo, dtype=src.dtype, device=src.device) for _ in range(self.t_tp)]
                dist.all_gather(parts, src[lo:hi].contiguous(), group=self.group)
            else:
                parts = [src[lo:hi]]
            for p in self.pieces:
                # a piece may straddle buckets: copy the part of every row that falls into this one
                for r in range(p.rows):
                    a = p.src_off + r * p.src_pitch
                    x, y = max(a, lo), min(a + p.row_elems, hi)
                    if x < y:
                        d0 = p.dst_off + r * p.dst_pitch + (x - a)
                        dst[d0:d0 + (y - x)].copy_(parts[p.src_rank][x - lo:y - lo])
        self._barrier()
        return self.total_bytes


class PeerPullResharder(_Base):
    """One kernel launch per sync: every piece is read from its owner's symmetric-memory flat buffer."""

    def __init__(self, trainer_model, engine_model, group, t_rank: int, peer_ptrs: list[int]):
        """``peer_ptrs[r]``: address, in this process, of trainer tensor-parallel rank r's flat buffer."""
        super().__init__(trainer_model, engine_model, group, t_rank)
        from ..ops import _native

        self.lib = _native.lib()
        self.lib.ix_reshard_pull.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        self.lib.ix_reshard_desc_bytes.restype = C.c_int
        self.lib.ix_reshard_pull.restype = C.c_int
        fmt = "<QQqqqqii"
        assert self.lib.ix_reshard_desc_bytes() == struct.calcsize(fmt), "descriptor layout differs between host and kernel"
        es = self.e.store.flat.element_size()
        dst0 = self.e.store.flat.data_ptr()
        recs = [struct.pack(fmt, peer_ptrs[p.src_rank] + p.src_off * es, dst0 + p.dst_off * es, p.rows, p.row_elems * es,
                            p.src_pitch * es, p.dst_pitch * es, 0, 0) for p in self.pieces]
        self.n_desc = len(recs)
        self.descs = torch.frombuffer(bytearray(b"".join(recs)), dtype=torch.uint8).to(self.e.store.flat.device)

    @torch.no_grad()
    def sync(self) -> int:
        from ..ops import _native

        torch.cuda.current_stream().synchronize()      # this rank's update has landed ...
        self._barrier()                                # ... and so has everyone else's
        _native.check(self.lib.ix_reshard_pull(self.descs.data_ptr(), self.n_desc, _native.stream()), "ix_reshard_pull")
        torch.cuda.current_stream().synchronize()
        self._barrier()                                # nobody's weights change while a peer still reads them
        return self.total_bytes


def symmetric_flat_allocator(group):
    """Allocator for ``ParamStore``: the flat buffer comes from symmetric memory of ``group`` so that the other ranks of
    the group can read it. Returns (alloc(numel, dtype, device) -> tensor, rendezvous(tensor) -> [peer addresses])."""
    import torch.distributed._symmetric_memory as sm

    name = group.group_name if group is not None else dist.group.WORLD.group_name

    def alloc(numel, dtype, device):
        t = sm.empty(numel, dtype=dtype, device=device)
        t.zero_()
        return t

    def rendezvous(t):
        h = sm.rendezvous(t, group=name)
        dist.barrier(group=group)
        return [int(p) for p in h.buffer_ptrs], h

    return alloc, rendezvous


class PipelineStageSync:
    """Trainer with pipeline parallelism, engines without: every pipeline stage holds the parameters of its own layers,
    every engine needs all of them. Stage by stage, the owning rank broadcasts its flat buffer inside the pipeline
    group and every rank copies that stage's parameters into its engine model (same tensor-parallel layout on both
    sides, so each parameter is one contiguous copy). Reference: the Megatron backend gathers across pipeline ranks
    when it exports weights for the engines, B/workers/megatron/megatron_worker.py:569-571."""

    def __init__(self, trainer_model, engine_model, ps):
        from ..models.decoder import ParamStore, build_param_specs
        from ..parallel.pp import stage_layers
        import copy

        self.t, self.e, self.ps = trainer_model, engine_model, ps
        if engine_model.ps.tp != ps.tp or engine_model.ps.ep != ps.ep:
            raise ValueError("with a pipelined trainer the engines use the trainer's tensor- and expert-parallel degrees")
        cfg = trainer_model.cfg
        self.stages = []          # per stage: (numel of its flat buffer, [(name, offset, numel)])
        for s in range(ps.pp):
            ps_s = copy.copy(ps)
            ps_s.pp_rank = s
            specs = build_param_specs(cfg, ps_s, stage_layers(cfg.num_layers, ps.pp, s))
            off, items = 0, []
            for sp in specs:
                n = math.prod(sp.shape)
                items.append((sp.name, off, n))
                off += (n + ParamStore.ALIGN - 1) // ParamStore.ALIGN * ParamStore.ALIGN
            self.stages.append((off, items))
        assert self.stages[ps.pp_rank][0] == trainer_model.store.numel, "stage layout differs from the live parameter store"
        self.total_bytes = sum(n for n, _ in self.stages) * trainer_model.store.flat.element_size()
        self.remote_bytes = self.total_bytes - self.stages[ps.pp_rank][0] * trainer_model.store.flat.element_size()

    @torch.no_grad()
    def sync(self) -> int:
        ps = self.ps
        mine = self.t.store.flat.detach()
        done = set()
        for s, (numel, items) in enumerate(self.stages):
            buf = mine if s == ps.pp_rank else torch.empty(numel, dtype=mine.dtype, device=mine.device)
            dist.broadcast(buf, src=ps.pp_ranks[s], group=ps.pp_group)
            for name, off, n in items:
                if name in done or name not in self.e.store.views:      # a tied embedding lives on two stages: first wins
                    continue
                dst = self.e.store.views[name]
                dst.copy_(buf[off:off + n].view(dst.shape))
                done.add(name)
        missing = [n for n in self.e.store.order if n not in done]
        if missing:
            raise KeyError(f"no pipeline stage delivered {missing[:4]}")
        return self.total_bytes
