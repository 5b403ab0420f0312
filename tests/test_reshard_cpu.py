"""The resharding plan of the weight sync (sync/reshard.py): executing the planned pieces on plain tensors rebuilds
every engine shard exactly, for plain splits, sectioned gate|up / GDN projections, row-parallel (column-split) weights,
replicated KV heads, and an engine degree above the trainer's."""
import math

import pytest
import torch

from skyrl_isoexec_b200.models.config import get_config
from skyrl_isoexec_b200.models.decoder import ParamStore, build_param_specs
from skyrl_isoexec_b200.parallel.state import ParallelState
from skyrl_isoexec_b200.sync.reshard import bytes_moved, plan_pieces, shard_ranges


def _stores(cfg, tp):
    out = []
    for r in range(tp):
        ps = ParallelState(tp=tp, tp_rank=r, world_size=tp)
        st = ParamStore(build_param_specs(cfg, ps), torch.float32, "cpu")
        st.init_weights(3, r, tp)
        out.append(st)
    return out


@pytest.mark.parametrize("model,t_tp,e_tp", [("tiny-qwen3", 2, 1), ("tiny-qwen3", 4, 2), ("tiny-qwen3", 4, 1), ("tiny-qwen3", 1, 2),
                                             ("tiny-hybrid", 2, 1), ("tiny-moe", 2, 1)])
def test_planned_pieces_rebuild_every_engine_shard(model, t_tp, e_tp):
    cfg = get_config(model)
    T, E = _stores(cfg, t_tp), _stores(cfg, e_tp)
    for er in range(e_tp):
        for prefer in range(t_tp):
            pcs = plan_pieces(T[0].specs, E[er].specs, E[er].order, t_tp, e_tp, er, prefer_rank=prefer)
            dst = torch.full_like(E[er].flat, float("nan"))
            for p in pcs:
                for r in range(p.rows):
                    a, b = p.dst_off + r * p.dst_pitch, p.src_off + r * p.src_pitch
                    assert torch.isnan(dst[a:a + p.row_elems]).all()          # pieces never overlap in the destination
                    dst[a:a + p.row_elems] = T[p.src_rank].flat[b:b + p.row_elems]
            for name in E[er].order:
                s = E[er].specs[name]
                n = math.prod(s.shape)
                assert torch.equal(dst[s.offset:s.offset + n], E[er].flat[s.offset:s.offset + n]), (er, prefer, name)
            tot, far = bytes_moved(pcs, 2, prefer)
            assert tot == sum(math.prod(E[er].specs[n].shape) for n in E[er].order) * 2 and far <= tot


def test_shard_ranges_tile_the_full_dim():
    cfg = get_config("tiny-qwen3")
    for tp in (1, 2, 4):
        specs = {s.name: s for s in build_param_specs(cfg, ParallelState(tp=tp, tp_rank=0, world_size=tp))}
        for name, s in specs.items():
            if s.shard_dim is None:
                continue
            seen = []
            for r in range(tp):
                seen += shard_ranges(s, r, tp)
            covered = set()
            for lo, n in seen:
                covered |= set(range(lo, lo + n))
            assert covered == set(range(s.full_shape[s.shard_dim])), (name, tp)
