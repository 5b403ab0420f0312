"""Checkpoints in ``torch.distributed.checkpoint`` (DCP) format: a directory (``.metadata`` + ``__{rank}_0.distcp``) that
torch's own tools read, e.g. ``python -m torch.distributed.checkpoint.format_utils dcp_to_torch <dir> <file.pt>`` or
``dcp.load`` from a job of any size (the reference's trainers write DCP through Megatron dist-checkpointing and FSDP,
R/train/trainer.py:1858-2036; docs/content/docs/checkpointing-logging/checkpointing.mdx:36-85).

Layout of the saved state dict:

    model.<native parameter name>        every parameter at its FULL logical shape, in the model's dtype
    optimizer.master.<name>              fp32 master weight           \\
    optimizer.exp_avg.<name>             Adam first moment             > full shape, when the optimizer is included
    optimizer.exp_avg_sq.<name>          Adam second moment           /
    meta.step / meta.global_step         scalars (as 0-d tensors)

Full shapes make the checkpoint independent of the layout that wrote it: tensor-parallel and expert-parallel shards are
gathered on save (collectives over those groups; every rank of them calls ``save_dcp``), the slices of an optimizer
sharded over data parallelism are gathered over the data-parallel group, and ``load_dcp`` cuts what the loading rank
owns. One rank per distinct set of parameters writes (the first rank of every pipeline stage), the others contribute
nothing. Pipeline stages write disjoint keys into the same directory.
"""

from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist


def _dcp():
    import torch.distributed.checkpoint as dcp

    return dcp


def _full_optimizer(policy, ps) -> dict | None:
    """{kind: flat fp32 tensor over ALL of this rank's parameters}: the local state, or the data-parallel slices joined."""
    opt = getattr(policy, "opt", None)
    if opt is None:
        return None
    sd = opt.state_dict()
    lo, hi, n = sd.get("slice", (0, opt.n, opt.n))
    out = {}
    for kind in ("master", "exp_avg", "exp_avg_sq"):
        t = sd[kind].detach()
        if hi - lo != n:
            # every rank of the shard group holds one contiguous slice (equal sizes but the last): pad, gather, trim
            _idx, cnt, grp = opt.shard
            per = max(b - a for a, b in opt.slices)
            pad = torch.zeros(per, dtype=t.dtype, device=t.device)
            pad[:t.numel()] = t
            parts = [torch.empty_like(pad) for _ in range(cnt)]
            dist.all_gather(parts, pad, group=grp)
            t = torch.cat(parts)[:n]
        out[kind] = t
    return out


def _gather_like_weight(flat_local: torch.Tensor, spec, model):
    """A per-parameter view of a flat fp32 state tensor, brought to the parameter's full shape like the weight itself."""
    from ..sync.strategies import gather_full

    ps = model.ps
    t = flat_local[spec.offset:spec.offset + math.prod(spec.shape)].view(spec.shape)
    if ps.tp > 1 and spec.shard_dim is not None:
        t = gather_full(t, spec, ps)
    if ps.ep > 1 and spec.ep_sharded:
        parts = [torch.empty_like(t) for _ in range(ps.ep)]
        dist.all_gather(parts, t.contiguous(), group=ps.ep_group)
        t = torch.cat(parts, dim=0)
    return t


def save_dcp(policy_or_model, path: str, ps, step: int = 0, with_optimizer: bool = True) -> str:
    """Collective over the job. Returns ``path``."""
    from ..models.hf_export import full_named_weights

    model = getattr(policy_or_model, "model", policy_or_model)
    writer = ps.dp_rank == 0 and ps.tp_rank == 0 and (ps.ep_rank == 0 or ps.ep == 1) and getattr(ps, "cp_rank", 0) == 0
    sd: dict = {}
    for name, t in full_named_weights(model):                 # collectives inside: every rank iterates
        if writer:
            sd[f"model.{name}"] = t.detach().cpu().contiguous()
    if with_optimizer:
        flat = _full_optimizer(policy_or_model, ps)
        if flat is not None:
            for name in model.store.specs:
                spec = model.store.specs[name]
                for kind, buf in flat.items():
                    t = _gather_like_weight(buf, spec, model)
                    if writer:
                        sd[f"optimizer.{kind}.{name}"] = t.detach().cpu().contiguous()
            if writer:
                sd["meta.step"] = torch.tensor(int(policy_or_model.opt.step_count))
    if writer and (ps.pp_rank == 0 or ps.pp == 1):
        sd["meta.global_step"] = torch.tensor(int(step))
    from ..utils import io as uio

    if uio.is_cloud_path(path):
        # every rank writes into a directory of its own (its shard file; the coordinator's also holds ``.metadata``) and
        # uploads it; the files of the ranks have distinct names
        import tempfile

        with tempfile.TemporaryDirectory(prefix="isoexec-dcp-") as tmp:
            _save(sd, tmp)
            uio.upload_directory(tmp, path)
        if dist.is_initialized():
            dist.barrier()
        return path
    _save(sd, path)
    return path


def _save(sd: dict, path: str) -> None:
    dcp = _dcp()
    if dist.is_initialized() and dist.get_world_size() > 1:
        os.makedirs(path, exist_ok=True)
        dist.barrier()
        dcp.save(sd, checkpoint_id=path)                      # ranks that write nothing contribute an empty plan
    else:
        os.makedirs(path, exist_ok=True)
        dcp.save(sd, checkpoint_id=path, no_dist=True)


def _load_keys(path: str, want: dict) -> None:
    """Fill the tensors of ``want`` ({key: preallocated tensor}) from the checkpoint, without collectives."""
    dcp = _dcp()
    dcp.load(want, checkpoint_id=path, no_dist=True)


def load_dcp(policy_or_model, path: str, with_optimizer: bool = True, group_bytes: int = 1 << 30) -> dict:
    """Load a checkpoint written by ``save_dcp`` (at any layout) into this rank's shards. No collectives: every rank reads
    the keys it needs, a group of parameters at a time so that at most ``group_bytes`` of full-shape tensors are held.
    Returns {"global_step": ..., "optimizer": bool}."""
    from ..models.decoder import shard_of

    model = getattr(policy_or_model, "model", policy_or_model)
    ps = model.ps
    dcp = _dcp()
    reader = dcp.FileSystemReader(path)
    keys = set(reader.read_metadata().state_dict_metadata)
    opt = getattr(policy_or_model, "opt", None) if with_optimizer else None
    has_opt = opt is not None and any(k.startswith("optimizer.master.") for k in keys)
    kinds = ("master", "exp_avg", "exp_avg_sq") if has_opt else ()
    if has_opt:
        osd = opt.state_dict()
        lo, hi, _n = osd.get("slice", (0, opt.n, opt.n))

    def cut(full, spec):
        if tuple(full.shape) == tuple(spec.shape):
            return full
        return shard_of(full, spec, ps.tp_rank, ps.tp, ps.ep_rank, ps.ep)

    group: list = []
    held = 0

    def flush():
        nonlocal group, held
        if not group:
            return
        want = {}
        for name, spec, t in group:
            want[f"model.{name}"] = torch.empty(tuple(spec.full_shape), dtype=t.dtype)
            for kind in kinds:
                want[f"optimizer.{kind}.{name}"] = torch.empty(tuple(spec.full_shape), dtype=torch.float32)
        _load_keys(path, want)
        with torch.no_grad():
            for name, spec, t in group:
                t.copy_(cut(want[f"model.{name}"], spec).reshape(t.shape).to(t.device))
                for kind in kinds:
                    # this rank's optimizer slice [lo, hi) of the flat buffer may cover part of the parameter
                    a, b = max(lo, spec.offset), min(hi, spec.offset + math.prod(spec.shape))
                    if a < b:
                        src = cut(want[f"optimizer.{kind}.{name}"], spec).reshape(-1)
                        osd[kind][a - lo:b - lo].copy_(src[a - spec.offset:b - spec.offset].to(osd[kind].device))
        group, held = [], 0

    for name, t in model.named_weights():
        spec = model.store.specs[name]
        if f"model.{name}" not in keys:
            raise KeyError(f"{path} has no tensor model.{name}")
        nbytes = int(torch.Size(spec.full_shape).numel()) * (t.element_size() + 4 * len(kinds))
        if group and held + nbytes > group_bytes:
            flush()
        group.append((name, spec, t))
        held += nbytes
    flush()
    out = {"global_step": 0, "optimizer": bool(has_opt)}
    meta = {k: torch.zeros((), dtype=torch.int64) for k in ("meta.global_step", "meta.step") if k in keys}
    if meta:
        _load_keys(path, meta)
        out["global_step"] = int(meta.get("meta.global_step", torch.zeros(())).item())
        if has_opt and "meta.step" in meta:
            opt.step_count = int(meta["meta.step"].item())
    return out


def main(argv=None) -> None:
    """``python -m skyrl_isoexec_b200.train.dcp_checkpoint list <dir>`` prints every tensor of a checkpoint with its shape."""
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("cmd", choices=["list"])
    ap.add_argument("path")
    a = ap.parse_args(argv)
    md = _dcp().FileSystemReader(a.path).read_metadata().state_dict_metadata
    for k in sorted(md):
        m = md[k]
        print(f"{k:70s} {tuple(getattr(m, 'size', ()))} {getattr(getattr(m, 'properties', None), 'dtype', '')}")


if __name__ == "__main__":
    main()
