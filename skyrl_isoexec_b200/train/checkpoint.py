"""Checkpoint save / resume in the reference's directory layout
(docs/content/docs/checkpointing-logging/checkpointing.mdx:36-85,116-128; R/train/trainer.py:1858-2036):

    {ckpt_path}/latest_ckpt_global_step.txt
    {ckpt_path}/global_step_N/policy/metadata.json
    {ckpt_path}/global_step_N/policy/__{rank}_0.distcp     (one shard file per rank)
    {ckpt_path}/global_step_N/data.pt                       (dataloader state)
    {ckpt_path}/global_step_N/trainer_state.pt

A shard file holds the rank's slice of the sharded state dict with the keys ``model`` /
``optimizer`` / ``lr_scheduler`` / ``rng``. The files follow the naming of torch's distributed
checkpoints but are ``torch.save`` pickles with a JSON index: they are NOT readable by
``torch.distributed.checkpoint`` or Megatron's dist-checkpointing tools; for interchange there are the
torch.distributed.checkpoint export (``train/dcp_checkpoint.py``, ``trainer.dcp_save_interval``) and the HF export. A critic, when there is one, is saved the same way under ``critic/``. ``metadata.json`` records every parameter's full
shape, shard dim and sections so a checkpoint written at one TP degree loads at another
(parameters are reassembled to full shape and re-sliced). The step directory is written under
a temporary name and renamed, and ``latest_ckpt_global_step.txt`` is replaced last, so a crash
mid-save never leaves a directory that ``resume_mode=latest`` would pick up.

``ckpt_path`` (and ``resume_path``) may name an object store or any other fsspec scheme (``s3://``, ``gs://`` ...;
``utils/io.py``): every rank then writes its files into a private temporary directory and uploads them, rank 0 replaces
the remote ``latest_ckpt_global_step.txt`` after all uploads returned (a step directory without that marker pointing at it
is never resumed from) and deletes the steps beyond ``max_to_keep``; a resume downloads the step directory once per node
into a staging directory that lives until the process exits.
"""

from __future__ import annotations

import atexit
import hashlib
import json
import os
import random
import re
import shutil
import tempfile

import torch
import torch.distributed as dist

from ..utils import io as uio

LATEST = "latest_ckpt_global_step.txt"
_STEP_RE = re.compile(r"^global_step_(\d+)$")


def _barrier():
    if dist.is_initialized():
        dist.barrier()


def _rank():
    return dist.get_rank() if dist.is_initialized() else 0


def step_dir(ckpt_path: str, step: int) -> str:
    return os.path.join(ckpt_path, f"global_step_{step}")


def _write_step(tmp: str, step: int, policy, data_state: dict, trainer_state: dict, ps, extra_shards: dict | None) -> list[str]:
    """This rank's files of one checkpoint into the directory ``tmp``; returns their paths relative to ``tmp``."""
    rank = _rank()
    model = policy.model
    wrote = []
    os.makedirs(os.path.join(tmp, "policy"), exist_ok=True)
    shard = {
        "model": {name: t.detach().cpu().clone() for name, t in model.named_weights()},
        "optimizer": {k: (v.detach().cpu().clone() if torch.is_tensor(v) else v) for k, v in policy.opt.state_dict().items()},
        "lr_scheduler": {"step": policy.opt.step_count},
        "rng": {"torch": torch.get_rng_state(), "python": random.getstate(),
                "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None},
        "parallel": {"tp": ps.tp, "tp_rank": ps.tp_rank, "dp_rank": ps.dp_rank, "pp_rank": ps.pp_rank, "ep_rank": ps.ep_rank},
    }
    torch.save(shard, os.path.join(tmp, "policy", f"__{rank}_0.distcp"))
    wrote.append(f"policy/__{rank}_0.distcp")
    for folder, state in (extra_shards or {}).items():
        os.makedirs(os.path.join(tmp, folder), exist_ok=True)
        torch.save(state, os.path.join(tmp, folder, f"__{rank}_0.distcp"))
        wrote.append(f"{folder}/__{rank}_0.distcp")
    if rank == 0:
        meta = {
            "format": "skyrl_isoexec_b200.sharded.v1", "global_step": step, "world_size": dist.get_world_size() if dist.is_initialized() else 1,
            "tp": ps.tp, "pp": ps.pp, "dp": ps.dp, "ep": ps.ep, "model_config": model.cfg.to_dict(),
            "params": {n: {"full_shape": list(s.full_shape), "shard_dim": s.shard_dim, "sections": list(s.sections),
                           "ep_sharded": s.ep_sharded, "offset": s.offset, "shape": list(s.shape),
                           "kv_rep": s.kv_rep, "kv_layout": list(s.kv_layout)}
                       for n, s in model.store.specs.items()},
        }
        with open(os.path.join(tmp, "policy", "metadata.json"), "w") as f:
            json.dump(meta, f, indent=1, sort_keys=True)
        torch.save(data_state, os.path.join(tmp, "data.pt"))
        torch.save(trainer_state, os.path.join(tmp, "trainer_state.pt"))
        wrote += ["policy/metadata.json", "data.pt", "trainer_state.pt"]
    return wrote


def save_checkpoint(ckpt_path: str, step: int, policy, data_state: dict, trainer_state: dict, ps, max_to_keep: int = -1,
                    extra_shards: dict | None = None) -> str:
    """``extra_shards``: ``{folder: this rank's state}`` written as ``{folder}/__{rank}_0.distcp`` beside ``policy/``."""
    final = step_dir(ckpt_path, step)
    rank = _rank()
    if uio.is_cloud_path(ckpt_path):
        final = ckpt_path.rstrip("/") + f"/global_step_{step}"
        if rank == 0:
            uio.remove(final)                                   # a partial upload of an earlier attempt at this step
        _barrier()
        with tempfile.TemporaryDirectory(prefix="isoexec-ckpt-") as tmp:
            wrote = _write_step(tmp, step, policy, data_state, trainer_state, ps, extra_shards)
            uio.upload_directory(tmp, final, only=wrote)
        _barrier()                                              # every rank's files are up before the marker moves
        if rank == 0:
            with uio.atomic_write(ckpt_path.rstrip("/") + "/" + LATEST) as f:
                f.write(str(step))
            cleanup_old_checkpoints(ckpt_path, max_to_keep)
        _barrier()
        return final
    tmp = final + ".tmp"
    if rank == 0:
        if os.path.isdir(tmp):
            shutil.rmtree(tmp)
        os.makedirs(os.path.join(tmp, "policy"), exist_ok=True)
    _barrier()
    _write_step(tmp, step, policy, data_state, trainer_state, ps, extra_shards)
    _barrier()
    if rank == 0:
        if os.path.isdir(final):
            shutil.rmtree(final)
        os.replace(tmp, final)
        with open(os.path.join(ckpt_path, LATEST + ".tmp"), "w") as f:
            f.write(str(step))
        os.replace(os.path.join(ckpt_path, LATEST + ".tmp"), os.path.join(ckpt_path, LATEST))
        cleanup_old_checkpoints(ckpt_path, max_to_keep)
    _barrier()
    return final


def list_checkpoints(ckpt_path: str) -> list[int]:
    if not uio.isdir(ckpt_path):
        return []
    steps = []
    for d in uio.list_dir(ckpt_path):
        m = _STEP_RE.match(d)
        if m and uio.isdir(ckpt_path.rstrip("/") + "/" + d):
            steps.append(int(m.group(1)))
    return sorted(steps)


def cleanup_old_checkpoints(ckpt_path: str, max_to_keep: int) -> list[int]:
    if max_to_keep is None or max_to_keep < 0:
        return []
    steps = list_checkpoints(ckpt_path)
    drop = steps[:-max_to_keep] if max_to_keep > 0 else steps
    for s in drop:
        if uio.is_cloud_path(ckpt_path):
            uio.remove(ckpt_path.rstrip("/") + f"/global_step_{s}")
        else:
            shutil.rmtree(step_dir(ckpt_path, s), ignore_errors=True)
    return drop


def validate_checkpoint_dir(path: str) -> None:
    if os.path.exists(os.path.join(path, ".metadata")):
        return                     # a torch.distributed.checkpoint directory (train/dcp_checkpoint.py)
    if not _STEP_RE.match(os.path.basename(os.path.normpath(path))):
        raise ValueError(f"resume_path must be a global_step_N directory, got {path!r}")
    for need in ("policy/metadata.json", "data.pt", "trainer_state.pt"):
        if not os.path.exists(os.path.join(path, need)):
            raise FileNotFoundError(f"checkpoint {path} is incomplete: missing {need}")


_STAGED: dict[str, str] = {}


def _stage_remote(path: str) -> str:
    """Download a remote checkpoint directory once per node (the rank with LOCAL_RANK 0 fetches, the others wait) into a
    staging directory removed when the process exits; returns the local directory, named like the remote one."""
    if path in _STAGED:
        return _STAGED[path]
    root = os.path.join(os.environ.get("SKYRL_ISOEXEC_STAGE_DIR") or tempfile.gettempdir(),
                        "isoexec-resume-" + hashlib.sha1(path.encode()).hexdigest()[:12])
    local = os.path.join(root, path.rstrip("/").rsplit("/", 1)[-1])
    leader = int(os.environ.get("LOCAL_RANK", "0")) == 0
    err = None
    if leader:
        try:
            shutil.rmtree(root, ignore_errors=True)
            if uio.download_directory(path, local) == 0:
                raise FileNotFoundError(f"nothing under {path}")
            atexit.register(shutil.rmtree, root, True)
        except Exception as e:  # noqa: BLE001 - raised after the barrier so that the waiting ranks are released first
            err = e
    _barrier()
    if err is not None:
        raise err
    _STAGED[path] = local
    return local


def resolve_resume_path(ckpt_path: str, resume_mode: str, resume_path: str = "") -> str | None:
    """The LOCAL directory to resume from, or None. Remote checkpoints are downloaded first (``_stage_remote``)."""
    if resume_mode == "none":
        return None
    if resume_mode == "from_path":
        if uio.is_cloud_path(resume_path):
            resume_path = _stage_remote(resume_path)
        validate_checkpoint_dir(resume_path)
        return resume_path
    latest = ckpt_path.rstrip("/") + "/" + LATEST if uio.is_cloud_path(ckpt_path) else os.path.join(ckpt_path, LATEST)
    if not uio.exists(latest):
        return None
    with uio.open_file(latest) as f:
        step = int(str(f.read()).strip())
    if uio.is_cloud_path(ckpt_path):
        path = _stage_remote(ckpt_path.rstrip("/") + f"/global_step_{step}")
    else:
        path = step_dir(ckpt_path, step)
    validate_checkpoint_dir(path)
    return path


def _assemble_full(name: str, meta: dict, shards: list[dict]) -> torch.Tensor:
    """Rebuild a parameter at full shape from the shards of one data-parallel replica of the saved layout.
    ``shards``: the saved shard dicts of one pipeline stage; TP shards are joined on the shard dim (per section),
    expert-parallel shards on the leading expert dim."""
    info = meta["params"][name]

    def join_tp(parts):
        if info["shard_dim"] is None or len(parts) == 1:
            return parts[0]
        if info.get("kv_rep", 1) > 1:
            from types import SimpleNamespace

            from ..models.decoder import unshard_kv_rep

            return unshard_kv_rep(parts, SimpleNamespace(kv_rep=info["kv_rep"], kv_layout=tuple(info["kv_layout"])))
        d, tp = info["shard_dim"], len(parts)
        secs = info["sections"] or [info["full_shape"][d]]
        cols = []
        for si, sz in enumerate(secs):
            lo = sum(x // tp for x in secs[:si])
            cols += [p.narrow(d, lo, sz // tp) for p in parts]
        return torch.cat(cols, dim=d)

    if info.get("ep_sharded") and meta.get("ep", 1) > 1:
        # one (tp-joined) block per saved expert-parallel rank, concatenated on the expert dim
        blocks = []
        for e in range(meta["ep"]):
            mine = sorted((s for s in shards if s["parallel"]["ep_rank"] == e), key=lambda s: s["parallel"]["tp_rank"])
            seen, uniq = set(), []
            for s in mine:                       # ranks of other expert-data-parallel replicas hold copies
                if s["parallel"]["tp_rank"] not in seen:
                    seen.add(s["parallel"]["tp_rank"])
                    uniq.append(s)
            if not uniq:
                raise KeyError(f"checkpoint has no shard of expert-parallel rank {e} for {name}")
            blocks.append(join_tp([s["model"][name] for s in uniq]))
        return torch.cat(blocks, dim=0)
    seen, parts = set(), []
    for s in sorted(shards, key=lambda s: s["parallel"]["tp_rank"]):
        if s["parallel"]["tp_rank"] not in seen:
            seen.add(s["parallel"]["tp_rank"])
            parts.append(s["model"][name])
    return join_tp(parts)


def _assemble_optimizer_state(shards: list[dict]) -> dict | None:
    """Full optimizer state of one (tp, pp, ep) position from what its data-parallel ranks saved: either every rank
    saved everything (take one), or each saved one slice of the flat buffer (concatenate in slice order)."""
    pieces = {}
    for s in shards:
        o = s["optimizer"]
        lo, hi, n = o.get("slice", (0, o["master"].numel(), o["master"].numel()))
        pieces[(lo, hi)] = (o, n)
    if not pieces:
        return None
    n = next(iter(pieces.values()))[1]
    if (0, n) in pieces:
        return dict(pieces[(0, n)][0])
    spans = sorted(k for k in pieces if k[1] > k[0])
    if not spans or spans[0][0] != 0 or spans[-1][1] != n or any(a[1] != b[0] for a, b in zip(spans, spans[1:])):
        return None                                   # slices do not tile the buffer
    out = {k: torch.cat([pieces[sp][0][k] for sp in spans]) for k in ("master", "exp_avg", "exp_avg_sq")}
    out["step"] = pieces[spans[0]][0]["step"]
    out["slice"] = (0, n, n)
    return out


def load_extra_shard(path: str, folder: str):
    """This rank's file of an extra folder written by ``save_checkpoint(extra_shards=...)``; None if absent."""
    f = os.path.join(path, folder, f"__{_rank()}_0.distcp")
    return torch.load(f, map_location="cpu", weights_only=False) if os.path.exists(f) else None


def _restore_rng(rng: dict) -> None:
    torch.set_rng_state(rng["torch"])
    random.setstate(rng["python"])
    if rng.get("cuda") is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(rng["cuda"])


def load_checkpoint(path: str, policy, ps) -> tuple[dict, dict]:
    """Load the policy (weights, optimizer, RNG) saved under ``path`` into this job's layout.

    Same layout: every rank reads its own file. A different tensor-, expert- or data-parallel degree: parameters are
    rebuilt at full shape from one saved replica and re-sliced; the optimizer state carries over only when the flat
    layout of a rank is unchanged (data-parallel degree changed alone) and is otherwise started fresh, with a warning.
    A different pipeline-parallel degree is refused (a stage's file holds its own layers only)."""
    validate_checkpoint_dir(path)
    with open(os.path.join(path, "policy", "metadata.json")) as f:
        meta = json.load(f)
    model = policy.model
    rank = _rank()
    same_layout = (meta["tp"] == ps.tp and meta["pp"] == ps.pp and meta["ep"] == ps.ep
                   and meta["world_size"] == (dist.get_world_size() if dist.is_initialized() else 1))
    from ..models.decoder import shard_of

    if same_layout:
        shard = torch.load(os.path.join(path, "policy", f"__{rank}_0.distcp"), map_location="cpu", weights_only=False)
        with torch.no_grad():
            for name, dst in model.named_weights():
                dst.copy_(shard["model"][name].to(dst.dtype))
        policy.opt.load_state_dict({k: (v.to(policy.opt.master.device) if torch.is_tensor(v) else v)
                                    for k, v in shard["optimizer"].items()})
        _restore_rng(shard["rng"])
    else:
        if meta["pp"] != ps.pp:
            raise ValueError(f"checkpoint was written with pipeline_parallel={meta['pp']}; this job uses {ps.pp}. Resharding "
                             f"covers tensor-, expert- and data-parallel changes only")
        files = sorted(f for f in os.listdir(os.path.join(path, "policy")) if f.endswith(".distcp"))
        every = [torch.load(os.path.join(path, "policy", f), map_location="cpu", weights_only=False) for f in files]
        stage = [s for s in every if s["parallel"]["pp_rank"] == ps.pp_rank]
        if not stage:
            raise KeyError(f"checkpoint holds no shard of pipeline stage {ps.pp_rank}")
        with torch.no_grad():
            for name, dst in model.named_weights():
                full = _assemble_full(name, meta, stage)
                want = tuple(model.store.specs[name].full_shape)
                if tuple(full.shape) != want:
                    raise ValueError(f"{name}: rebuilt shape {tuple(full.shape)} from the checkpoint, expected {want}")
                dst.copy_(shard_of(full, model.store.specs[name], ps.tp_rank, ps.tp, ps.ep_rank, ps.ep).to(dst.dtype))
            if policy.opt.low_precision:
                policy.opt.master.copy_(model.store.flat[policy.opt.lo:policy.opt.hi].float())
        policy.opt.step_count = int(stage[0]["lr_scheduler"]["step"])
        carried = False
        if meta["tp"] == ps.tp and meta["ep"] == ps.ep:
            # only the data-parallel degree changed: the flat layout of this rank is the saved one, so the optimizer
            # state (whole, or the slices a sharded optimizer wrote) is put back together and cut again
            full = _assemble_optimizer_state([s for s in stage if s["parallel"]["tp_rank"] == ps.tp_rank
                                              and s["parallel"]["ep_rank"] == ps.ep_rank])
            if full is not None:
                policy.opt.load_state_dict({k: (v.to(policy.opt.master.device) if torch.is_tensor(v) else v) for k, v in full.items()})
                carried = True
        if not carried and rank == 0:
            print(f"[warn] checkpoint layout (tp={meta['tp']} ep={meta['ep']} dp={meta['dp']}) differs from this job's "
                  f"(tp={ps.tp} ep={ps.ep} dp={ps.dp}): weights were resharded, Adam moments start from zero")
    data_state = torch.load(os.path.join(path, "data.pt"), weights_only=False)
    trainer_state = torch.load(os.path.join(path, "trainer_state.pt"), weights_only=False)
    return data_state, trainer_state


def save_hf_export(export_path: str, step: int, model) -> str:
    """Export full-shape weights + config as ``{export_path}/global_step_N/policy/`` (single-rank layouts)."""
    out = export_path.rstrip("/") + f"/global_step_{step}/policy" if uio.is_cloud_path(export_path) \
        else os.path.join(export_path, f"global_step_{step}", "policy")
    with uio.local_work_dir(out) as d:
        torch.save({n: t.detach().cpu() for n, t in model.named_weights()}, os.path.join(d, "pytorch_model.bin"))
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump({"architectures": [model.cfg.architecture], **model.cfg.to_dict()}, f, indent=1)
    return out
