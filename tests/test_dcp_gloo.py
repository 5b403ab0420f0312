"""torch.distributed.checkpoint format: a checkpoint written by a tensor-parallel job with a sharded optimizer is read by
torch's own converter and loads into a single-process model (and back), weights and optimizer state alike."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _param_views(worker, flat):
    m = worker.model
    out = {}
    for n, p in m.named_weights():
        s = m.store.specs[n]
        out[n] = flat[s.offset:s.offset + p.numel()].view(p.shape)
    return out


def _fill(worker, seed):
    g = torch.Generator().manual_seed(seed)
    for kind in ("master", "exp_avg", "exp_avg_sq"):
        t = getattr(worker.opt, kind)
        t.copy_(torch.randn(t.shape, generator=g))
    worker.opt.step_count = 11


def _worker(rank, world, port, path, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    err = None
    try:
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.models.decoder import DecoderLM
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train import dcp_checkpoint as D
        from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

        ps = ParallelState.build(tp=2)                       # 4 ranks: tp2 x dp2, optimizer state cut over dp
        model = DecoderLM(get_config("tiny-qwen3"), ps, "cpu", seed=4)
        w = PolicyWorker(model, WorkerConfig())
        assert w.opt.shard is not None and w.opt.hi - w.opt.lo < w.opt.n
        # what a single-process job saved (path/single) loads into this layout ...
        info = D.load_dcp(w, os.path.join(path, "single"))
        assert info == {"global_step": 5, "optimizer": True} and w.opt.step_count == 11
        # ... and is written back from it
        D.save_dcp(w, os.path.join(path, "tp2dp2"), ps, step=6)
    except Exception as e:  # noqa: BLE001
        import traceback

        err = traceback.format_exc()
    q.put((rank, err))
    if err is None:
        dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_dcp_checkpoint_round_trips_between_layouts_and_is_read_by_torch(tmp_path):
    from torch.distributed.checkpoint.format_utils import dcp_to_torch_save

    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train import dcp_checkpoint as D
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    cfg = get_config("tiny-qwen3")
    ref = PolicyWorker(DecoderLM(cfg, device="cpu", seed=9), WorkerConfig())
    _fill(ref, 1)
    D.save_dcp(ref, str(tmp_path / "single"), ref.model.ps, step=5)
    assert {".metadata", "__0_0.distcp"} <= set(os.listdir(tmp_path / "single"))
    # torch's own converter reads it: full-shape tensors under plain names
    dcp_to_torch_save(str(tmp_path / "single"), str(tmp_path / "single.pt"))
    sd = torch.load(tmp_path / "single.pt", weights_only=False)
    for n, p in ref.model.named_weights():
        assert torch.equal(sd[f"model.{n}"], p.detach()) and sd[f"optimizer.exp_avg.{n}"].shape == p.shape
    assert int(sd["meta.global_step"]) == 5 and int(sd["meta.step"]) == 11
    # a 4-rank job (tp2 x dp2, sharded optimizer) loads it and saves its own
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 4, port, str(tmp_path), q)) for r in range(4)]
    for p in procs:
        p.start()
    for _ in range(4):
        r, err = q.get(timeout=200)
        assert err is None, f"rank {r}:\n{err}"
    for p in procs:
        p.join(timeout=60)
    # the checkpoint written by the 4-rank job loads into a fresh single-process model with the same bits
    back = PolicyWorker(DecoderLM(cfg, device="cpu", seed=123), WorkerConfig())
    info = D.load_dcp(back, str(tmp_path / "tp2dp2"))
    assert info == {"global_step": 6, "optimizer": True} and back.opt.step_count == 11
    for (n, a), (_, b) in zip(ref.model.named_weights(), back.model.named_weights()):
        assert torch.equal(a, b), n
    for kind in ("master", "exp_avg", "exp_avg_sq"):
        va, vb = _param_views(ref, getattr(ref.opt, kind)), _param_views(back, getattr(back.opt, kind))
        for n in va:
            assert torch.equal(va[n], vb[n]), (kind, n)
    # weights only, into a bare model
    bare = DecoderLM(cfg, device="cpu", seed=77)
    assert D.load_dcp(bare, str(tmp_path / "tp2dp2"))["optimizer"] is False
    assert all(torch.equal(a, b) for (_, a), (_, b) in zip(ref.model.named_weights(), bare.named_weights()))
