"""Checkpoints, exports and enforcement verdicts under a remote path scheme. ``memory://`` is fsspec's in-process store (one
process); ``local://`` is the local disk reached through the same remote code path, which two gloo ranks can share."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from skyrl_isoexec_b200.train import checkpoint as ckpt
from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
from skyrl_isoexec_b200.utils import io as uio


def _cfg(root, steps, extra=()):
    return SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8",
        "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=16",
        "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16",
        "trainer.policy.optimizer_config.lr=1e-3", f"trainer.num_steps={steps}", f"trainer.ckpt_path={root}/ck",
        "trainer.ckpt_interval=1", "trainer.max_ckpts_to_keep=2", "trainer.logger=jsonl", *extra])


def test_io_helpers_on_a_remote_scheme(tmp_path):
    base = "memory://io-helpers/run"
    assert uio.is_cloud_path(base) and not uio.is_cloud_path(str(tmp_path)) and not uio.is_cloud_path("file:///x")
    with uio.local_work_dir(base + "/d") as d:
        os.makedirs(d + "/sub")
        open(d + "/sub/a.bin", "wb").write(b"123")
        open(d + "/top.txt", "w").write("t")
    assert uio.exists(base + "/d/top.txt") and uio.isdir(base + "/d") and uio.list_dir(base + "/d") == ["sub", "top.txt"]
    with uio.local_read_dir(base + "/d") as d:
        assert open(d + "/sub/a.bin", "rb").read() == b"123"
    with pytest.raises(FileNotFoundError):
        with uio.local_read_dir(base + "/nothing-here"):
            pass
    with uio.pack_and_upload(base + "/arch.tgz") as d:
        open(d + "/w.txt", "w").write("weights")
    with uio.download_and_unpack(base + "/arch.tgz") as d:
        assert open(d + "/w.txt").read() == "weights"
    uio.remove(base + "/d")
    assert not uio.exists(base + "/d")
    with pytest.raises(RuntimeError, match="s3fs"):
        uio.exists("s3://bucket/key")

    # an error that looks transient is retried on a fresh filesystem instance; any other error is raised at once
    calls = []

    def flaky(fs, p):
        calls.append(p)
        if len(calls) < 3:
            raise OSError("SlowDown: please reduce your request rate")
        return "done"

    old = uio.BACKOFF_S
    uio.BACKOFF_S = 0.0
    try:
        assert uio._retry(base + "/x", flaky) == "done" and len(calls) == 3
        with pytest.raises(KeyError):
            uio._retry(base + "/x", lambda fs, p: (_ for _ in ()).throw(KeyError("no")))
    finally:
        uio.BACKOFF_S = old


def test_trainer_checkpoints_and_exports_to_a_remote_store_and_resumes_from_it():
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    root = "memory://remote-ckpt-test"
    uio.remove(root)
    tr = RayPPOTrainer(_cfg(root, 3, [f"trainer.export_path={root}/out", "trainer.hf_save_interval=3", "trainer.dcp_save_interval=3"]), device="cpu")
    tr.train()
    assert ckpt.list_checkpoints(root + "/ck") == [2, 3]                     # step 1 went with max_ckpts_to_keep=2
    with uio.open_file(root + "/ck/" + ckpt.LATEST) as f:
        assert f.read() == "3"
    assert set(uio.list_dir(root + "/ck/global_step_3")) == {"data.pt", "policy", "trainer_state.pt"}
    assert {"metadata.json", "__0_0.distcp"} <= set(uio.list_dir(root + "/ck/global_step_3/policy"))
    assert {"enforcement.trainer.r0.json", "enforcement.engine.r0.json"} <= set(uio.list_dir(root + "/ck"))
    assert {"model.safetensors", "config.json"} <= set(uio.list_dir(root + "/out/global_step_3"))
    assert {".metadata", "__0_0.distcp"} <= set(uio.list_dir(root + "/out/global_step_3/dcp"))
    want = {n: t.clone() for n, t in tr.policy.model.named_weights()}
    tr3 = RayPPOTrainer(_cfg(root, 4, ["trainer.resume_mode=from_path", f"trainer.resume_path={root}/out/global_step_3/dcp"]), device="cpu")
    tr3.build_models()
    assert tr3.load_checkpoints() == 3 and all(torch.equal(t, want[n]) for n, t in tr3.policy.model.named_weights())
    tr2 = RayPPOTrainer(_cfg(root, 4), device="cpu")
    tr2.build_models()
    assert tr2.load_checkpoints() == 3 and tr2.policy.opt.step_count == tr.policy.opt.step_count
    assert all(torch.equal(t, want[n]) for n, t in tr2.policy.model.named_weights())
    # resume_mode=from_path with a remote step directory
    path = ckpt.resolve_resume_path("", "from_path", root + "/ck/global_step_2")
    assert os.path.isdir(path) and os.path.basename(path) == "global_step_2" and os.path.exists(path + "/policy/metadata.json")
    # a step directory that the marker does not point at (a crash between the uploads and the marker) is not resumed from
    with uio.atomic_write(root + "/ck/" + ckpt.LATEST) as f:
        f.write("2")
    ckpt._STAGED.clear()
    assert os.path.basename(ckpt.resolve_resume_path(root + "/ck", "latest")) == "global_step_2"


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, d, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      SKYRL_ISOEXEC_STAGE_DIR=d + "/stage")
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

        ps = ParallelState.build()
        root = "local://" + d + "/store"
        tr = RayPPOTrainer(_cfg(root, 2), ps=ps, device="cpu")
        tr.train()
        want = {n: t.clone() for n, t in tr.policy.model.named_weights()}
        opt = tr.policy.opt.state_dict()
        tr2 = RayPPOTrainer(_cfg(root, 3), ps=ps, device="cpu")
        tr2.build_models()
        step = tr2.load_checkpoints()
        ok_w = all(torch.equal(t, want[n]) for n, t in tr2.policy.model.named_weights())
        opt2 = tr2.policy.opt.state_dict()
        ok_o = all(torch.equal(opt[k], opt2[k]) for k in ("master", "exp_avg", "exp_avg_sq")) and tuple(opt["slice"]) == tuple(opt2["slice"])
        tr2.train()
        q.put((rank, step, ok_w, ok_o, tr2.global_step, sorted(os.listdir(d + "/store/ck/global_step_2/policy"))))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(600)
def test_two_ranks_upload_their_own_shards_and_resume_through_one_download(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=500) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, step, ok_w, ok_o, final, files in res:
        assert step == 2 and ok_w and ok_o and final == 3
        assert files == ["__0_0.distcp", "__1_0.distcp", "metadata.json"]
