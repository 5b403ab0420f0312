"""Resume fidelity on two data-parallel gloo ranks with a critic and an adaptive KL controller: after a restart every rank
draws the prompt shard it would have drawn without the restart (disjoint from the other rank's), the critic, its value
head and optimizers, the KL coefficient and the epoch come back, and training continues from the saved step."""
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


def _cfg(d, steps):
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig

    return SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8",
        "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=12",
        "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.epochs=4",
        "trainer.policy.optimizer_config.lr=1e-3", f"trainer.num_steps={steps}", f"trainer.ckpt_path={d}",
        "trainer.ckpt_interval=2", "trainer.logger=jsonl", "trainer.algorithm.advantage_estimator=gae",
        "trainer.algorithm.use_kl_in_reward=true", "trainer.algorithm.kl_ctrl_type=adaptive", "trainer.algorithm.init_kl_coef=0.05"])


def _worker(rank, world, port, d, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

        ps = ParallelState.build()
        seen = []

        from skyrl_isoexec_b200.train.callbacks import TrainingCallback

        class Spy(TrainingCallback):
            def on_step_start(self, trainer, inp, control):
                seen.append([r["uid"] for r in inp.batch])

        # uninterrupted run: 5 steps (12 prompts, global batch 4 -> 3 steps per epoch, so step 4 opens epoch 1)
        tr = RayPPOTrainer(_cfg(d + "/a", 5), ps=ps, device="cpu", callbacks=[Spy()])
        tr.train()
        full = list(seen)
        # the same run cut at step 4 (checkpoint at 2 and 4), then resumed to 5
        seen.clear()
        tr1 = RayPPOTrainer(_cfg(d + "/b", 4), ps=ps, device="cpu", callbacks=[Spy()])
        tr1.train()
        crit = {n: t.clone() for n, t in tr1.critic.model.named_weights()}
        head = tr1.critic.v_weight.detach().clone()
        klv = tr1.kl_ctrl.value
        seen.clear()
        tr2 = RayPPOTrainer(_cfg(d + "/b", 5), ps=ps, device="cpu", callbacks=[Spy()])
        tr2.build_models()
        assert tr2.load_checkpoints() == 4
        ok_critic = all(torch.equal(t, crit[n]) for n, t in tr2.critic.model.named_weights()) and torch.equal(tr2.critic.v_weight, head)
        ok_kl = tr2.kl_ctrl.value == klv and klv != 0.05
        ok_epoch = tr2.epoch == 1
        ok_opt = tr2.critic.opt.step_count == tr1.critic.opt.step_count > 0
        tr2.train()
        resumed = list(seen)
        q.put((rank, full, resumed, ok_critic, ok_kl, ok_epoch, ok_opt, tr2.global_step))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(600)
def test_dp2_resume_keeps_shards_disjoint_and_restores_critic_and_kl(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    res = []
    import queue as _q
    import time as _t
    t0 = _t.time()
    while len(res) < 2 and _t.time() - t0 < 560:
        try:
            res.append(q.get(timeout=2))
        except _q.Empty:
            assert all(p.is_alive() or p.exitcode == 0 for p in procs), "a rank died"
    res.sort()
    for p in procs:
        p.join(timeout=60)
    (_, full0, res0, *flags0, gs0), (_, full1, res1, *flags1, gs1) = res
    assert all(flags0) and all(flags1), (flags0, flags1)
    assert gs0 == gs1 == 5
    for a, b in zip(full0, full1):                       # the two ranks never share a prompt within a step
        assert not set(a) & set(b) and len(a) == len(b) == 2
    for e in range(0, 3, 3):                             # an epoch visits every prompt exactly once across the job
        uids = [u for s in range(e, e + 3) for u in full0[s] + full1[s]]
        assert len(uids) == len(set(uids)) == 12
    # the resumed run's step 5 draws exactly what the uninterrupted run drew at step 5, on each rank
    assert res0 == [full0[4]] and res1 == [full1[4]]
