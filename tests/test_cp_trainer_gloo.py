"""Context parallelism driven from the trainer configuration (two gloo ranks on CPU): every micro-batch is cut over the
cp ranks, attention exchanges heads for tokens, each rank scores and trains the tokens of its share, gradients are
summed over the cp group. Rollout logprobs equal the context-parallel scoring forward bit for bit, and the updated
weights agree with a single-rank trainer given the same batch."""
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
        "generator.n_samples_per_prompt=4", "generator.sampling_params.max_generate_length=11",
        "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=9", "data.synthetic_prompts=16",
        "trainer.max_prompt_length=9", "generator.inference_engine.num_kv_pages=16", "trainer.policy.optimizer_config.lr=1e-2",
        "trainer.logger=jsonl", "trainer.max_tokens_per_microbatch=70"])


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig
        from skyrl_isoexec_b200.models.decoder import DecoderLM
        from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

        ps = ParallelState.build(cp=world)
        tr = RayPPOTrainer(_cfg(), ps=ps, device="cpu")
        tr.build_models()
        assert tr.engines_per_replica == world and not tr.separate_engine
        tr.sync_weights()
        rows = next(iter(tr.loader))
        # the same batch through a single-rank worker with the same initial weights, for comparison
        solo = DecoderLM(tr.policy.model.cfg, ParallelState.single(), "cpu", seed=tr.cfg.trainer.policy.seed)
        assert torch.equal(solo.store.flat, tr.policy.model.store.flat)
        captured = {}
        orig = tr.train_critic_and_policy

        def spy(batch):
            captured["batch"] = batch.slice(0, batch.batch_size)
            return orig(batch)

        tr.train_critic_and_policy = spy
        m = tr.train_step(rows)
        mism = int(m["policy/rollout_train_logprob_bit_mismatches"])
        b = captured["batch"]
        w1 = PolicyWorker(solo, WorkerConfig(max_tokens_per_microbatch=70, optimizer=tr.policy.cfg.optimizer), tr.policy.algo)
        lp1 = w1.forward(b)
        same_lp = bool(torch.equal(lp1, b["action_log_probs"]))
        b["advantages"] = b["advantages"] / b["loss_mask"].sum()          # the trainer's token_mean pre-scaling of a mini-batch
        w1.forward_backward(b)
        gn1 = w1.optim_step()
        diff = float((solo.store.flat - tr.policy.model.store.flat).abs().max())
        q.put((rank, mism, same_lp, diff, float(m["policy/grad_norm"]), gn1, int(m["generate/response_tokens"])))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(600)
def test_context_parallel_trainer_matches_single_rank():
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
    for rank, mism, same_lp, diff, gn, gn1, toks in sorted(res):
        assert mism == 0 and same_lp                          # scoring under cp = the single-rank scoring, bit for bit
        assert toks == 2 * 4 * 11
        # Adam's first step moves every weight by about lr * g / |g|: where a gradient is within rounding of zero the two
        # summation orders may disagree on its sign, so single weights can differ by a fraction of lr = 1e-2
        assert abs(gn - gn1) < 1e-5 * max(1.0, gn1) and diff < 2e-3, (gn, gn1, diff)
