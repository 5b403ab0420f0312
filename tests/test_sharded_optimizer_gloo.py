"""Optimizer state cut over the data-parallel group: two gloo ranks, each holding the fp32 master weights and Adam
moments of half the flat buffer, end every step with exactly the weights of the unsharded run; the state round-trips
through state_dict, and a full (unsharded) state loads into a sharded optimizer."""
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


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.models.decoder import DecoderLM
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
        from skyrl_isoexec_b200.train.policy_worker import FlatAdamW, OptimizerConfig, PolicyWorker, WorkerConfig

        ps = ParallelState.build()
        g = torch.Generator().manual_seed(20 + rank)
        prompts = [torch.randint(0, 2048, (8,), generator=g).tolist() for _ in range(4)]
        resp = [torch.randint(0, 2048, (10,), generator=g).tolist() for _ in range(4)]
        seq, att, rmask = build_sequences(prompts, resp)
        batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                    "advantages": torch.randn(rmask.shape, generator=g)})
        final, states = {}, {}
        for sharded in (True, False):
            model = DecoderLM(get_config("tiny-qwen3"), ps, seed=3)
            w = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=64, shard_optimizer=sharded,
                                                 optimizer=OptimizerConfig(lr=1e-2)))
            assert (w.opt.shard is not None) == sharded
            if sharded:
                assert w.opt.master.numel() < w.opt.n and w.opt.exp_avg.numel() == w.opt.hi - w.opt.lo
                assert w.opt.slices[0][1] == w.opt.slices[1][0] and w.opt.slices[-1][1] == w.opt.n
            for _ in range(2):
                w.forward_backward(batch)
                w.optim_step()
            final[sharded] = model.store.flat.detach().clone()
            states[sharded] = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in w.opt.state_dict().items()}
        same = bool(torch.equal(final[True], final[False]))
        # a full state loads into a sharded optimizer (cut to the slice); a sharded state loads back into its own slice
        model = DecoderLM(get_config("tiny-qwen3"), ps, seed=4)
        opt = FlatAdamW(model, OptimizerConfig(), shard=(ps.dp_rank, ps.dp, ps.dp_group))
        opt.load_state_dict(states[False])
        cut_ok = bool(torch.equal(opt.exp_avg, states[True]["exp_avg"]) and torch.equal(model.store.flat.detach(), final[False]))
        opt.load_state_dict(states[True])
        cut_ok = cut_ok and bool(torch.equal(opt.master, states[True]["master"]))
        refused = False
        try:
            other = dict(states[True])
            other["slice"] = (opt.hi, opt.hi + 64, opt.n) if rank == 0 else (0, 64, opt.n)
            opt.load_state_dict(other)
        except ValueError:
            refused = True
        q.put((rank, same, cut_ok, refused))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(240)
def test_sharded_optimizer_matches_unsharded_bit_for_bit():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=150) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    for rank, same, cut_ok, refused in got:
        assert same, f"rank {rank}: sharded and unsharded weights differ"
        assert cut_ok, f"rank {rank}: state did not round-trip"
        assert refused, f"rank {rank}: a state of another slice was accepted"


def _ckpt_worker(rank, world, port, q, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.models.decoder import DecoderLM
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train import checkpoint as ckpt
        from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
        from skyrl_isoexec_b200.train.policy_worker import OptimizerConfig, PolicyWorker, WorkerConfig

        ps = ParallelState.build()
        g = torch.Generator().manual_seed(40 + rank)
        prompts = [torch.randint(0, 2048, (8,), generator=g).tolist() for _ in range(4)]
        resp = [torch.randint(0, 2048, (10,), generator=g).tolist() for _ in range(4)]
        seq, att, rmask = build_sequences(prompts, resp)
        batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                    "advantages": torch.randn(rmask.shape, generator=g)})

        def worker(seed):
            return PolicyWorker(DecoderLM(get_config("tiny-qwen3"), ps, seed=seed),
                                WorkerConfig(max_tokens_per_microbatch=64, optimizer=OptimizerConfig(lr=1e-2)))

        def step(w):
            w.forward_backward(batch)
            w.optim_step()

        a = worker(5)                                  # uninterrupted: three steps
        for _ in range(3):
            step(a)
        b = worker(5)                                  # two steps, save, resume into a fresh worker, one more step
        for _ in range(2):
            step(b)
        ckpt.save_checkpoint(tmp, 2, b, {"pos": 2}, {"global_step": 2}, ps)
        c = worker(77)
        assert c.opt.shard is not None
        data_state, trainer_state = ckpt.load_checkpoint(ckpt.step_dir(tmp, 2), c, ps)
        resumed_same = bool(torch.equal(c.model.store.flat.detach(), b.model.store.flat.detach())
                            and torch.equal(c.opt.exp_avg, b.opt.exp_avg) and c.opt.step_count == 2)
        step(c)
        q.put((rank, resumed_same, bool(torch.equal(c.model.store.flat.detach(), a.model.store.flat.detach())),
               data_state["pos"], trainer_state["global_step"]))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(300)
def test_checkpoint_resume_with_a_sharded_optimizer_continues_bit_for_bit(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ckpt_worker, args=(r, 2, port, q, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=200) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    for rank, resumed_same, continued_same, pos, step in got:
        assert resumed_same, f"rank {rank}: the resumed worker does not hold the saved state"
        assert continued_same, f"rank {rank}: save + resume + step differs from three uninterrupted steps"
        assert pos == 2 and step == 2
    # the same checkpoint read by ONE process (the data-parallel degree changed): weights, step count and the Adam
    # state put back together from the two slices
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.parallel.state import ParallelState
    from skyrl_isoexec_b200.train import checkpoint as ckpt
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    ps1 = ParallelState.single()
    w = PolicyWorker(DecoderLM(get_config("tiny-qwen3"), ps1, seed=1), WorkerConfig())
    ckpt.load_checkpoint(ckpt.step_dir(str(tmp_path), 2), w, ps1)
    shards = [torch.load(f"{ckpt.step_dir(str(tmp_path), 2)}/policy/__{r}_0.distcp", weights_only=False) for r in range(2)]
    want = torch.cat([s["optimizer"]["exp_avg"] for s in shards])
    assert w.opt.shard is None and w.opt.step_count == 2
    assert w.opt.exp_avg.numel() == w.opt.n and torch.equal(w.opt.exp_avg, want) and float(want.abs().sum()) > 0
    assert torch.equal(w.opt.master, w.model.store.flat.detach().float())
