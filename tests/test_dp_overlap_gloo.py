"""Data-parallel gradient reduction overlapped with the last micro-batch's backward gives the same gradients
as reducing after the backward (two gloo ranks on CPU, different data per rank)."""
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
        from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

        ps = ParallelState.build()
        assert ps.dp == world
        g = torch.Generator().manual_seed(10 + rank)
        prompts = [torch.randint(0, 2048, (8,), generator=g).tolist() for _ in range(6)]
        resp = [torch.randint(0, 2048, (10,), generator=g).tolist() for _ in range(6)]
        seq, att, rmask = build_sequences(prompts, resp)
        batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                    "advantages": torch.randn(rmask.shape, generator=g)})
        grads = {}
        for overlap in (True, False):
            model = DecoderLM(get_config("tiny-qwen3"), ps, seed=1)
            w = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=40, overlap_grad_reduce=overlap))
            if overlap:
                w.opt.setup_overlap(ps, bucket_elems=200_000)        # several buckets
            w.forward_backward(batch)
            if overlap:
                assert w.opt._ov["active"] and len(w.opt._ov["done"]) >= len(w.opt._ov["buckets"]) - 1
            w.reduce_gradients()
            grads[overlap] = w.opt.main_grad.clone()
        local = DecoderLM(get_config("tiny-qwen3"), ParallelState.single(), seed=1)
        wl = PolicyWorker(local, WorkerConfig(max_tokens_per_microbatch=40))
        wl.forward_backward(batch)
        q.put((rank, bool(torch.equal(grads[True], grads[False])), wl.opt.main_grad.numpy(), grads[True].numpy()))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(240)
def test_overlapped_reduction_equals_reduction_after_backward():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        r, same, local, summed = q.get(timeout=120)
        got[r] = (same, torch.from_numpy(local), torch.from_numpy(summed))
    for p in procs:
        p.join(timeout=60)
    assert got[0][0] and got[1][0]
    assert torch.equal(got[0][2], got[1][2])                                   # both ranks hold the same sum
    assert torch.allclose(got[0][2], got[0][1] + got[1][1], atol=1e-6)         # and it is the sum of the local gradients
