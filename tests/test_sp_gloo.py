"""Sequence parallelism on CPU/gloo: with the residual stream, norms and adds cut over the tensor-parallel ranks the
trainer's log-probabilities keep their bits (TP = 2 with and without it, and TP = 1), the gradients agree, uneven row
counts and recomputed layers work, and the norm weights' partial gradients are summed over the group."""
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

    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.models.decoder import DecoderLM
        from skyrl_isoexec_b200.parallel import tp as tp_ops
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
        from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

        ps = ParallelState.build(tp=world)
        assert [tp_ops.sp_rows(7, ps_) for ps_ in [ps]][0] == ((0, 3) if rank == 0 else (3, 7))      # the remainder goes to the last rank
        g = torch.Generator().manual_seed(1)
        out = {}
        for ckpt in (False, True):
            res = {}
            for sp in (False, True):
                cfg = get_config("tiny-qwen3", tp_invariant=True, sequence_parallel=sp)
                prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(2)).tolist() for n in (20, 33, 9)]
                resps = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(3)).tolist() for n in (12, 7, 14)]
                seq, att, rmask = build_sequences(prompts, resps)          # 95 tokens: an odd number of rows per micro-batch
                adv = torch.randn(rmask.shape, generator=torch.Generator().manual_seed(4)) / rmask.sum()
                model = DecoderLM(cfg, ps, seed=3)
                w = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=64, checkpoint_layers=ckpt))
                b = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                        "advantages": adv.clone()})
                lp = w.forward(b)
                b["action_log_probs"] = lp - 0.05
                w.forward_backward(b)
                w.reduce_gradients()
                grads = {n: w.opt.main_grad[s.offset:s.offset + v.numel()].view(v.shape).clone()
                         for n, v in model.named_weights() for s in [model.store.specs[n]]}
                res[sp] = (lp, grads)
            same_lp = bool(torch.equal(res[False][0].view(torch.int32), res[True][0].view(torch.int32)))
            worst = max(float((res[False][1][n] - res[True][1][n]).abs().max() / res[False][1][n].abs().max().clamp(min=1e-8))
                        for n in res[False][1])
            out[ckpt] = (same_lp, worst)
        q.put((rank, out, res[True][0].numpy()))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(400)
def test_sequence_parallel_keeps_the_logprob_bits_and_the_gradients():
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        r, out, lp = q.get(timeout=300)
        got[r] = (out, torch.from_numpy(lp))
    for p in procs:
        p.join(timeout=60)
    for r in (0, 1):
        for ckpt in (False, True):
            same_lp, worst = got[r][0][ckpt]
            assert same_lp, f"rank {r}, recompute={ckpt}: sequence parallelism changed the log-probability bits"
            assert worst < 2e-4, f"rank {r}, recompute={ckpt}: gradients differ by {worst}"
    # and against a single rank
    cfg = get_config("tiny-qwen3", tp_invariant=True)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(2)).tolist() for n in (20, 33, 9)]
    resps = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(3)).tolist() for n in (12, 7, 14)]
    seq, att, rmask = build_sequences(prompts, resps)
    w = PolicyWorker(DecoderLM(cfg, seed=3), WorkerConfig(max_tokens_per_microbatch=64))
    lp1 = w.forward(TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask}))
    assert torch.equal(lp1.view(torch.int32), got[0][1].view(torch.int32))
