"""Pipeline parallelism on CPU/gloo: two stages reproduce the single-stage logprobs and gradients."""
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


def _batch():
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (9, 14, 7, 11, 12, 6)]
    resp = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (10, 6, 12, 8, 5, 9)]
    seq, att, rmask = build_sequences(prompts, resp)
    B, R = rmask.shape
    return TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                               "advantages": torch.randn(B, R, generator=g), "rollout_logprobs": torch.zeros(B, R)})


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.parallel.pp import PipelinePolicyWorker, build_stage_model, stage_layers
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.policy_worker import WorkerConfig

        ps = ParallelState.build(pp=world)
        cfg = get_config("tiny-qwen3", num_layers=3)
        assert [len(stage_layers(3, 2, r)) for r in range(2)] == [2, 1]
        model = build_stage_model(cfg, ps, "cpu", seed=5)
        w = PipelinePolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=48))      # several micro-batches -> 1F1B
        b = _batch()
        lp = w.forward(b)
        b["action_log_probs"] = lp
        m = w.forward_backward(b)
        w.reduce_gradients()
        grads = {n: w.opt.main_grad[s.offset:s.offset + v.numel()].view(v.shape).clone()
                 for n, v in model.named_weights() for s in [model.store.specs[n]]}
        q.put((rank, lp.numpy(), m["policy_loss"], {n: g.numpy() for n, g in grads.items()}))   # by value: the child may exit first
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(240)
def test_two_stage_pipeline_equals_single_stage():
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(2):
        r, lp, loss, grads = q.get(timeout=200)
        got[r] = (torch.from_numpy(lp), loss, {n: torch.from_numpy(g) for n, g in grads.items()})
    for p in procs:
        p.join(timeout=60)
    ref_model = DecoderLM(get_config("tiny-qwen3", num_layers=3), seed=5)
    ref = PolicyWorker(ref_model, WorkerConfig(max_tokens_per_microbatch=48))
    b = _batch()
    lp = ref.forward(b)
    b["action_log_probs"] = lp
    m = ref.forward_backward(b)
    assert torch.equal(got[0][0], lp) and torch.equal(got[1][0], lp)            # same kernels, same order: same bits
    assert abs(got[1][1] - m["policy_loss"]) < 1e-5 and got[0][1] == got[1][1]
    ref_grads = {n: ref.opt.main_grad[s.offset:s.offset + v.numel()].view(v.shape) for n, v in ref_model.named_weights()
                 for s in [ref_model.store.specs[n]]}
    seen = set()
    for r in (0, 1):
        for n, g in got[r][2].items():
            assert torch.allclose(g, ref_grads[n], atol=1e-5, rtol=1e-4), n
            seen.add(n)
    assert seen == set(ref_grads)
