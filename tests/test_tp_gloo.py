"""Tensor-parallel invariance without a GPU: a TP=2 model on two gloo ranks (CPU kernels, fp32)
produces the same logprobs, bit for bit, as the TP=1 model with the same weights, for the dense,
MoE and hybrid families; its gradients match too (to fp32 tolerance), and a TP=1 checkpoint
loads into the TP=2 layout."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="2")
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=2)
    try:
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.models.decoder import DecoderLM
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
        from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

        ps2 = ParallelState.build(tp=2)
        out = {}
        for name in ("tiny-qwen3", "tiny-moe", "tiny-hybrid", "tiny-mla", "tiny-deepseek"):
            cfg = get_config(name, tp_invariant=True)
            g = torch.Generator().manual_seed(1)
            prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (20, 33, 9)]
            resps = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (12, 7, 15)]
            seq, att, rmask = build_sequences(prompts, resps)
            adv = torch.randn(rmask.shape, generator=g) / rmask.sum()

            def run(ps):
                model = DecoderLM(cfg, ps, seed=3)
                w = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=64))
                b = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                        "advantages": adv.clone()})
                lp = w.forward(b)
                b["action_log_probs"] = lp - 0.05          # off-policy on purpose so the gradient is not trivial
                w.forward_backward(b)
                w.reduce_gradients()
                gsq = float(w.opt.grad_sq_norm(ps))
                return lp, gsq, model

            lp2, g2, m2 = run(ps2)
            # Hugging Face export from the tensor-parallel model (a collective over the TP group) and import back
            from skyrl_isoexec_b200.models import hf_export

            hf2 = hf_export.to_hf_state_dict(m2)
            if rank == 0:
                lp1, g1, m1 = run(ParallelState.single())
                hf1 = hf_export.to_hf_state_dict(m1)
                same_export = sorted(hf1) == sorted(hf2) and all(torch.equal(hf1[k], hf2[k]) for k in hf1)
                out[name] = (int((lp1.view(torch.int32) != lp2.view(torch.int32)).sum()), g1, g2, same_export)
            else:
                out[name] = None
            import tempfile

            d = tempfile.gettempdir() + f"/hf_tp_{port}_{name}"
            hf_export.save_hf(m2, d, write=rank == 0)
            dist.barrier()
            m3 = DecoderLM(cfg, ps2, seed=99)
            hf_export.load_hf(m3, d)
            assert torch.equal(m3.store.flat, m2.store.flat), f"{name}: import into TP shards differs on rank {rank}"
        if rank == 0:
            q.put(out)
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(900)
def test_tp2_equals_tp1_bitwise_on_cpu():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
    for name, (mism, g1, g2, same_export) in out.items():
        assert mism == 0, f"{name}: {mism} logprob bits differ between TP=1 and TP=2"
        assert same_export, f"{name}: the export gathered from TP=2 differs from the TP=1 export"
        assert abs(g1 - g2) <= 2e-3 * max(g1, 1e-12), f"{name}: grad norms {g1} vs {g2}"
