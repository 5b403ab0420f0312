"""More tensor-parallel ranks than KV heads (tp = 4, two KV heads: pairs of ranks share a head). Four gloo ranks on CPU:
logprobs equal the TP = 1 model bit for bit, the gradient norm agrees, replicated k|v rows stay identical after an
optimizer step, the gathered weights equal the TP = 1 weights after its step, and a checkpoint saved at TP = 4
reshards to TP = 1."""
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


def _worker(rank, port, q, tmp, gate):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="4")
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=4)
    try:
        from skyrl_isoexec_b200.models import hf_export
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.models.decoder import DecoderLM, kv_rows
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train import checkpoint as ckpt
        from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
        from skyrl_isoexec_b200.train.policy_worker import OptimizerConfig, PolicyWorker, WorkerConfig

        cfg = get_config("tiny-qwen3", tp_invariant=True, attn_output_gate=gate)      # 4 query heads, 2 KV heads
        ps4 = ParallelState.build(tp=4, kv_rep=2)
        assert ps4.kvr_ranks == [2 * (rank // 2), 2 * (rank // 2) + 1] and ps4.kvr_rank == rank % 2
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (20, 33, 9)]
        resps = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (12, 7, 15)]
        seq, att, rmask = build_sequences(prompts, resps)
        adv = torch.randn(rmask.shape, generator=g) / rmask.sum()

        def run(ps):
            model = DecoderLM(cfg, ps, seed=3)
            w = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=64, optimizer=OptimizerConfig(lr=1e-2, eps=1e-2, max_grad_norm=0.0)))     # a large eps keeps Adam's first step
            # smooth in the gradient, so fp32 noise in near-zero gradients stays noise in the weights
            b = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                    "advantages": adv.clone()})
            lp = w.forward(b)
            b["action_log_probs"] = lp - 0.05
            w.forward_backward(b)
            w.reduce_gradients()
            gsq = float(w.opt.grad_sq_norm(ps))
            w.opt.step(ps)
            return lp, gsq, model, w

        lp4, g4, m4, w4 = run(ps4)
        assert m4.hq == 1 and m4.hkv == 1 and m4.kv_rep == 2
        # the two ranks of a sharing group hold the same k|v rows after the step
        spec = m4.store.specs["layers.0.attn.qkv.weight"]
        r0, nr = kv_rows(spec)
        mine = m4.p("layers.0.attn.qkv.weight").detach()[r0:r0 + nr].contiguous()
        both = [torch.empty_like(mine) for _ in range(2)]
        dist.all_gather(both, mine, group=ps4.kvr_group)
        kv_same = bool(torch.equal(both[0], both[1]))
        # the rollout engine on the same tensor-parallel model: one KV head per rank in its paged cache, and the sampled
        # tokens' logprobs equal a trainer forward bit for bit
        from skyrl_isoexec_b200.core.testing import count_bit_mismatches
        from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
        from skyrl_isoexec_b200.engine.sampler import SamplingParams

        eng = LLMEngine(m4, EngineConfig(max_num_seqs=4, num_kv_pages=16, max_num_batched_tokens=128, seed=9))
        outs = eng.generate(prompts, SamplingParams(max_generate_length=6, ignore_eos=True))
        seq_e, att_e, rm_e = build_sequences([o.prompt_ids for o in outs], [o.response_ids for o in outs])
        lp_e = w4.forward(TrainingInputBatch({"sequences": seq_e, "attention_mask": att_e, "response_mask": rm_e}))
        ro = torch.zeros_like(lp_e)
        for i, o in enumerate(outs):
            ro[i, :len(o.response_logprobs)] = torch.tensor(o.response_logprobs)
        engine_mism = count_bit_mismatches((lp_e * rm_e).contiguous(), (ro * rm_e).contiguous())
        hf4 = hf_export.to_hf_state_dict(m4)                          # gathers (collective over the TP group)
        ckpt.save_checkpoint(tmp, 1, w4, {}, {"global_step": 1}, ps4)
        res = None
        if rank == 0:
            single = ParallelState.single()
            lp1, g1, m1, w1 = run(single)
            hf1 = hf_export.to_hf_state_dict(m1)
            worst = max(float((hf1[k].float() - hf4[k].float()).abs().max()) for k in hf1)
            m_r = DecoderLM(cfg, single, seed=99)
            w_r = PolicyWorker(m_r, WorkerConfig())
            ckpt.load_checkpoint(ckpt.step_dir(tmp, 1), w_r, single)
            resharded = bool(torch.equal(hf_export.to_hf_state_dict(m_r)["model.layers.0.self_attn.k_proj.weight"],
                                         hf4["model.layers.0.self_attn.k_proj.weight"]))
            res = (int((lp1.view(torch.int32) != lp4.view(torch.int32)).sum()), g1, g4, worst, sorted(hf1) == sorted(hf4), resharded)
        q.put((rank, kv_same and engine_mism == 0, res))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(600)
@pytest.mark.parametrize("gate", [False, True])          # plain query heads, and [q | output gate] blocks per head
def test_tp4_with_two_kv_heads_equals_tp1(tmp_path, gate):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, q, str(tmp_path), gate)) for r in range(4)]
    for p in procs:
        p.start()
    got = [q.get(timeout=400) for _ in range(4)]
    for p in procs:
        p.join(timeout=60)
    assert all(kv_same for _, kv_same, _ in got)
    (mism, g1, g4, worst, same_keys, resharded), = [r for _, _, r in got if r is not None]
    assert mism == 0, f"{mism} logprob bits differ between TP=1 and TP=4 with replicated KV heads"
    assert abs(g1 - g4) <= 2e-3 * max(g1, 1e-12), (g1, g4)
    assert same_keys and worst < 1e-5, worst
    assert resharded
