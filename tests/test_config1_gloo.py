"""The CPU/gloo configuration: trainer (rank 0) and rollout engine (rank 1) as SEPARATE processes,
tiny Qwen3-style fp32 decoder, GRPO with 8 prompts x 4 samples, 32-token prompts, up to 64-token
responses at temperature 1, reward = fraction of even token ids. Asserts that the contract hashes
agree, that rollout and trainer logprobs are bitwise equal before and after a policy update +
weight broadcast, and that a corrupted hash makes both sides refuse."""
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


def _worker(rank, port, negative, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="2")
    if negative and rank == 0:
        os.environ["ISOEXEC_HANDSHAKE_NEGATIVE_CONTROL"] = "1"
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=2)
    from skyrl_isoexec_b200.core import process as P
    from skyrl_isoexec_b200.core.adapter import ContractAdapter
    from skyrl_isoexec_b200.core.testing import count_bit_mismatches
    from skyrl_isoexec_b200.engine.interface import NativeInferenceEngine
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.remote import DistEngineClient, DistEngineServer
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.sync import strategies as S
    from skyrl_isoexec_b200.train import algorithms as alg
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    cfg = get_config("tiny-qwen3")
    try:
        if rank == 1:
            # rollout process: different init seed on purpose; the weights must arrive by sync
            model = DecoderLM(cfg, seed=123)
            ContractAdapter("engine", model, rank).run_install()
            eng = NativeInferenceEngine(LLMEngine(model, EngineConfig(max_num_seqs=32, num_kv_pages=64, seed=5)))
            try:
                DistEngineServer(eng, client_rank=0).serve()
                q.put((rank, "served", P.contract_hash()))
            except P.ContractMismatch as e:
                q.put((rank, "refused", str(e)))
            return
        model = DecoderLM(cfg, seed=0)
        ad = ContractAdapter("trainer", model, rank)
        ad.run_install()
        worker = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=2048))
        worker.cfg.optimizer.lr = 1e-3
        client = DistEngineClient(server_rank=1)
        info = S.create_init_info("broadcast", group_ranks=[0, 1], src_rank=0)
        import asyncio

        try:
            asyncio.run(client.init_weight_update_communicator(info))
        except P.ContractMismatch as e:
            q.put((rank, "refused", str(e)))
            return
        sender = S.create_sender(info, model)

        def sync():
            asyncio.run(client.update_named_weights(None, send_fn=lambda: sender.send_chunks(S.extract_native_weights(model))))

        sync()
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (32,), generator=g).tolist() for _ in range(8)]
        results = []
        for _round in range(2):
            rep = [p for p in prompts for _ in range(4)]
            out = asyncio.run(client.generate({"prompt_token_ids": rep, "sampling_params": {"max_generate_length": 64, "ignore_eos": True}}))
            seq, att, rmask = build_sequences(rep, out["response_ids"])
            rewards = torch.zeros_like(rmask)
            for i, r in enumerate(out["response_ids"]):
                rewards[i, len(r) - 1] = sum(1 for t in r if t % 2 == 0) / len(r)
            batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                        "rewards": rewards})
            lp = worker.forward(batch)
            ro = torch.zeros_like(lp)
            for i, l in enumerate(out["response_logprobs"]):
                ro[i, :len(l)] = torch.tensor(l)
            mism = count_bit_mismatches((lp * rmask).contiguous(), (ro * rmask).contiguous())
            uids = [f"p{i // 4}" for i in range(32)]
            adv, _ = alg.compute_advantages_and_returns(rewards, rmask, uids, "grpo", alg.AlgorithmConfig())
            batch["advantages"] = adv / rmask.sum()
            batch["action_log_probs"] = lp
            batch["rollout_logprobs"] = ro
            m = worker.forward_backward(batch)
            gn = worker.optim_step()
            sync()
            results.append((mism, int(rmask.sum()), gn, float(rewards.sum(-1).mean())))
        asyncio.run(client.teardown())
        q.put((rank, "done", P.contract_hash(), results))
    finally:
        dist.destroy_process_group()


def _run(negative):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, negative, q)) for r in range(2)]
    for p in procs:
        p.start()
    msgs = {}
    for _ in range(2):
        m = q.get(timeout=600)
        msgs[m[0]] = m[1:]
    for p in procs:
        p.join(timeout=60)
    return msgs


@pytest.mark.timeout(900)
def test_trainer_and_rollout_processes_agree_bitwise():
    msgs = _run(negative=False)
    assert msgs[0][0] == "done" and msgs[1][0] == "served"
    assert msgs[0][1] == msgs[1][1]                       # contract hashes match across the two processes
    for mism, ntok, gn, reward in msgs[0][2]:
        assert ntok == 32 * 64 and mism == 0              # every response token's logprob is bit-identical
        assert gn > 0 and 0.3 < reward < 0.7


@pytest.mark.timeout(300)
def test_handshake_negative_control_refuses_on_both_sides():
    msgs = _run(negative=True)
    assert msgs[0][0] == "refused" and msgs[1][0] == "refused"
    assert "mismatch" in msgs[0][1].lower()
