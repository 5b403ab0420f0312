"""Length-balanced data parallelism on CPU/gloo: ranks whose rollouts differ a lot in length pool them and deal whole
prompt groups back out; every rank ends with the same number of groups, about the same number of tokens, no sample
lost or duplicated, and the training step runs on the regrouped batch."""
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


def _worker(rank, world, port, q, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
        from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

        ps = ParallelState.build()
        ov = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=8", "trainer.policy_mini_batch_size=8",
              "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=24", "data.synthetic_prompt_len=10",
              "trainer.num_steps=1", "trainer.logger=jsonl", f"trainer.ckpt_path={tmp}/r{rank}", "trainer.ckpt_interval=0",
              "environment.env_class=even_tokens", "trainer.balance_dp_by_length=true"]
        tr = RayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(ov), ps=ps, device="cpu")
        tr.build_models()
        # a rollout whose lengths depend on the rank: rank 0 short, rank 1 long (what balancing is for)
        g = torch.Generator().manual_seed(rank)
        n_resp = [3, 4, 2, 3, 3, 2, 4, 3] if rank == 0 else [24, 20, 22, 24, 18, 24, 21, 23]
        go = {"prompt_token_ids": [[1 + rank, 2, 3]] * 8, "response_ids": [torch.randint(5, 900, (n,), generator=g).tolist() for n in n_resp],
              "rewards": [float(i % 2) for i in range(8)], "loss_masks": [[1] * n for n in n_resp], "stop_reasons": ["length"] * 8,
              "rollout_logprobs": [[-1.0] * n for n in n_resp], "rollout_metrics": {}}
        uids = [f"p{i // 2}" for i in range(8)]
        go2, uids2 = tr.balance_rollouts(go, uids)
        toks = sum(len(p) + len(r) for p, r in zip(go2["prompt_token_ids"], go2["response_ids"]))
        groups = {}
        for u, p, r in zip(uids2, go2["prompt_token_ids"], go2["response_ids"]):
            groups.setdefault(u, []).append((tuple(p), tuple(r)))
        batch = tr.convert_to_training_input(go2, uids2)
        q.put((rank, toks, {k: v for k, v in groups.items()}, tr.all_metrics["generate/dp_token_imbalance_before"],
               tr.all_metrics["generate/dp_token_imbalance_after"], tuple(batch["sequences"].shape),
               [(tuple(p), tuple(r)) for p, r in zip(go["prompt_token_ids"], go["response_ids"])]))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(300)
def test_rollouts_are_regrouped_by_length_over_the_data_parallel_ranks(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        r = q.get(timeout=200)
        got[r[0]] = r
    for p in procs:
        p.join(timeout=60)
    t0, t1 = got[0][1], got[1][1]
    assert abs(t0 - t1) / max(t0, t1) < 0.15 and got[0][3] > 1.5 and got[0][4] < 1.1          # 1.6x skew before, balanced after
    assert all(len(v) == 2 for g in (got[0][2], got[1][2]) for v in g.values())               # groups stayed whole
    assert len(got[0][2]) == len(got[1][2]) == 4                                              # same number of groups per rank
    before = sorted(got[0][6] + got[1][6])
    after = sorted(s for g in (got[0][2], got[1][2]) for v in g.values() for s in v)
    assert before == after                                                                    # nothing lost, nothing twice
    assert got[0][5][0] == got[1][5][0] == 8
