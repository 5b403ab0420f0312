"""Trainer and rollout engines with DIFFERENT tensor-parallel layouts in one colocated job (gloo ranks on CPU):

  * world 2: trainer TP2 feeds two TP1 engines;
  * world 4: trainer TP2 x DP2 feeds four TP1 engines, and trainer TP4 (KV heads replicated) feeds two TP2 engines.

Each GRPO step reshards the updated weights into the engines' own buffers (sync/reshard.py), the engines of one trainer
replica split its requests, and the rollout logprobs must equal the trainer's scoring forward bit for bit although the
two sides reduce over different numbers of ranks."""
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


def _worker(rank, world, port, tp_t, tp_e, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
        from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

        kv = get_config("tiny-qwen3").num_kv_heads
        ps = ParallelState.build(tp=tp_t, kv_rep=max(1, tp_t // kv))
        cfg = SkyRLTrainConfig.from_cli_overrides([
            "trainer.policy.model=tiny-qwen3", f"trainer.train_batch_size={2 * ps.dp}", f"trainer.policy_mini_batch_size={2 * ps.dp}",
            "generator.n_samples_per_prompt=4", "generator.sampling_params.max_generate_length=12",
            "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=10", "data.synthetic_prompts=32",
            "trainer.max_prompt_length=10", "generator.inference_engine.num_kv_pages=16", "trainer.policy.optimizer_config.lr=1e-2",
            "trainer.logger=jsonl", f"generator.inference_engine.tensor_parallel_size={tp_e}"])
        tr = RayPPOTrainer(cfg, ps=ps, device="cpu")
        tr.build_models()
        assert tr.separate_engine and tr.engine.model is not tr.policy.model and tr.engine.model.ps.tp == tp_e
        assert tr.policy.model.cfg.tp_invariant
        tr.sync_weights()
        it = iter(tr.loader)
        mism, moved, w0 = [], [], tr.policy.model.store.flat.clone()
        for _ in range(2):
            m = tr.train_step(next(it))
            mism.append(int(m["policy/rollout_train_logprob_bit_mismatches"]))
            moved.append(int(m["sync/bytes"]))
            assert m["generate/response_tokens"] == 2 * 4 * 12
        changed = not torch.equal(w0, tr.policy.model.store.flat)
        # the engine's shard after the last sync equals a direct slice of the trainer's full weights
        from skyrl_isoexec_b200.models.decoder import shard_of
        from skyrl_isoexec_b200.sync.strategies import gather_full

        ok = True
        for name, t in tr.policy.model.named_weights():
            spec = tr.policy.model.store.specs[name]
            full = gather_full(t, spec, ps) if (spec.shard_dim is not None and ps.tp > 1) else t
            es = tr.engine.model.store.specs[name]
            want = shard_of(full, es, tr.engine_ps.tp_rank, tr.engine_ps.tp)
            ok = ok and torch.equal(want, tr.engine.model.store.views[name])
        q.put((rank, mism, moved, changed, ok, tr.engines_per_replica))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


def _run(world, tp_t, tp_e):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, tp_t, tp_e, q)) for r in range(world)]
    for p in procs:
        p.start()
    res, t0 = [], time.time()
    while len(res) < world and time.time() - t0 < 500:
        try:
            res.append(q.get(timeout=2))
        except _q.Empty:
            assert all(p.is_alive() or p.exitcode == 0 for p in procs), "a rank died"
    for p in procs:
        p.join(timeout=60)
    assert len(res) == world
    for rank, mism, moved, changed, ok, k in sorted(res):
        assert mism == [0, 0], (rank, mism)
        assert changed and ok and k == tp_t // tp_e and all(b > 0 for b in moved)


@pytest.mark.timeout(600)
def test_trainer_tp2_feeds_two_tp1_engines_bitwise():
    _run(2, 2, 1)


@pytest.mark.timeout(600)
def test_trainer_tp2_dp2_feeds_four_tp1_engines_bitwise():
    _run(4, 2, 1)


@pytest.mark.timeout(600)
def test_trainer_tp4_with_replicated_kv_feeds_two_tp2_engines_bitwise():
    _run(4, 4, 2)
