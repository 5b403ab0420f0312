"""Expert parallelism end to end on CPU/gloo: a GRPO loop at EP=2 (each rank its own prompts, experts split over the
two ranks, engine steps and trainer micro-batches in lockstep) keeps rollout == trainer logprobs bit for bit."""
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

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
        from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

        ps = ParallelState.build(ep=world)
        assert ps.dp == world and ps.ep == world and ps.edp_group is None
        # rank 1 generates longer responses than rank 0: its engine keeps stepping while rank 0 idles in lockstep
        cfg = SkyRLTrainConfig.from_cli_overrides([
            "trainer.policy.model=tiny-moe", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
            "generator.n_samples_per_prompt=2", f"generator.sampling_params.max_generate_length={10 + 6 * rank}",
            "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=12", "data.synthetic_prompts=32",
            "trainer.max_prompt_length=12", "generator.inference_engine.num_kv_pages=32", "trainer.policy.optimizer_config.lr=1e-3",
            "trainer.num_steps=2", f"trainer.ckpt_path={tmp}/r{rank}", "trainer.ckpt_interval=0", "trainer.logger=jsonl",
            f"trainer.max_tokens_per_microbatch={40 if rank == 0 else 4096}"])        # rank 0 cuts more micro-batches than rank 1 would
        tr = RayPPOTrainer(cfg, ps=ps, device="cpu")
        tr.build_models()
        tr.sync_weights()
        it = iter(tr.loader)
        m1 = tr.train_step(next(it))
        m2 = tr.train_step(next(it))
        # Hugging Face export: every rank contributes its experts, the result has all of them and both ranks agree
        from skyrl_isoexec_b200.models import hf_export

        sd = hf_export.to_hf_state_dict(tr.policy.model)
        n_exp = len([k for k in sd if k.startswith("model.layers.0.mlp.experts.") and k.endswith("down_proj.weight")])
        mine = tr.policy.model.p("layers.0.moe.experts.down").detach()
        per = mine.shape[0]
        own_ok = all(torch.equal(sd[f"model.layers.0.mlp.experts.{rank * per + e}.down_proj.weight"], mine[e]) for e in range(per))
        digest = float(sum(v.double().sum() for v in sd.values()))
        # ... and the import cuts the full expert stack back to this rank's experts
        hf_export.save_hf(tr.policy.model, f"{tmp}/hf", write=rank == 0)
        dist.barrier()
        before = tr.policy.model.store.flat.detach().clone()
        tr.policy.model.store.flat.detach().zero_()
        hf_export.load_hf(tr.policy.model, f"{tmp}/hf")
        own_ok = own_ok and bool(torch.equal(tr.policy.model.store.flat.detach(), before))
        q.put((rank, m1["policy/rollout_train_logprob_bit_mismatches"], m2["policy/rollout_train_logprob_bit_mismatches"],
               m1["policy/grad_norm"], m2["policy/grad_norm"], int(tr.engine.stats["steps"]), n_exp, own_ok, digest))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(300)
def test_grpo_loop_with_expert_parallelism(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        r = q.get(timeout=240)
        got[r[0]] = r[1:]
    for p in procs:
        p.join(timeout=60)
    for r in (0, 1):
        assert got[r][0] == 0 and got[r][1] == 0
    assert got[0][2] == got[1][2] > 0 and got[0][3] == got[1][3] > 0          # one global gradient norm, seen by both
    assert got[0][5] == got[1][5] == 8 and got[0][6] and got[1][6] and got[0][7] == got[1][7]     # export: all 8 experts, same on both
