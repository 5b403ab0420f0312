"""Flag table, lifecycle ordering checks, dataset/packing/replay helpers, SFT, evaluation, the
fully-asynchronous trainer and the entry point, all on CPU."""
import json
import threading

import pytest
import torch

from skyrl_isoexec_b200.core import flags, lifecycle
from skyrl_isoexec_b200.train import dataset as D
from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
from skyrl_isoexec_b200.train.evaluate import evaluate, pass_at_k
from skyrl_isoexec_b200.train.fully_async_trainer import (AsyncConfig, AsyncPromptSource, FullyAsyncTrainer, GenerationGroupQueue,
                                                           StalenessManager)
from skyrl_isoexec_b200.train.sft_trainer import SFTConfig, SFTTrainer
from skyrl_isoexec_b200.train.trainer import RayPPOTrainer


def test_flag_table_is_consistent_and_detects_split_brain():
    assert flags.check_table() == []
    snap = flags.snapshot({})
    assert set(snap) == {f.name for f in flags.FLAGS}
    fn = flags.function_flags()
    assert fn and all(f.selects for f in fn)
    both = [f for f in fn if flags.TRAIN in f.sides and flags.ENGINE in f.sides]
    assert both, "at least one function flag is read by both sides"
    f = both[0]
    other = "1" if f.get({}) != "1" else "0"
    out = flags.latent_split_brain({}, {f.name: other})
    assert len(out) == 1 and f.name in out[0]
    assert flags.latent_split_brain({f.name: other}, {f.name: other}) == []
    assert f.name in flags.actor_forwarding_list(flags.ENGINE)


def test_lifecycle_checks_flag_wrong_orders():
    good = lifecycle.LifecycleLog()
    for name, d in (("handshake_ok", {}), ("engine_wake", {"tags": ["weights"]}), ("sync_begin", {}), ("weight_sync", {}),
                    ("sync_end", {}), ("state_invalidated", {}), ("engine_wake", {"tags": ["kv_cache"]}), ("generate", {}),
                    ("engine_sleep", {"level": 1})):
        good.add(name, **d)
    assert lifecycle.run_all(good) == []
    bad = lifecycle.LifecycleLog()
    for name, d in (("engine_sleep", {"level": 2}), ("sync_begin", {}), ("weight_sync", {}), ("generate", {}), ("handshake_ok", {})):
        bad.add(name, **d)
    errs = lifecycle.run_all(bad)
    # asleep during sync, transfer still open at generate, state not invalidated, handshake after the first sync
    assert len(errs) == 4, errs
    dropped = lifecycle.LifecycleLog()
    dropped.add("engine_sleep", level=2)
    dropped.add("generate")
    assert lifecycle.check_sleep_tag_scoping(dropped)


def test_packing_boundaries_and_replay_buffer():
    lens = [700, 300, 300, 200, 512, 100, 50]
    bins = D.pack_first_fit_decreasing(lens, 1024)
    assert sorted(i for b in bins for i in b) == list(range(len(lens)))
    assert all(sum(lens[i] for i in b) <= 1024 for b in bins) and len(bins) == 3
    assert D.pack_first_fit_decreasing([2000, 10], 1024) == [[0], [1]]      # an oversize sequence gets its own bin
    bal = D.pack_balanced(lens, 2)
    loads = [sum(lens[i] for i in b) for b in bal]
    assert sorted(i for b in bal for i in b) == list(range(len(lens))) and abs(loads[0] - loads[1]) <= 200
    uids = ["a", "a", "b", "b", "b", "c"]
    assert D.compute_prompt_boundaries(uids) == [(0, 2), (2, 5), (5, 6)]
    assert D.compute_prompt_mini_batch_boundaries(uids, 2) == [(0, 5), (5, 6)]
    rb = D.ReplayBuffer(capacity=4, max_staleness=1)
    for v, item in enumerate("wxyz"):
        rb.add(item, version=v)
    rb.add("q", version=3)                 # over capacity: the oldest goes
    assert len(rb) == 4
    assert rb.evict_stale(current_version=3) == 1   # versions 1 is staler than 1 step; 2, 3, 3 stay
    got = rb.pop_batch(2, current_version=3)
    assert got == [("y", 2), ("z", 3)] and len(rb) == 1


def test_prompt_dataset_reads_jsonl_and_filters(tmp_path):
    p = tmp_path / "train.jsonl"
    rows = [{"prompt": list(range(5)), "env_class": "even_tokens"}, {"prompt": list(range(50)), "env_class": "even_tokens"},
            {"prompt": [1, 2, 3], "reward_spec": {"ground_truth": "7"}}]
    p.write_text("\n".join(json.dumps(r) for r in rows))
    ds = D.PromptDataset([str(p)], max_prompt_length=10, env_class="gsm8k")
    assert len(ds) == 2
    assert ds[0]["env_class"] == "even_tokens" and ds[1]["env_class"] == "gsm8k"
    assert ds[0]["uid"] != ds[1]["uid"]


def test_pass_at_k_matches_closed_forms():
    assert pass_at_k(10, 0, 1) == 0.0 and pass_at_k(10, 10, 3) == 1.0
    assert abs(pass_at_k(10, 3, 1) - 0.3) < 1e-12
    assert abs(pass_at_k(4, 2, 2) - (1 - (2 / 4) * (1 / 3))) < 1e-12


def _rl_cfg(tmp, steps, *extra):
    return SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
        "generator.n_samples_per_prompt=4", "generator.sampling_params.max_generate_length=16",
        "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=12", "data.synthetic_prompts=32",
        "trainer.max_prompt_length=12", "generator.inference_engine.num_kv_pages=64",
        "trainer.policy.optimizer_config.lr=1e-3", f"trainer.num_steps={steps}", f"trainer.ckpt_path={tmp}",
        "trainer.ckpt_interval=0", "trainer.logger=jsonl", *extra])


def test_evaluate_reports_reward_and_pass_at_k(tmp_path):
    tr = RayPPOTrainer(_rl_cfg(str(tmp_path), 1, "trainer.dump_eval_results=true", "trainer.eval_batch_size=3"), device="cpu")
    tr.build_models()
    tr.sync_weights()
    ev = tr.eval()
    import json as _json

    lines = [_json.loads(x) for x in open(tmp_path / "dumped_evals" / "global_step_0.jsonl")]
    assert len(lines) == 3 * max(1, tr.cfg.generator.eval_n_samples_per_prompt) and {"uid", "env_class", "prompt_ids", "response_ids", "reward", "stop_reason"} <= set(lines[0])
    assert abs(sum(x["reward"] for x in lines) / len(lines) - ev["eval/avg_reward"]) < 1e-9
    tr.engine.wake_up()
    rows = [tr.dataset[i] for i in range(3)]
    out = evaluate(tr.generator, rows, {"max_generate_length": 8, "ignore_eos": True}, n_samples=4, ks=(1, 4))
    assert out["eval/num_prompts"] == 3 and out["eval/avg_response_length"] == 8
    assert 0.0 <= out["eval/pass_at_1"] <= out["eval/pass_at_4"] <= 1.0


def test_sft_lowers_the_loss_on_a_fixed_batch():
    g = torch.Generator().manual_seed(0)
    ex = [{"prompt_ids": torch.randint(0, 200, (6,), generator=g).tolist(),
           "response_ids": torch.randint(0, 200, (10,), generator=g).tolist()} for _ in range(8)]
    cfg = SFTConfig(model="tiny-qwen3", batch_size=8, logger="jsonl")
    cfg.optimizer.lr = 3e-3
    cfg.optimizer.num_warmup_steps = 0
    tr = SFTTrainer(cfg, ex, device="cpu")
    losses = [tr.train_step(ex)["sft/loss"] for _ in range(6)]
    assert losses[-1] < losses[0] * 0.9, losses
    assert tr.global_step == 6


def test_staleness_manager_bounds_rollouts_in_flight():
    sm = StalenessManager(max_staleness_steps=1, mini_batch_prompts=2)
    assert sm.capacity == 4
    assert all(sm.acquire(timeout=0.0) for _ in range(4))
    assert not sm.acquire(timeout=0.01)
    sm.finished()
    sm.finished()
    assert not sm.acquire(timeout=0.01)          # buffered groups still count against the budget
    sm.consumed(2)
    assert sm.acquire(timeout=0.0) and sm.acquire(timeout=0.0) and not sm.acquire(timeout=0.0)
    q = GenerationGroupQueue()
    t = threading.Timer(0.05, lambda: [q.put(1), q.put(2)])
    t.start()
    assert q.get_many(2, timeout=2.0) == [1, 2]
    with pytest.raises(TimeoutError):
        q.get_many(1, timeout=0.01)
    src = AsyncPromptSource([{"uid": i} for i in range(3)])
    assert [src.next()["uid"] for _ in range(4)] == [0, 1, 2, 0] and src.epoch == 1
    src.mark_consumed(1)
    sd = src.state_dict()
    src2 = AsyncPromptSource([{"uid": i} for i in range(3)])
    src2.load_state_dict(sd)
    assert src2.cursor == 1 and src2.consumed == {1}


def test_fully_async_trainer_runs_with_bounded_staleness(tmp_path):
    cfg = _rl_cfg(str(tmp_path), 3, "trainer.isoexec.strict=false")
    tr = FullyAsyncTrainer(cfg, AsyncConfig(max_staleness_steps=1, num_parallel_generation_workers=3, mini_batch_prompts=4), device="cpu")
    tr.train()
    assert tr.global_step == 3 and tr.stale.version == 3
    assert 0 <= tr.all_metrics["async/staleness_max"] <= 2
    assert tr.all_metrics["policy/grad_norm"] > 0
    assert len(tr.source.consumed) >= 4
    # with weights of its own the engine keeps generating during the update: engine steps happen while the trainer trains
    cfg = _rl_cfg(str(tmp_path / "own"), 3, "trainer.isoexec.strict=false", "generator.inference_engine.own_weights=true")
    tr = FullyAsyncTrainer(cfg, AsyncConfig(max_staleness_steps=2, num_parallel_generation_workers=3, mini_batch_prompts=4), device="cpu")
    during = []
    real = tr._run_training

    def spy(batch, fresh):
        before = tr.engine.stats["steps"]
        real(batch, fresh)
        during.append(tr.engine.stats["steps"] - before)

    tr._run_training = spy
    tr.train()
    assert tr.global_step == 3 and tr.separate_engine and sum(during) > 0
    assert torch.equal(tr.engine.model.store.flat, tr.policy.model.store.flat)


def test_entrypoint_runs_one_step(tmp_path, capsys):
    from skyrl_isoexec_b200.train.entrypoints import main_base

    ov = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
          "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8",
          "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=8",
          "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.num_steps=1",
          f"trainer.ckpt_path={tmp_path}", "trainer.ckpt_interval=0", "trainer.logger=jsonl"]
    exp = main_base.BasePPOExp(SkyRLTrainConfig.from_cli_overrides(ov))
    trainer = exp.run()
    assert trainer.global_step == 1


# ------------------------------------------------------------------ more policy losses, dynamic sampling, ref / critic
def test_rollout_is_dppo_clip_cov_kl_cov_losses():
    from skyrl_isoexec_b200.train import algorithms as alg

    torch.manual_seed(0)
    cfg = alg.AlgorithmConfig(clip_cov_ratio=0.2, clip_cov_lb=-10.0, clip_cov_ub=10.0)
    lp = (torch.randn(4, 9) * 0.3 - 1.0).requires_grad_()
    old = lp.detach() + torch.randn(4, 9) * 0.3
    adv, mask = torch.randn(4, 9), (torch.rand(4, 9) > 0.2).float()
    # rollout_is: gradient coefficient is the ratio inside the band and zero outside
    loss, m = alg.get_policy_loss("rollout_is")(lp, old, adv, cfg, loss_mask=mask, rollout_logprobs=old)
    (g,) = torch.autograd.grad(loss, lp)
    ratio = torch.exp(lp.detach() - old)
    keep = (ratio > 0.8) & (ratio < 1.2)
    assert torch.allclose(g, -(torch.where(keep, ratio, torch.zeros_like(ratio)) * adv * mask), atol=1e-6)
    assert 0.0 <= float(m["clip_ratio"]) <= 1.0
    with pytest.raises(ValueError):
        alg.get_policy_loss("rollout_is")(lp, old, adv, cfg, loss_mask=mask)
    # dppo: dropped tokens carry no gradient; both divergence types run
    for kind in ("binary_tv", "binary_kl"):
        cfg.dppo_type, cfg.dppo_delta_low, cfg.dppo_delta_high = kind, 0.02, 0.02
        loss, m = alg.get_policy_loss("dppo")(lp, old, adv, cfg, loss_mask=mask, rollout_logprobs=old)
        (g,) = torch.autograd.grad(loss, lp)
        assert float(m["clip_ratio"]) > 0 and int((g == 0).sum()) >= int((mask == 0).sum())
    # clip_cov: deterministic given the seed; detached tokens have zero gradient
    l1, m1 = alg.get_policy_loss("clip_cov")(lp, old, adv, cfg, loss_mask=mask)
    l2, _ = alg.get_policy_loss("clip_cov")(lp, old, adv, cfg, loss_mask=mask)
    assert torch.equal(l1, l2) and float(m1["clip_ratio"]) > 0
    # kl_cov: equals the unclipped objective plus the penalty on exactly k tokens
    cfg.kl_cov_frac, cfg.kl_cov_ppo_kl_coef = 0.25, 2.0
    lk, _ = alg.get_policy_loss("kl_cov")(lp, old, adv, cfg, loss_mask=mask)
    base = (-adv * torch.exp(lp - old) * mask).sum()
    k = max(1, int(int(mask.sum()) * 0.25))
    extra = float(lk - base) / 2.0
    topk_sum = None
    cov = alg._token_covariance(lp, adv, mask).masked_fill(mask == 0, float("-inf")).reshape(-1)
    topk_sum = float((lp - old).abs().reshape(-1)[torch.topk(cov, k).indices].sum())
    assert abs(extra - topk_sum) < 1e-4


def test_dynamic_sampling_filter_and_replace():
    from skyrl_isoexec_b200.train import algorithms as alg
    from skyrl_isoexec_b200.train.trainer_utils import cleanup_old_checkpoints, handle_dynamic_sampling, informative_groups, list_checkpoints

    def batch(tag, rewards):
        n = len(rewards)
        return ({"prompt_token_ids": [[1]] * n, "response_ids": [[tag, i] for i in range(n)], "rewards": rewards,
                 "loss_masks": [[1, 1]] * n, "rollout_logprobs": [[0.0, 0.0]] * n},
                [f"{tag}{i // 2}" for i in range(n)])

    go, uids = batch("a", [1.0, 0.0, 1.0, 1.0, 0.0, 0.0, 0.5, 0.2])      # groups a0 (mixed) a1 (all 1) a2 (all 0) a3 (mixed)
    good, bad = informative_groups(go, uids)
    assert good == ["a0", "a3"] and bad == ["a1", "a2"]
    cfg = alg.AlgorithmConfig(dynamic_sampling_type="filter", dynamic_sampling_max_sample_batches=3)
    st: dict = {}
    out, u, more = handle_dynamic_sampling(go, uids, cfg, st, prompts_needed=3, n_samples=2)
    assert more and out is None and st["batches"] == 1
    go2, uids2 = batch("b", [0.0, 1.0, 1.0, 1.0])                          # b0 mixed, b1 flat
    out, u, more = handle_dynamic_sampling(go2, uids2, cfg, st, prompts_needed=3, n_samples=2)
    assert not more and u == ["a0", "a0", "a3", "a3", "b0", "b0"] and out["rewards"] == [1.0, 0.0, 0.5, 0.2, 0.0, 1.0]
    assert st == {}
    cfg2 = alg.AlgorithmConfig(dynamic_sampling_type="filter", dynamic_sampling_max_sample_batches=1)
    with pytest.raises(RuntimeError, match="informative"):
        handle_dynamic_sampling(go2, uids2, cfg2, {}, prompts_needed=5, n_samples=2)
    cfg3 = alg.AlgorithmConfig(dynamic_sampling_type="replace", dynamic_sampling_min_replace_ratio=0.5)
    out, u, more = handle_dynamic_sampling(go, uids, cfg3, {}, prompts_needed=4, n_samples=2, seed=1)
    assert not more and len(u) == 8 and informative_groups(out, u)[1] == []
    cfg3.dynamic_sampling_min_replace_ratio = 0.9
    out, u, more = handle_dynamic_sampling(go, uids, cfg3, {}, prompts_needed=4, n_samples=2)
    assert out is go                                                        # too few informative groups: left alone
    import os
    import tempfile

    with tempfile.TemporaryDirectory() as d:
        for s in (1, 2, 3, 10):
            os.makedirs(os.path.join(d, f"global_step_{s}"))
        assert cleanup_old_checkpoints(d, 2) == [1, 2] and list_checkpoints(d) == [3, 10]


def test_ppo_with_critic_and_reference_kl_runs(tmp_path):
    cfg = _rl_cfg(str(tmp_path), 2, "trainer.algorithm.advantage_estimator=gae", "trainer.algorithm.use_kl_loss=true",
                  "trainer.algorithm.kl_loss_coef=0.01", "trainer.algorithm.lambd=0.95")
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.train()
    assert tr.critic is not None and tr.ref is not None and tr.global_step == 2
    m = tr.all_metrics
    assert m["critic/critic_loss"] > 0 and m["policy/rollout_train_logprob_bit_mismatches"] == 0
    assert m["policy/policy_kl"] >= 0 and m["policy/grad_norm"] > 0
    # the reference stayed frozen while the policy moved
    assert not torch.equal(tr.ref.model.store.flat, tr.policy.model.store.flat)


def test_lora_adapter_store_merges_exactly_and_trains():
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train import algorithms as alg
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.lora import AdapterStore, LoRAAdapter, LoRAConfig, LoRATrainer
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    model = DecoderLM(get_config("tiny-qwen3"), seed=1)
    base = model.store.flat.clone()
    store = AdapterStore(model)
    a1 = LoRAAdapter.init(model, LoRAConfig(rank=4, lr=5e-3, seed=1))
    a2 = LoRAAdapter.init(model, LoRAConfig(rank=2, seed=2))
    for b in a2.B.values():
        b.normal_(0, 0.02)
    store.register("tenant1", a1)
    store.register("tenant2", a2)
    store.activate("tenant2")
    assert not torch.equal(model.store.flat, base)
    store.activate("tenant1")                          # B = 0: a fresh adapter is a no-op, and tenant2 is fully removed
    assert torch.equal(model.store.flat, base)
    # train tenant1 on a fixed SFT batch; the loss goes down, the base does not move
    g = torch.Generator().manual_seed(0)
    ex = [(torch.randint(0, 300, (6,), generator=g).tolist(), torch.randint(0, 300, (9,), generator=g).tolist()) for _ in range(6)]
    seq, att, rmask = build_sequences([p for p, _ in ex], [r for _, r in ex])
    batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                "advantages": torch.zeros_like(rmask)})
    worker = PolicyWorker(model, WorkerConfig(), alg.AlgorithmConfig(policy_loss_type="cross_entropy"))
    tr = LoRATrainer(worker, store, "tenant1")
    losses = []
    for _ in range(8):
        losses.append(worker.forward_backward(batch)["policy_loss"])
        assert tr.optim_step() > 0
    assert losses[-1] < losses[0] * 0.97, losses
    store.deactivate()
    assert torch.equal(model.store.flat, base)
    sd = a1.state_dict()
    a1b = LoRAAdapter.from_state_dict(sd)
    assert a1b.num_parameters() == a1.num_parameters() and torch.equal(a1b.B["layers.0.attn.o.weight"], a1.B["layers.0.attn.o.weight"].cpu())


def test_fusion_ledger_digest_and_checkers():
    from skyrl_isoexec_b200.core import fusion_ledger as FL

    d = FL.ledger_digest()
    assert len(d) == 24 and d == FL.ledger_digest()
    assert FL.ledger_digest(FL.REGIONS[:-1]) != d                       # a different fusion set is a different contract
    res = FL.run_checkers("cpu")
    assert set(res) == {r.name for r in FL.REGIONS}                     # every fused region has a checker
    cpu_checkable = ("rmsnorm+residual", "logprob_fused", "qk_norm+rope+kv_write", "leaftree_gemm (LOCAL)",
                     "attention (prefill | decode | chunk)", "gdn_scan (chunked | recurrent)")
    assert all(res[n] is True for n in cpu_checkable), res
    assert all(v is not False for v in res.values())                    # the rest is deferred to a GPU, never "differs"
    # a region nobody can prove blocks the preflight instead of passing as "unknown"
    extra = FL.REGIONS + (FL.FusedRegion("made_up_fusion", ("a", "b"), "bitwise"),)
    old_regions, FL.REGIONS = FL.REGIONS, extra
    try:
        import pytest as _pt

        with _pt.raises(LookupError):
            FL.run_checkers("cpu")
        from skyrl_isoexec_b200.core import preflight

        assert any("made_up_fusion" in e for e in preflight.check_fusion_ledger())
    finally:
        FL.REGIONS = old_regions
    x = FL.hazard_population((64, 64), torch.float32, "cpu")
    assert (x == 0).any() and (x.abs() > 1e30).any() and (x.abs() < 1e-35).logical_and(x != 0).any()


def test_moe_utils_io_and_nccl_capabilities(tmp_path):
    from skyrl_isoexec_b200.parallel import nccl_runtime
    from skyrl_isoexec_b200.train.moe_utils import RouterReplay, balanced_dp_assignment, imbalance
    from skyrl_isoexec_b200.utils import io

    lens = [900, 40, 800, 60, 700, 100, 650, 120]
    a = balanced_dp_assignment(lens, 2)
    assert sorted(i for r in a for i in r) == list(range(8)) and len(a[0]) == len(a[1]) == 4
    assert imbalance(lens, a) < 1.05 < imbalance(lens, [[0, 2, 4, 6], [1, 3, 5, 7]])
    rr = RouterReplay()
    rr.mode = "record"
    idx = torch.tensor([[0, 3], [1, 2], [2, 0]])
    assert rr.route(5, idx) is idx
    rr.mode = "replay"
    other = torch.tensor([[3, 0], [1, 3], [2, 0]])                         # same set in row 0 (order differs), a flip in row 1
    got = rr.route(5, other)
    assert torch.equal(got, idx) and rr.flips == 1
    p = str(tmp_path / "a" / "marker.txt")
    with io.atomic_write(p) as f:
        f.write("7")
    assert io.exists(p) and io.list_dir(str(tmp_path / "a")) == ["marker.txt"] and io.scheme("s3://b/k") == "s3"
    with pytest.raises(RuntimeError, match="s3"):
        io.exists("s3://bucket/key")
    caps = nccl_runtime.capabilities()
    assert caps["backend"] in ("none", "gloo", "nccl") and "peer_access" in caps
    with pytest.raises(RuntimeError):
        nccl_runtime.require({"peer_access": False}, "peer_access")


def test_hf_export_roundtrip_and_dispatch_helpers(tmp_path):
    from safetensors.torch import load_file

    from skyrl_isoexec_b200.models import hf_export
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.parallel import dispatch
    from skyrl_isoexec_b200.parallel.state import ParallelState

    for preset in ("tiny-qwen3", "tiny-moe", "tiny-llama"):
        cfg = get_config(preset)
        m = DecoderLM(cfg, seed=3)
        d = str(tmp_path / preset)
        hf_export.save_hf(m, d)
        sd = load_file(d + "/model.safetensors")
        Hq, Hkv, D = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
        assert sd["model.layers.0.self_attn.q_proj.weight"].shape == (Hq * D, cfg.hidden_size)
        assert sd["model.layers.0.self_attn.k_proj.weight"].shape == (Hkv * D, cfg.hidden_size)
        # q head h of the export is the h-th query head of the fused, group-major storage
        G = Hq // Hkv
        fused = m.p("layers.0.attn.qkv.weight").detach().view(Hkv, G * D + 2 * D, -1)
        assert torch.equal(sd["model.layers.0.self_attn.q_proj.weight"].view(Hq, D, -1)[G], fused[1, :D])
        m2 = DecoderLM(cfg, seed=99)
        assert hf_export.load_hf(m2, d) == len(m.store.order) and torch.equal(m2.store.flat, m.store.flat)
        assert json.load(open(d + "/config.json"))["num_hidden_layers"] == cfg.num_layers
    ps = ParallelState.single()
    assert dispatch.dp_slice(12, 1, 3) == slice(4, 8)
    with pytest.raises(ValueError):
        dispatch.dp_slice(10, 0, 3)
    assert dispatch.reduce_metrics({"a": 1.0, "s": "x"}, ps) == {"a": 1.0, "s": "x"}
    x = torch.arange(6).view(3, 2)
    assert dispatch.gather_rows(x, ps) is x


def test_trainer_eval_and_hf_export_hooks(tmp_path):
    cfg = _rl_cfg(str(tmp_path / "ck"), 2, "trainer.eval_interval=1", "trainer.eval_before_train=true", "trainer.eval_batch_size=3",
                  "generator.eval_n_samples_per_prompt=2", "generator.eval_sampling_params.max_generate_length=6",
                  "generator.eval_sampling_params.temperature=1.0", "generator.eval_sampling_params.ignore_eos=true",
                  f"trainer.export_path={tmp_path / 'hf'}", "trainer.hf_save_interval=2")
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.train()
    assert tr.last_eval["eval/num_prompts"] == 3 and "eval/pass_at_2" in tr.last_eval
    import os

    assert sorted(os.listdir(tmp_path / "hf" / "global_step_2")) == ["config.json", "model.safetensors"]


def test_preflight_gate_ready_and_blocks_on_a_missing_kernel(monkeypatch, capsys):
    from skyrl_isoexec_b200.core import preflight

    assert preflight.main(["--model", "qwen3-8b"]) == 0
    assert "PREFLIGHT: READY" in capsys.readouterr().out
    monkeypatch.setattr(preflight, "check_native", lambda: ["libisoexec_b200.so is missing"])
    assert preflight.main(["--model", "tiny-qwen3"]) == 1
    out = capsys.readouterr().out
    assert "PREFLIGHT: BLOCKED" in out and "native         BLOCKED" in out


def test_weight_sync_factory_dispatches_the_peer_strategy(monkeypatch):
    from skyrl_isoexec_b200.sync import peer_push, strategies

    made = []

    class _S:
        def __init__(self, info, model, **kw):
            made.append(("sender", kw))

    class _R:
        def __init__(self, info, model):
            made.append(("receiver", {}))

    monkeypatch.setattr(peer_push, "PeerPushSender", _S)
    monkeypatch.setattr(peer_push, "PeerPushReceiver", _R)
    info = peer_push.PeerPushInitInfo("h", 8, "bfloat16", None)
    assert info.strategy_type() == "peer"
    strategies.create_sender(info, None, from_master=None)
    strategies.create_receiver(info, None)
    assert made == [("sender", {"from_master": None}), ("receiver", {})]
    with pytest.raises(ValueError):
        strategies.create_init_info("carrier-pigeon", contract_hash="h")


def test_kept_layer_budget_and_activation_estimate():
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.parallel.state import ParallelState
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig, layers_that_fit

    gb = 1 << 30
    assert layers_that_fit(5 * gb, gb, 36) == 0                       # under the margin: recompute everything
    assert layers_that_fit(10 * gb + 5 * gb, gb, 36) == 4             # 5 GB over the margin, 1.25 GB per layer
    assert layers_that_fit(500 * gb, gb, 36) == 36                    # never more than the model has
    assert layers_that_fit(50 * gb, 0, 36) == 0
    w = PolicyWorker(DecoderLM(get_config("tiny-qwen3"), ParallelState.single(), seed=0), WorkerConfig(keep_last_layers=-1))
    c = w.model.cfg
    per_tok = 6 * c.hidden_size + (c.num_q_heads + 2 * c.num_kv_heads) * c.head_dim + (c.num_q_heads + c.num_kv_heads) * c.head_dim \
        + c.num_q_heads * c.head_dim + 3 * c.ffn_size
    assert w.activation_bytes_per_layer(100) == 2 * per_tok * 100
    assert w.keep_layers() == 0 and w._ckpt_arg() in (True, False)    # auto: nothing kept before the first step calibrates
    w._calibrate_keep()                                               # CPU: calibrates to 0 and stays there
    assert w._auto_keep == 0 and w.keep_layers() == 0


def test_attention_backward_work_lists_cover_every_tile_once_heaviest_first():
    from skyrl_isoexec_b200.ops import functional as F

    lens = [300, 17, 129, 128, 513]
    Hq, Hkv = 8, 2
    tq = 128 // (Hq // Hkv)
    meta = F.AttnMeta.packed(lens, Hq, Hkv, "cpu")
    iq, ik = meta.bwd_items(Hq, Hkv, "cpu")
    assert meta.bwd_items(Hq, Hkv, "cpu")[0] is iq                       # built once
    starts, s = [], 0
    for n in lens:
        starts.append((s, s + n))
        s += n
    want_q = {(a + t0, a, b) for a, b in starts for t0 in range(0, b - a, tq)}
    want_k = {(a + k0, a, b) for a, b in starts for k0 in range(0, b - a, 128)}
    got_q = [tuple(r[:3]) for r in iq.tolist()]
    got_k = [tuple(r[:3]) for r in ik.tolist()]
    assert len(got_q) == len(want_q) and set(got_q) == want_q
    assert len(got_k) == len(want_k) and set(got_k) == want_k
    # dQ work grows with the tile's last position, dK/dV work with the distance to the end of the sequence
    wq = [min(t + tq, b) - a for t, a, b in got_q]
    wk = [b - t for t, a, b in got_k]
    assert wq == sorted(wq, reverse=True) and wk == sorted(wk, reverse=True)


def test_scoring_forward_can_be_skipped_on_policy_with_the_same_weights_bit_for_bit(tmp_path):
    """With the contract enforced and one optimizer step per rollout batch, the engine's logprobs are the old-policy
    logprobs: skipping the scoring forward leaves the updated weights unchanged bit for bit, the gate still runs (on
    the training forward), and a rollout logprob that is off by one ulp is refused BEFORE the weights move."""
    from skyrl_isoexec_b200.train.entrypoints import main_base
    from skyrl_isoexec_b200.core.ledger import ContractViolation
    from skyrl_isoexec_b200.train.trainer import ForwardGateError

    def run(reuse, tamper=False):
        ov = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
              "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8",
              "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=8",
              "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.num_steps=2",
              f"trainer.ckpt_path={tmp_path}/r{int(reuse)}{int(tamper)}", "trainer.ckpt_interval=0", "trainer.logger=jsonl",
              "trainer.policy.optimizer_config.lr=1e-3", f"trainer.isoexec.reuse_rollout_logprobs={'true' if reuse else 'false'}"]
        exp = main_base.BasePPOExp(SkyRLTrainConfig.from_cli_overrides(ov))
        tr = exp.get_trainer()
        tr.build_models()
        tr.sync_weights()
        it = iter(tr.loader)
        if tamper:
            orig = tr.convert_to_training_input

            def bent(go, uids):
                b = orig(go, uids)
                ro = b["rollout_logprobs"]
                ro[0, -1] = torch.nextafter(ro[0, -1], torch.tensor(0.0))
                return b

            tr.convert_to_training_input = bent
        before = tr.policy.model.store.flat.detach().clone()
        m = [tr.train_step(next(it)) for _ in range(2)] if not tamper else None
        return tr, m, before

    tr_a, m_a, _ = run(False)
    tr_b, m_b, _ = run(True)
    assert torch.equal(tr_a.policy.model.store.flat.detach(), tr_b.policy.model.store.flat.detach())
    assert all(m["policy/rollout_train_logprob_bit_mismatches"] == 0 for m in m_a + m_b)
    assert all(m.get("policy/scoring_forward_skipped") == 1 for m in m_b) and "policy/scoring_forward_skipped" not in m_a[0]
    assert m_b[0]["timing/fwd_logprobs"] < m_a[0]["timing/fwd_logprobs"]
    tr_c, _, before = run(True, tamper=True)
    with pytest.raises((ForwardGateError, ContractViolation)):      # the ledger refuses at step 1, the gate afterwards
        tr_c.train_step(next(iter(tr_c.loader)))
    assert torch.equal(tr_c.policy.model.store.flat.detach(), before)       # refused before the optimizer step


def test_fused_tp_admission_probe_and_transport_census():
    """A shape is admitted to the fused GEMM+collective kernel only if its first call reproduces the plain path bit
    for bit; a refused shape stays on the plain path; the census says who served what."""
    from types import SimpleNamespace

    from skyrl_isoexec_b200.parallel import tp

    ps = SimpleNamespace(tp=1, tp_group=None)
    torch.manual_seed(0)
    x, w = torch.randn(12, 64), torch.randn(16, 64)
    want = tp.leaftree_gemm(x, w, 4, False)

    class Good:
        calls = 0

        def row_parallel(self, x, w, leaves, out_dtype=torch.float32):
            Good.calls += 1
            return tp.leaftree_gemm(x, w, leaves, False).to(out_dtype)

        def check(self):
            pass

    class Bad(Good):
        def row_parallel(self, x, w, leaves, out_dtype=torch.float32):
            out = super().row_parallel(x, w, leaves, out_dtype).clone()
            out[0, 0] = torch.nextafter(out[0, 0], torch.tensor(float("inf")))      # one ulp off
            return out

    class Broken(Good):
        def check(self):
            raise RuntimeError("a wait ran out")

    tp._ADMITTED.clear()
    ok, first = tp.admit_fused_row_parallel(Good(), ps, x, w, 4, torch.float32)
    assert ok and torch.equal(first, want)
    ok2, first2 = tp.admit_fused_row_parallel(Good(), ps, x, w, 4, torch.float32)
    assert ok2 and first2 is None and Good.calls == 1                          # probed once per shape
    ok3, first3 = tp.admit_fused_row_parallel(Bad(), ps, x, w[:8], 4, torch.float32)
    assert not ok3 and torch.equal(first3, tp.leaftree_gemm(x, w[:8], 4, False))   # refused: the plain result is served
    ok4, _ = tp.admit_fused_row_parallel(Broken(), ps, x, w[:4], 4, torch.float32)
    assert not ok4
    assert sorted(tp.admitted_shapes().values()) == [False, False, True]
    tp._CENSUS.clear()
    cfg = SimpleNamespace(pik_leaves=4, tp_invariant=True)
    from skyrl_isoexec_b200.parallel.state import ParallelState

    y = tp.row_parallel_linear(x, w, ParallelState.single(), cfg)
    assert torch.equal(y, want)
    assert tp.transport_census(reset=True) == {"row_parallel/local": 1} and tp.transport_census() == {}
    tp._ADMITTED.clear()


def test_llama_style_decoder_runs_one_rl_step_with_bitwise_rollout_logprobs(tmp_path):
    """The dense family without QK-norm (Llama-3 style preset): one full step on CPU, engine == trainer bit for bit."""
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.train.entrypoints import main_base

    assert get_config("llama3-8b").param_count() > 7.5e9 and not get_config("llama3-8b").qk_norm
    ov = ["trainer.policy.model=tiny-llama", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
          "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8",
          "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=8",
          "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.num_steps=1",
          f"trainer.ckpt_path={tmp_path}", "trainer.ckpt_interval=0", "trainer.logger=jsonl"]
    tr = main_base.BasePPOExp(SkyRLTrainConfig.from_cli_overrides(ov)).get_trainer()
    tr.build_models()
    tr.sync_weights()
    m = tr.train_step(next(iter(tr.loader)))
    assert m["policy/rollout_train_logprob_bit_mismatches"] == 0 and m["policy/grad_norm"] > 0


def test_profiler_window_and_phase_timers_are_wired_into_the_step(tmp_path):
    from skyrl_isoexec_b200.train.entrypoints import main_base

    ov = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
          "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=4",
          "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=12",
          "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.num_steps=3",
          f"trainer.ckpt_path={tmp_path}", "trainer.ckpt_interval=0", "trainer.logger=jsonl",
          "trainer.profiler.enable=true", "trainer.profiler.start_step=1", "trainer.profiler.end_step=2",
          f"trainer.profiler.save_path={tmp_path}/prof", "trainer.nvtx=true"]
    tr = main_base.BasePPOExp(SkyRLTrainConfig.from_cli_overrides(ov)).run()
    assert tr.global_step == 3
    assert (tmp_path / "prof" / "trace_rank0.json").stat().st_size > 1000      # the window [1, 2) was captured
    assert {"timing/generate", "timing/fwd_logprobs", "timing/policy_train"} <= set(tr.all_metrics)
    from skyrl_isoexec_b200.utils.tracking import Timer

    Timer.nvtx = False


def test_gpu_monitor_parses_and_summarises_with_a_fake_query():
    import time

    from skyrl_isoexec_b200.utils.gpu_monitor import GpuMonitor, parse_row

    assert parse_row("garbage") is None and parse_row("a, b, c, d, e, f") is None
    r = parse_row("1740, 1965, 985.2, 99, 160000, Not Active, Not Active, Not Active, Active")
    assert r["sm_mhz"] == 1740 and r["reasons"] == {"sw_power_cap"}
    lines = iter(["1700, 1965, 900.0, 98, 1000, Not Active, Not Active, Not Active, Active",
                  "1800, 1965, 950.0, 99, 2000, Not Active, Not Active, Not Active, Not Active",
                  "1750, 1965, 990.0, 97, 1500, Not Active, Active, Not Active, Active"] + ["bad"] * 1000)
    mon = GpuMonitor(0, period_s=0.01, runner=lambda: next(lines))
    mon.start()
    t0 = time.time()
    while len(mon.rows) < 3 and time.time() - t0 < 10:
        time.sleep(0.02)
    s = mon.stop()
    assert s["samples"] == 3 and s["sm_mhz"] == 1750 and s["sm_max_mhz"] == 1965 and s["mem_mib"] == 2000
    assert s["reasons"] == ["hw_thermal_slowdown", "sw_power_cap"]


def test_tinker_and_memory_sweep_benchmarks_run_on_cpu():
    from skyrl_isoexec_b200.benchmarks import bench_tinker, memory_sweep

    r = bench_tinker.run("tiny-qwen3", requests=2, device="cpu", prompt_len=6, response_len=4)
    assert r["sample"]["tokens_per_s"] > 0 and r["train"]["steps_per_s"] > 0
    rows = memory_sweep.run("tiny-qwen3", 0, [64, 128], 32, "cpu")
    assert [x["tokens"] for x in rows] == [64, 128] and all(x["tokens_per_s"] > 0 and x["estimate_gib"] >= 0 for x in rows)


def test_config_file_with_nested_keys_legacy_names_and_overrides(tmp_path):
    p = tmp_path / "run.yaml"
    p.write_text("""
trainer:
  train_batch_size: 4
  policy_mini_batch: 2            # legacy name
  policy:
    model: tiny-moe
    model_overrides: {num_layers: 1}
  algorithm:
    eps_clip: 0.3                 # legacy name
  isoexec:
    reuse_rollout_logprobs: true
generator:
  num_samples: 2                  # legacy name
  sampling_params:
    stop: null
""")
    cfg = SkyRLTrainConfig.from_file(str(p), ["trainer.train_batch_size=8", "generator.temperature=0.5"])
    t = cfg.trainer
    assert t.train_batch_size == 8 and t.policy_mini_batch_size == 2 and t.policy.model == "tiny-moe"
    assert t.policy.model_overrides == {"num_layers": 1} and t.algorithm.eps_clip_low == 0.3 and t.isoexec.reuse_rollout_logprobs
    assert cfg.generator.n_samples_per_prompt == 2 and cfg.generator.sampling_params.temperature == 0.5
    j = tmp_path / "run.json"
    j.write_text(json.dumps({"trainer": {"epochs": 3}}))
    assert SkyRLTrainConfig.from_file(str(j)).trainer.epochs == 3
    bad = tmp_path / "bad.yaml"
    bad.write_text("trainer:\n  no_such_key: 1\n")
    with pytest.raises(KeyError):
        SkyRLTrainConfig.from_file(str(bad))


def test_worker_dispatch_verbs_staging_lcm_and_residency(tmp_path):
    from types import SimpleNamespace

    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.parallel.state import ParallelState
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig
    from skyrl_isoexec_b200.train.worker_dispatch import WorkerDispatch

    ps = ParallelState.single()
    policy = PolicyWorker(DecoderLM(get_config("tiny-qwen3"), ps, seed=1), WorkerConfig(max_tokens_per_microbatch=64))
    critic = PolicyWorker(DecoderLM(get_config("tiny-qwen3"), ps, seed=2), WorkerConfig(max_tokens_per_microbatch=64))
    ref = SimpleNamespace(ps=SimpleNamespace(dp=3), opt=None, forward=lambda b: "ref-forward")
    synced = []
    d = WorkerDispatch({"policy": policy, "critic": critic, "ref": ref, "absent": None}, sync_fn=lambda: synced.append(1))
    assert sorted(d.workers) == ["critic", "policy", "ref"] and d.get_lcm_dp_size() == 3
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (6,), generator=g).tolist() for _ in range(4)]
    resp = [torch.randint(0, 2048, (5,), generator=g).tolist() for _ in range(4)]
    seq, att, rmask = build_sequences(prompts, resp)
    batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                "advantages": torch.ones(rmask.shape)})
    assert d.pad_batch(batch).batch_size == 6                           # 4 rows -> next multiple of 3
    assert d.forward("ref", batch) == "ref-forward"
    key = d.stage_data(batch)
    m1 = d.forward_backward_from_staged("policy", key, 0, 2)
    m2 = d.forward_backward_from_staged("policy", key, 2, 4)
    assert m1["loss_tokens"] == m2["loss_tokens"] == 10 and d.optim_step("policy") > 0
    assert d.residency == {"policy": "gpu", "critic": "cpu", "ref": "gpu"}     # the critic's state was parked, the ref has none
    d.forward_backward("critic", batch)
    assert d.residency["policy"] == "cpu" and d.residency["critic"] == "gpu"
    assert d.transitions == [("critic", "cpu"), ("policy", "cpu"), ("critic", "gpu")]
    d.offload_all()
    assert d.residency["critic"] == "cpu"
    d.drop_staged(key)
    with pytest.raises(KeyError):
        d.forward_backward_from_staged("policy", key, 0, 1)
    d.save_weights_for_sampler()
    assert synced == [1]
    path = d.save_checkpoint(str(tmp_path), 1, {"pos": 1}, {"global_step": 1})
    ds, ts = d.load_checkpoint(path)
    assert ds["pos"] == 1 and ts["global_step"] == 1 and d.residency["policy"] == "gpu"


def test_generate_sft_and_serve_entry_points(tmp_path):
    import urllib.request

    from skyrl_isoexec_b200.train.entrypoints import main_generate, main_sft, serve

    ov = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
          "generator.n_samples_per_prompt=2", "generator.eval_n_samples_per_prompt=2", "generator.eval_sampling_params.max_generate_length=4",
          "generator.eval_sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=8",
          "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.eval_batch_size=3",
          f"trainer.ckpt_path={tmp_path}/ck", "trainer.resume_mode=none", "trainer.logger=jsonl", f"trainer.export_path={tmp_path}/out"]
    out = main_generate.run(SkyRLTrainConfig.from_cli_overrides(ov))
    assert any(k.startswith("eval/") for k in out) and json.load(open(tmp_path / "out" / "eval.json")) == out
    data = tmp_path / "sft.jsonl"
    g = torch.Generator().manual_seed(0)
    with open(data, "w") as f:
        for _ in range(6):
            f.write(json.dumps({"prompt_ids": torch.randint(0, 500, (5,), generator=g).tolist(),
                                "response_ids": torch.randint(0, 500, (7,), generator=g).tolist()}) + "\n")
    tr = main_sft.main(["--data", str(data), "--batch-size", "3", "--num-steps", "2", "--lr", "1e-3", "--logger", "jsonl"])
    assert tr.global_step == 2
    # a config file, a key=value override of it, and a command-line option that overrides both
    (tmp_path / "sft.yaml").write_text("model: tiny-qwen3\nbatch_size: 2\nnum_steps: 5\nlogger: jsonl\noptimizer:\n  lr: 1.0e-3\n  weight_decay: 0.0\n")
    tr = main_sft.main(["--data", str(data), "--config", str(tmp_path / "sft.yaml"), "--num-steps", "1", "optimizer.lr=2e-3", "batch_size=3"])
    assert tr.global_step == 1 and tr.cfg.batch_size == 3 and tr.cfg.optimizer.lr == 2e-3 and tr.cfg.optimizer.weight_decay == 0.0
    with pytest.raises(KeyError):
        main_sft.SFTConfig.from_file(str(tmp_path / "sft.yaml"), ["no_such_field=1"])
    srv = serve.build(["--model", "tiny-qwen3", "--num-kv-pages", "16", "--device", "cpu"]).start()
    try:
        with urllib.request.urlopen(srv.url + "/health", timeout=10) as r:
            assert json.loads(r.read())["status"] == "ok"
        with urllib.request.urlopen(srv.url + "/metrics", timeout=10) as r:
            assert b"isoexec_requests_served_total" in r.read()
    finally:
        srv.shutdown()


def test_example_configs_load_and_validate():
    import glob
    import os

    from skyrl_isoexec_b200.train.config import validate_cfg

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    files = sorted(glob.glob(os.path.join(root, "*.yaml")))
    assert len(files) >= 8
    for f in files:
        cfg = SkyRLTrainConfig.from_file(f)
        validate_cfg(cfg, 8 if any(k in f for k in ("8gpu", "ep8", "tp4dp2", "tp2dp4", "tp8")) else 2 if "tp2" in f else 1)
    named = SkyRLTrainConfig.from_file(os.path.join(root, "qwen3_8b_tp4dp2_engines_tp2.yaml"))
    assert named.trainer.policy.parallel.tensor_model_parallel_size == 4 and named.generator.inference_engine.tensor_parallel_size == 2
    big = SkyRLTrainConfig.from_file(os.path.join(root, "qwen3_8b_grpo_8gpu.yaml"))
    assert big.trainer.policy.model == "qwen3-8b" and big.trainer.policy.keep_last_layers == -1 and big.generator.n_samples_per_prompt == 8


def test_runnable_examples_run(tmp_path):
    """The two CPU-sized example configs that bring their own algorithm variant run their steps; the callbacks example
    stops early and checkpoints on a new best."""
    import importlib.util
    import os

    from skyrl_isoexec_b200.train.entrypoints import main_base

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    for name in ("ppo_gae_critic.yaml", "off_policy_tis_correction.yaml"):
        cfg = SkyRLTrainConfig.from_file(os.path.join(root, name), [f"trainer.ckpt_path={tmp_path / name}", "trainer.logger=jsonl"])
        tr = main_base.BasePPOExp(cfg).run()
        assert tr.global_step == 2 and tr.all_metrics["policy/grad_norm"] >= 0
    spec = importlib.util.spec_from_file_location("callbacks_early_stop", os.path.join(root, "callbacks_early_stop.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    tr = mod.main(str(tmp_path / "cb"), num_steps=12)
    cb = tr.callbacks.callbacks[0]
    assert 1 <= tr.global_step <= 12 and cb.best > float("-inf")
    assert tr.global_step == 12 or cb.since >= cb.patience
    assert any(d.startswith("global_step_") for d in os.listdir(tmp_path / "cb")), "a new best wrote a checkpoint"
    assert "early_stop/best_reward" in tr.all_metrics


def test_process_group_timeout_follows_the_environment_flag(monkeypatch):
    """``init_distributed`` takes its collective timeout from SKYRL_WORKER_NCCL_TIMEOUT_IN_S unless told otherwise."""
    import datetime

    import torch.distributed as dist

    from skyrl_isoexec_b200.parallel import state

    seen = {}
    monkeypatch.setattr(dist, "is_initialized", lambda: False)
    monkeypatch.setattr(dist, "init_process_group", lambda **kw: seen.update(kw))
    for k, v in (("RANK", "1"), ("WORLD_SIZE", "2"), ("LOCAL_RANK", "1")):
        monkeypatch.setenv(k, v)
    monkeypatch.delenv("SKYRL_WORKER_NCCL_TIMEOUT_IN_S", raising=False)
    assert state.init_distributed(backend="gloo") == (1, 2, 1) and seen["timeout"] == datetime.timedelta(seconds=600)
    monkeypatch.setenv("SKYRL_WORKER_NCCL_TIMEOUT_IN_S", "45")
    state.init_distributed(backend="gloo")
    assert seen["timeout"] == datetime.timedelta(seconds=45)
    state.init_distributed(backend="gloo", timeout_s=7)
    assert seen["timeout"] == datetime.timedelta(seconds=7)
    monkeypatch.setenv("WORLD_SIZE", "1")
    seen.clear()
    assert state.init_distributed() == (0, 1, 1) and not seen


def test_controller_drives_workers_through_the_dispatch_with_optimizer_residency(tmp_path):
    """The trainer reaches policy, critic and reference through WorkerDispatch; with ``placement.offload_optimizer`` only
    the model being trained keeps its optimizer state resident and nothing is resident during rollout."""
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer
    from skyrl_isoexec_b200.train.worker_dispatch import WorkerDispatch

    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=6",
        "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=8",
        "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=8", "trainer.logger=jsonl",
        "trainer.algorithm.advantage_estimator=gae", "trainer.algorithm.use_kl_loss=true", "trainer.placement.offload_optimizer=true"])
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.build_models()
    assert isinstance(tr.dispatch, WorkerDispatch) and set(tr.dispatch.workers) == {"policy", "critic", "ref"}
    calls = []
    for verb in ("forward", "forward_backward", "optim_step"):
        orig = getattr(tr.dispatch, verb)
        setattr(tr.dispatch, verb, (lambda o, v: (lambda name, *a: (calls.append((v, name)), o(name, *a))[1]))(orig, verb))
    tr.sync_weights()
    m = tr.train_step(next(iter(tr.loader)))
    assert m["policy/rollout_train_logprob_bit_mismatches"] == 0 and m["policy/grad_norm"] > 0
    assert {("forward", "policy"), ("forward", "ref"), ("forward", "critic"), ("forward_backward", "critic"), ("optim_step", "critic"),
            ("forward_backward", "policy"), ("optim_step", "policy")} <= set(calls)
    tl = tr.dispatch.transitions
    # rollout first: both optimizers parked; then the critic trains (its state comes back), then the policy (critic parked again)
    assert tl[:2] == [("policy", "cpu"), ("critic", "cpu")] and ("critic", "gpu") in tl and tl[-1] == ("policy", "gpu")
    assert tr.dispatch.residency == {"policy": "gpu", "critic": "cpu", "ref": "gpu"}


def test_model_resolution_from_a_hf_style_directory_round_trips(tmp_path):
    """``trainer.policy.model`` may name a checkpoint directory: ``config.json``'s architecture picks the family and the
    exported weights load back bit for bit."""
    from skyrl_isoexec_b200.models import hf_export
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM

    for preset in ("tiny-qwen3", "tiny-moe", "tiny-llama", "tiny-hybrid"):
        src = DecoderLM(get_config(preset), device="cpu", seed=5)
        d = str(tmp_path / preset)
        hf_export.save_hf(src, d)
        cfg = get_config(d)
        ref = get_config(preset)
        for f in ("hidden_size", "num_layers", "num_q_heads", "num_kv_heads", "head_dim", "ffn_size", "vocab_size", "num_experts",
                  "top_k", "moe_ffn_size", "qk_norm", "tie_embeddings"):
            assert getattr(cfg, f) == getattr(ref, f), (preset, f, getattr(cfg, f), getattr(ref, f))
        assert cfg.layer_types == ref.layer_types and cfg.gdn_v_heads == ref.gdn_v_heads
        dst = DecoderLM(cfg.with_(dtype=ref.dtype), device="cpu", seed=9)
        hf_export.load_hf(dst, d)
        assert torch.equal(dst.store.flat, src.store.flat)
    with pytest.raises(KeyError):
        get_config(str(tmp_path / "nowhere"))


def test_samples_of_one_prompt_share_its_full_kv_pages_with_the_same_bits():
    """The n samples of a prompt take the first sample's full prompt pages instead of recomputing them: greedy outputs and
    logprobs equal the unshared run bit for bit, sampled-token logprobs equal the trainer's forward, fewer tokens are
    prefilled, every page is free afterwards, and a pool tight enough to preempt still ends clean."""
    from skyrl_isoexec_b200.core.testing import count_bit_mismatches
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import SamplingParams
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    cfg = get_config("tiny-qwen3")
    model = DecoderLM(cfg, device="cpu", seed=3)
    g = torch.Generator().manual_seed(5)
    base = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (380, 250, 129)]
    prompts = [p for p in base for _ in range(3)]                 # 3 samples each; 129 tokens: one full page to share

    def run(share, pages, sp):
        eng = LLMEngine(model, EngineConfig(max_num_seqs=9, num_kv_pages=pages, max_num_batched_tokens=512, share_prompt_pages=share))
        outs = eng.generate(prompts, sp)
        assert eng.cache.allocator.num_free == pages and not any(eng.cache.allocator.refs)
        return eng, outs

    greedy = SamplingParams(max_generate_length=10, ignore_eos=True, temperature=0.0)
    e0, o0 = run(False, 40, greedy)
    e1, o1 = run(True, 40, greedy)
    assert [o.response_ids for o in o0] == [o.response_ids for o in o1]
    assert [o.response_logprobs for o in o0] == [o.response_logprobs for o in o1]
    assert e1.scheduler.shared_prompt_tokens == 2 * (256 + 128 + 128) and e0.scheduler.shared_prompt_tokens == 0
    assert e1.stats["prefill_tokens"] == e0.stats["prefill_tokens"] - e1.scheduler.shared_prompt_tokens
    # sampled rollout with sharing: the trainer's forward gives the same logprob bits
    e2, o2 = run(True, 40, SamplingParams(max_generate_length=12, ignore_eos=True))
    seq, att, rmask = build_sequences([o.prompt_ids for o in o2], [o.response_ids for o in o2])
    batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask})
    lp = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=1024)).forward(batch)
    ro = torch.zeros_like(lp)
    for i, o in enumerate(o2):
        ro[i, :len(o.response_logprobs)] = torch.tensor(o.response_logprobs)
    assert count_bit_mismatches((lp * rmask).contiguous(), (ro * rmask).contiguous()) == 0
    # a pool that cannot hold all nine sequences once the longest cross a page boundary (19 pages with sharing, 27
    # without): preemptions happen, reference counts still balance, the greedy outputs do not change
    e3, o3 = run(True, 17, greedy)
    assert e3.scheduler.preemptions > 0
    assert [o.response_ids for o in o3] == [o.response_ids for o in o0]


def test_sft_chat_records_loss_masks_eval_callbacks_export_and_cache(tmp_path):
    """Chat records with tool calls are tokenized with assistant-only loss masks (all turns or the last one), cached on
    disk, trained on; the held-out loss falls; callbacks fire; the Hugging Face export is written at the end."""
    from skyrl_isoexec_b200.train import sft_data
    from skyrl_isoexec_b200.train.policy_worker import OptimizerConfig

    class ByteTok:
        vocab_size = 256
        name_or_path = "bytes"

        def encode(self, text):
            return list(text.encode())

    tok = ByteTok()
    chat = {"messages": [{"role": "system", "content": "be brief"}, {"role": "user", "content": "2+2?"},
                         {"role": "assistant", "content": "", "tool_calls": '{"function": {"name": "calc", "arguments": "{\\"e\\": \\"2+2\\"}"}}'},
                         {"role": "tool", "name": "calc", "content": "4"}, {"role": "assistant", "content": "four"}],
            "tools": '{"name": "calc"}'}
    row_all = sft_data.tokenize_chat(chat, tok, 4096, "all")
    row_last = sft_data.tokenize_chat(chat, tok, 4096, "last")
    full = row_all["prompt_ids"] + row_all["response_ids"]
    assert full == row_last["prompt_ids"] + row_last["response_ids"]              # same sequence, different split
    assert bytes(row_last["response_ids"]).decode() == "<|assistant|>\nfour<|end|>\n" and all(row_last["loss_mask"])
    text = bytes(row_all["response_ids"]).decode()
    masked_out = bytes(t for t, m in zip(row_all["response_ids"], row_all["loss_mask"]) if not m).decode()
    assert text.startswith("<|assistant|>") and "calc" in text and masked_out == "<|tool|>\n4<|end|>\n"   # only the tool turn carries no loss
    assert sft_data.tokenize_chat({"messages": [{"role": "user", "content": "x"}]}, tok, 4096) is None      # nothing to learn
    recs = [chat, {"instruction": "add", "input": "1 2", "output": "3"}, {"prompt_ids": [1, 2, 3], "response_ids": [4, 5]},
            {"instruction": "long", "output": "y" * 5000}]
    rows, st = sft_data.tokenize_dataset(recs, tok, 512, "all", str(tmp_path / "cache"))
    assert st["rows"] == 3 and st["dropped"] == 1 and st["cache"] == "miss" and st["len_max"] <= 512
    assert sft_data.tokenize_dataset(recs, tok, 512, "all", str(tmp_path / "cache"))[1]["cache"] == "hit"
    assert sft_data.tokenize_dataset(recs, tok, 512, "last", str(tmp_path / "cache"))[1]["cache"] == "miss"  # another key

    events = []

    class Spy:
        def on_train_begin(self, **kw):
            events.append("begin")

        def on_step_end(self, metrics, **kw):
            events.append(("step", round(metrics["sft/loss"], 3)))

        def on_eval_end(self, metrics, **kw):
            events.append(("eval", metrics["eval/loss"]))

        def on_train_end(self, **kw):
            events.append("end")

    train = [dict(chat), {"instruction": "add", "input": "1 2", "output": "3"}] * 4
    cfg = SFTConfig(model="tiny-qwen3", batch_size=4, num_steps=6, epochs=10, max_seq_len=512, train_on="all", logger="jsonl",
                    eval_interval=3, export_path=str(tmp_path / "export"), tokenize_cache_dir=str(tmp_path / "cache"),
                    optimizer=OptimizerConfig(lr=2e-3))
    tr = SFTTrainer(cfg, train, device="cpu", tokenizer=tok, eval_examples=[chat], callbacks=[Spy()])
    assert tr.data_stats["rows"] == 8
    tr.train()
    evals = [e[1] for e in events if isinstance(e, tuple) and e[0] == "eval"]
    assert events[0] == "begin" and events[-1] == "end" and len(evals) == 3 and evals[-1] < evals[0]
    assert sum(1 for e in events if isinstance(e, tuple) and e[0] == "step") == 6
    assert (tmp_path / "export" / "global_step_6" / "model.safetensors").exists()
    # timing mode: synthetic rows, no data
    tr2 = SFTTrainer(SFTConfig(model="tiny-qwen3", batch_size=2, max_seq_len=64, dummy_steps=2, logger="jsonl"), [], device="cpu")
    tr2.train()
    assert tr2.global_step == 2


def test_generator_utils_metrics_filtering_chat_masks_and_stepwise_merge(tmp_path):
    from skyrl_isoexec_b200.train import generator_utils as GU

    # trajectory- and token-level rewards
    m = GU.get_metrics_from_generator_output({"rewards": [1.0, 0.0, -1.0, 0.0]}, ["a", "a", "b", "b"])
    assert m == {"avg_score": 0.0, "mean_positive_reward": 0.25, "pass_at_n": 0.5}
    m = GU.get_metrics_from_generator_output({"rewards": [[0.0, 1.0], [0.5, -0.5], [0.0, 0.0]]}, ["a", "a", "b"])
    assert m["avg_score"] == pytest.approx(1 / 3) and m["pass_at_n"] == 0.5 and m["mean_positive_reward"] == pytest.approx(0.5)
    with pytest.raises(ValueError):
        GU.get_metrics_from_generator_output({"rewards": []}, [])
    assert GU.apply_overlong_filtering([[1, 1], [1, 0, 1]], ["stop", "length"]) == [[1, 1], [0, 0, 0]]
    assert GU.compute_turn_token_counts([[1, 1, 0, 0, 1], [0, 0], [], [0, 1, 1, 1]]) == [2, 1, 3]
    # chat templates
    assert "im_start" in GU.get_custom_chat_template({"source": "name", "name_or_path": "qwen3_with_thinking"})
    f = tmp_path / "t.jinja"
    f.write_text("{{ messages }}")
    assert GU.get_custom_chat_template({"source": "file", "name_or_path": str(f)}) == "{{ messages }}"
    assert GU.get_custom_chat_template(None) is None
    with pytest.raises(ValueError):
        GU.get_custom_chat_template({"source": "name", "name_or_path": "nope"})

    class ByteTok:
        def encode(self, text):
            return list(text.encode())

    tok = ByteTok()
    gen = GU.get_generation_prompt_ids(tok)
    assert bytes(gen).decode() == "<|assistant|>\n"
    msgs = [{"role": "assistant", "content": "let me look"}, {"role": "user", "content": "<observation>4</observation>"},
            {"role": "assistant", "content": "four"}]
    lp = [[-0.1] * len("let me look"), [-0.2] * len("four")]
    ids, mask, lps = GU.get_response_ids_and_loss_mask_from_messages(msgs, tok, lp)
    text = bytes(ids).decode()
    assert text == "<|assistant|>\nlet me look<|end|>\n<|user|>\n<observation>4</observation><|end|>\n<|assistant|>\nfour<|end|>\n"
    trained = bytes(t for t, k in zip(ids, mask) if k).decode()
    assert trained == "let me lookfour" and len(lps) == len(ids)
    assert [round(x, 1) for x, k in zip(lps, mask) if k] == [-0.1] * 11 + [-0.2] * 4 and all(x == 0.0 for x, k in zip(lps, mask) if not k)
    assert bytes(GU.encode_messages_subset([msgs[1]], tok)).decode() == "<|user|>\n<observation>4</observation><|end|>\n"
    # step-wise rows of two trajectories back to one row each
    so = {"trajectory_ids": ["t0", "t1", "t0"], "is_last_step": [False, True, True],
          "prompt_token_ids": [[1, 2], [7], [1, 2, 3, 4, 9, 9]], "response_ids": [[3, 4], [8], [5]],
          "loss_masks": [[1, 1], [1], [1]], "rewards": [0.0, 1.0, 2.0], "stop_reasons": ["stop", "stop", "length"],
          "rollout_logprobs": [[-1.0, -2.0], [-3.0], [-4.0]]}
    mo = GU.merge_stepwise_output(so)
    assert mo["trajectory_ids"] == ["t0", "t1"] and mo["prompt_token_ids"] == [[1, 2], [7]]
    assert mo["response_ids"] == [[3, 4, 9, 9, 5], [8]] and mo["loss_masks"] == [[1, 1, 0, 0, 1], [1]]
    assert mo["rollout_logprobs"] == [[-1.0, -2.0, 0.0, 0.0, -4.0], [-3.0]] and mo["rewards"] == [2.0, 1.0]
    assert mo["stop_reasons"] == ["length", "stop"]
    bad = dict(so, prompt_token_ids=[[1, 2], [7], [1, 2, 5, 5, 9]])
    with pytest.raises(ValueError):
        GU.merge_stepwise_output(bad)


def test_samples_of_one_prompt_share_recurrent_state_in_a_hybrid_model():
    """GatedDeltaNet layers: the siblings of a prompt start from the leader's recurrent state, snapshotted when its
    prefill reaches the shared boundary. Greedy outputs and logprobs equal the unshared run, the sampled run's logprobs
    equal the trainer's forward, snapshots and state rows are all given back."""
    from skyrl_isoexec_b200.core.testing import count_bit_mismatches
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import SamplingParams
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    cfg = get_config("tiny-hybrid")
    model = DecoderLM(cfg, device="cpu", seed=6)
    g = torch.Generator().manual_seed(8)
    base = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (300, 140)]
    prompts = [p for p in base for _ in range(3)]

    def run(share, sp, budget=512):
        eng = LLMEngine(model, EngineConfig(max_num_seqs=6, num_kv_pages=30, max_num_batched_tokens=budget, share_recurrent_state=share))
        outs = eng.generate(prompts, sp)
        assert eng.cache.allocator.num_free == 30 and not eng.gdn_state.snapshots and not eng.gdn_state.row_of
        return eng, outs

    greedy = SamplingParams(max_generate_length=8, ignore_eos=True, temperature=0.0)
    e0, o0 = run(False, greedy)
    e1, o1 = run(True, greedy)
    assert e0.scheduler.shared_prompt_tokens == 0 and e1.scheduler.shared_prompt_tokens == 2 * (256 + 128)
    assert [o.response_ids for o in o0] == [o.response_ids for o in o1]
    assert [o.response_logprobs for o in o0] == [o.response_logprobs for o in o1]
    e2, o2 = run(True, greedy, budget=200)                        # the leader reaches the boundary over several chunks
    assert [o.response_logprobs for o in o2] == [o.response_logprobs for o in o0]
    e3, o3 = run(True, SamplingParams(max_generate_length=9, ignore_eos=True))
    seq, att, rmask = build_sequences([o.prompt_ids for o in o3], [o.response_ids for o in o3])
    lp = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=1024)).forward(
        TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask}))
    ro = torch.zeros_like(lp)
    for i, o in enumerate(o3):
        ro[i, :len(o.response_logprobs)] = torch.tensor(o.response_logprobs)
    assert count_bit_mismatches((lp * rmask).contiguous(), (ro * rmask).contiguous()) == 0


def test_sampling_penalties_min_tokens_and_logit_bias():
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import Sampler, SamplingParams, isoexec_sampling_constraints, needs_history
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM

    sam = Sampler("cpu", seed=0)
    logits = torch.cat([torch.tensor([[2.0, 1.0, -1.0, 0.5, 0.0]]), torch.full((1, 11), -3.0)], 1)     # 16 wide: at least one token per leaf
    greedy = lambda **kw: SamplingParams(temperature=0.0, **kw)
    pick = lambda p, hist=None, eos=None: int(sam(logits, [p], histories=[hist] if hist is not None else None, eos_token_id=eos)[0][0])
    assert pick(greedy()) == 0
    assert pick(greedy(repetition_penalty=4.0), ([0], [])) == 1                       # 2.0 / 4 < 1.0
    assert pick(greedy(repetition_penalty=4.0), ([2], [])) == 0                       # a negative logit gets more negative
    assert pick(greedy(presence_penalty=1.5), ([0], [])) == 0                         # the prompt does not count for presence
    assert pick(greedy(presence_penalty=1.5), ([], [0])) == 1
    assert pick(greedy(frequency_penalty=0.6), ([], [0])) == 0 and pick(greedy(frequency_penalty=0.6), ([], [0, 0])) == 1
    assert pick(greedy(logit_bias={3: 5.0})) == 3
    assert pick(greedy(min_tokens=2), ([], [4]), eos=0) == 1 and pick(greedy(min_tokens=1), ([], [4]), eos=0) == 0
    assert pick(greedy(min_tokens=2, stop_token_ids=(1,)), ([], []), eos=0) == 3
    # the reported logprob is the raw one whatever shaped the draw
    tok, lp = sam(logits, [greedy(logit_bias={3: 5.0})])
    assert abs(float(lp[0]) - float(torch.log_softmax(logits[0], -1)[3])) < 1e-6
    with pytest.raises(ValueError, match="histories"):
        sam(logits, [greedy(repetition_penalty=2.0)])
    assert needs_history(SamplingParams(min_tokens=1)) and not needs_history(SamplingParams(logit_bias={1: 1.0}))
    with pytest.raises(ValueError):
        isoexec_sampling_constraints(SamplingParams(repetition_penalty=1.1))
    assert SamplingParams.from_dict({"logit_bias": {"7": 2}}).logit_bias == {7: 2.0}
    # through the engine: a heavy repetition penalty makes every greedy token new; min_tokens holds the end of sequence back
    eng = LLMEngine(DecoderLM(get_config("tiny-qwen3"), seed=0), EngineConfig(num_kv_pages=8, seed=1, eos_token_id=7))
    prompt = [5, 6, 7, 8]
    plain = eng.generate([prompt], SamplingParams(max_generate_length=24, temperature=0.0, ignore_eos=True))[0].response_ids
    pen = eng.generate([prompt], SamplingParams(max_generate_length=24, temperature=0.0, ignore_eos=True, repetition_penalty=1e6))[0].response_ids
    assert len(set(pen)) == len(pen) and not set(pen) & set(prompt) and len(set(plain)) < len(plain)
    forced = SamplingParams(max_generate_length=12, temperature=0.0, logit_bias={7: 1e4})
    assert eng.generate([prompt], forced)[0].response_ids == [7]                      # the biased end-of-sequence token ends it at once
    held = SamplingParams(max_generate_length=12, temperature=0.0, logit_bias={7: 1e4}, min_tokens=5)
    out = eng.generate([prompt], held)[0]
    assert len(out.response_ids) == 6 and out.response_ids[-1] == 7 and 7 not in out.response_ids[:5] and out.stop_reason == "stop"


def test_prompt_logprobs_are_the_scoring_forwards_bits_across_prefill_chunks():
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import SamplingParams
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    m = DecoderLM(get_config("tiny-qwen3"), seed=0)
    eng = LLMEngine(m, EngineConfig(num_kv_pages=16, seed=1, max_num_batched_tokens=48))       # prompts are prefilled in pieces
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(5, 500, (n,), generator=g).tolist() for n in (130, 61, 7)]
    outs = eng.generate(prompts + [prompts[0]], [SamplingParams(max_generate_length=3, ignore_eos=True, prompt_logprobs=1)] * 3
                        + [SamplingParams(max_generate_length=3, ignore_eos=True)])
    assert outs[3].prompt_logprobs is None and eng.scheduler.shared_prompt_tokens == 0           # such requests compute every prompt row
    w = PolicyWorker(m, WorkerConfig(max_tokens_per_microbatch=4096))
    for p, o in zip(prompts, outs):
        assert o.prompt_logprobs[0] is None and len(o.prompt_logprobs) == len(p)
        # score tokens 1.. of the prompt as a "response" to its first token
        seq, att, rmask = build_sequences([p[:1]], [p[1:]])
        lp = w.forward(TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask}))[0]
        got = torch.tensor(o.prompt_logprobs[1:])
        assert torch.equal(got.view(torch.int32), lp.view(torch.int32))


def test_rope_scaling_tables_match_the_transformers_formulas_and_extend_the_context():
    from transformers import LlamaConfig
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS

    from skyrl_isoexec_b200.models.config import ModelConfig, get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.ops.functional import RopeTable, scaled_inv_freq

    D, theta, maxp = 64, 10000.0, 4096
    cases = [{"rope_type": "linear", "factor": 4.0},
             {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 1024},
             {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 1024},
             {"rope_type": "yarn", "factor": 16.0, "original_max_position_embeddings": 1024, "beta_fast": 32, "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 0.5}]
    for sc in cases:
        hf = LlamaConfig(hidden_size=D * 4, num_attention_heads=4, head_dim=D, max_position_embeddings=maxp, rope_parameters=dict(sc, rope_theta=theta))
        want_inv, want_att = ROPE_INIT_FUNCTIONS[sc["rope_type"]](hf, "cpu")
        inv, att = scaled_inv_freq(D, theta, sc, maxp)
        assert torch.allclose(inv.float(), want_inv.float(), rtol=1e-5, atol=1e-9), sc
        assert abs(att - float(want_att)) < 1e-6, sc
    plain, lin = RopeTable(D, 64, theta, "cpu"), RopeTable(D, 64, theta, "cpu", scaling={"type": "linear", "factor": 2.0})
    assert torch.allclose(lin.cos[8], plain.cos[4], atol=1e-6) and plain.attention_factor == 1.0       # position 8 at half speed is position 4
    yarn = RopeTable(D, 64, theta, "cpu", scaling=cases[2])
    assert abs(float(yarn.cos[0, 0]) - yarn.attention_factor) < 1e-6 and yarn.attention_factor > 1.0  # cos(0) carries the attention factor
    with pytest.raises(ValueError, match="not implemented"):
        RopeTable(D, 64, theta, "cpu", scaling={"type": "dynamic", "factor": 2.0})
    # through the model config: hashable, exported, and a rollout still scores to the trainer's bits
    cfg = get_config("tiny-qwen3", rope_scaling=cases[2], max_position=1024)
    assert isinstance(cfg.rope_scaling, tuple) and hash(cfg) and ModelConfig.from_dict(cfg.to_dict()) == cfg
    from skyrl_isoexec_b200.models.hf_export import hf_config

    assert hf_config(cfg)["rope_scaling"]["rope_type"] == "yarn"
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import SamplingParams
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    m = DecoderLM(cfg, seed=0)
    assert not torch.equal(m.rope.cos, DecoderLM(get_config("tiny-qwen3", max_position=1024), seed=0).rope.cos)
    p = torch.randint(5, 500, (20,), generator=torch.Generator().manual_seed(0)).tolist()
    o = LLMEngine(m, EngineConfig(num_kv_pages=8, seed=1)).generate([p], SamplingParams(max_generate_length=6, ignore_eos=True))[0]
    seq, att, rmask = build_sequences([p], [o.response_ids])
    lp = PolicyWorker(m, WorkerConfig()).forward(TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask}))[0]
    assert torch.equal(lp.view(torch.int32), torch.tensor(o.response_logprobs).view(torch.int32))
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig

    c = SkyRLTrainConfig.from_cli_overrides(['trainer.rope_scaling={"rope_type": "yarn", "factor": 4.0}'])
    assert c.trainer.policy.model_overrides == {"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}


def test_sft_with_lora_lowers_the_loss_and_leaves_the_base_alone(tmp_path):
    from skyrl_isoexec_b200.models import hf_export
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM

    g = torch.Generator().manual_seed(0)
    ex = [{"prompt_ids": torch.randint(0, 200, (6,), generator=g).tolist(), "response_ids": torch.randint(0, 200, (10,), generator=g).tolist()} for _ in range(8)]
    donor = DecoderLM(get_config("tiny-qwen3"), seed=5)
    hf_export.save_hf(donor, str(tmp_path / "init"))
    cfg = SFTConfig(model="tiny-qwen3", batch_size=8, logger="jsonl", num_steps=6, epochs=6, lora_rank=4, lora_alpha=8.0, hf_path=str(tmp_path / "init"),
                    export_path=str(tmp_path / "out"))
    cfg.optimizer.lr = 2e-2
    tr = SFTTrainer(cfg, ex, device="cpu")
    assert torch.equal(tr.model.store.flat, donor.store.flat)                  # started from the given weights
    first = tr.evaluate_rows(ex) if hasattr(tr, "evaluate_rows") else None
    tr.eval_examples = tr.examples
    before = tr.evaluate()
    tr.train()
    after = tr.evaluate()
    assert list(after.values())[0] < list(before.values())[0] and first is None          # mean negative log-likelihood went down
    ad = tr.lora_store.adapters["sft"]
    assert tr.global_step == 6 and any(float(b.abs().sum()) > 0 for b in ad.B.values()) and tr.worker.opt.step_count == 0
    merged = dict(tr.model.named_weights())
    for n, t in donor.named_weights():
        if n in ad.A:
            assert torch.allclose(merged[n], t + ad.delta(n), atol=1e-6)
        else:
            assert torch.equal(merged[n], t)
    # the export holds the merged weights
    back = DecoderLM(get_config("tiny-qwen3"), seed=99)
    hf_export.load_hf(back, str(tmp_path / "out" / f"global_step_{tr.global_step}"))
    assert torch.equal(back.store.flat, tr.model.store.flat)


def test_policy_starts_from_a_sharded_hugging_face_checkpoint_directory(tmp_path):
    import json as _json

    from safetensors.torch import save_file

    from skyrl_isoexec_b200.models import hf_export
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM

    donor = DecoderLM(get_config("tiny-qwen3", tie_embeddings=False), seed=21)
    d = tmp_path / "ckpt"
    hf_export.save_hf(donor, str(d))
    # re-cut the single file into two shards with an index, as released checkpoints come
    from safetensors.torch import load_file

    sd = load_file(str(d / "model.safetensors"))
    (d / "model.safetensors").unlink()
    keys = sorted(sd)
    parts = {"model-00001-of-00002.safetensors": keys[: len(keys) // 2], "model-00002-of-00002.safetensors": keys[len(keys) // 2:]}
    for fn, ks in parts.items():
        save_file({k: sd[k].contiguous() for k in ks}, str(d / fn), metadata={"format": "pt"})
    (d / "model.safetensors.index.json").write_text(_json.dumps({"metadata": {}, "weight_map": {k: fn for fn, ks in parts.items() for k in ks}}))
    assert hf_export.has_hf_weights(str(d))
    fresh = DecoderLM(get_config(str(d)), seed=0)
    assert hf_export.load_hf(fresh, str(d)) > 0 and torch.equal(fresh.store.flat, donor.store.flat)
    (d / "model.safetensors.index.json").unlink()                           # without an index the shard files are looked through
    again = DecoderLM(get_config(str(d)), seed=1)
    hf_export.load_hf(again, str(d))
    assert torch.equal(again.store.flat, donor.store.flat)
    # the trainer: the directory is the model name; config and weights both come from it
    tr = RayPPOTrainer(_rl_cfg(str(tmp_path / "run"), 1, f"trainer.policy.model={d}", "trainer.policy.optimizer_config.lr=0.0"), device="cpu")
    tr.build_models()
    assert torch.equal(tr.policy.model.store.flat, donor.store.flat) and torch.equal(tr.policy.opt.master, donor.store.flat)


def test_engine_stops_at_the_tokenizers_end_of_sequence_token():
    from skyrl_isoexec_b200.engine.interface import NativeInferenceEngine
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import SamplingParams
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM

    class Tok:
        eos_token_id = 42

        def decode(self, ids, **kw):
            return " ".join(map(str, ids))

    eng = LLMEngine(DecoderLM(get_config("tiny-qwen3"), seed=0), EngineConfig(num_kv_pages=8, seed=1))
    assert eng.cfg.eos_token_id is None
    NativeInferenceEngine(eng, Tok())
    assert eng.cfg.eos_token_id == 42
    out = eng.generate([[5, 6, 7]], SamplingParams(max_generate_length=20, temperature=0.0, logit_bias={42: 1e4}))[0]
    assert out.response_ids == [42] and out.stop_reason == "stop"
    out = eng.generate([[5, 6, 7]], SamplingParams(max_generate_length=4, temperature=0.0, logit_bias={42: 1e4}, ignore_eos=True))[0]
    assert out.response_ids == [42] * 4 and out.stop_reason == "length"


def _hf_fast_tokenizer():
    """A Hugging Face fast tokenizer built in memory (word level, with a chat template)."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    words = ["<unk>", "<eos>", "<|user|>", "<|assistant|>", "<|system|>", "hello", "world", "two", "plus", "four", "is"]
    tk = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tk.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    t = PreTrainedTokenizerFast(tokenizer_object=tk, unk_token="<unk>", eos_token="<eos>")
    t.chat_template = ("{% for m in messages %}<|{{ m['role'] }}|> {{ m['content'] }} <eos> {% endfor %}"
                       "{% if add_generation_prompt %}<|assistant|> {% endif %}")
    return t


def test_chat_ids_with_a_hugging_face_tokenizer():
    """``apply_chat_template(tokenize=True)`` of recent transformers returns a mapping, not a list: every place that
    tokenises a conversation must still get the flat id list."""
    from skyrl_isoexec_b200.engine.renderer import render_conversation
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.train.generator_utils import get_generation_prompt_ids
    from skyrl_isoexec_b200.train.sft_data import tokenize_record
    from skyrl_isoexec_b200.utils.tokenizer import chat_ids

    t = _hf_fast_tokenizer()
    msgs = [{"role": "user", "content": "two plus two"}]
    ids = chat_ids(t, msgs)
    assert ids == [2, 7, 8, 7, 1, 3] and all(isinstance(i, int) for i in ids)
    assert chat_ids(t, msgs, False) == [2, 7, 8, 7, 1]
    assert get_generation_prompt_ids(t) == [3]
    r = render_conversation(msgs, t, get_config("tiny-qwen3"))
    assert list(r["token_ids"]) == ids and r["features"] is None
    ex = tokenize_record({"messages": msgs + [{"role": "assistant", "content": "is four"}]}, t, max_length=64)
    assert ex is not None and ex["prompt_ids"] == [2, 7, 8, 7, 1] and ex["response_ids"] == [3, 10, 9, 1] and sum(ex["loss_mask"]) == 4


def test_observations_in_mid_context_do_not_repeat_the_template_preamble():
    from skyrl_isoexec_b200.utils.tokenizer import ByteTokenizer, chat_ids, chat_ids_continuation

    t = _hf_fast_tokenizer()
    # a template that injects a default system turn when the conversation does not start with one (as Qwen's does)
    t.chat_template = ("{% if messages[0]['role'] != 'system' %}<|system|> hello world <eos> {% endif %}"
                       "{% for m in messages %}<|{{ m['role'] }}|> {{ m['content'] }} <eos> {% endfor %}"
                       "{% if add_generation_prompt %}<|assistant|> {% endif %}")
    obs = [{"role": "user", "content": "is four"}]
    alone = chat_ids(t, obs)
    assert alone[:4] == [4, 5, 6, 1]                                   # the preamble
    assert chat_ids_continuation(t, obs) == [2, 10, 9, 1, 3]           # the turn and the generation prompt only
    b = ByteTokenizer()
    assert chat_ids_continuation(b, obs) == chat_ids(b, obs)           # no preamble: the same ids as before


def test_rl_step_with_a_hugging_face_tokenizer_directory(tmp_path):
    """``trainer.policy.tokenizer_path=<dir>``: chat prompts from a JSONL file are rendered by the directory's chat template,
    a multi-turn environment's observations are appended as conversation turns, and the step stays bitwise on-policy."""
    import json

    from skyrl_isoexec_b200.train.entrypoints import main_base

    tok_dir = tmp_path / "tok"
    _hf_fast_tokenizer().save_pretrained(str(tok_dir))
    data = tmp_path / "train.jsonl"
    with open(data, "w") as f:
        for _ in range(8):
            f.write(json.dumps({"prompt": [{"role": "user", "content": "two plus two"}], "env_class": "gsm8k_multi_turn",
                                "reward_spec": {"ground_truth": "4"}}) + "\n")
    ov = ["trainer.policy.model=tiny-qwen3", f"trainer.policy.tokenizer_path={tok_dir}", f"data.train_data={data}",
          "environment.env_class=gsm8k_multi_turn", "generator.batched=false", "generator.max_turns=2",
          "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2", "generator.n_samples_per_prompt=2",
          "generator.sampling_params.max_generate_length=4", "trainer.max_prompt_length=32", "generator.max_input_length=64",
          "generator.inference_engine.num_kv_pages=16", "trainer.num_steps=1", "trainer.ckpt_interval=0"]
    tr = main_base.BasePPOExp(SkyRLTrainConfig.from_cli_overrides(ov)).run()
    assert tr.global_step == 1
    assert tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0
