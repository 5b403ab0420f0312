"""Algorithm core, batch containers, config overrides, scheduler behaviour, the full GRPO loop on
CPU, and checkpoint save / resume / reshard (no GPU)."""
import os

import pytest
import torch

from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
from skyrl_isoexec_b200.engine.sampler import SamplingParams, isoexec_sampling_constraints
from skyrl_isoexec_b200.models.config import get_config
from skyrl_isoexec_b200.models.decoder import DecoderLM
from skyrl_isoexec_b200.train import algorithms as alg
from skyrl_isoexec_b200.train import checkpoint as ckpt
from skyrl_isoexec_b200.train.batch import TensorBatch, TrainingInputBatch, build_sequences, pad_training_input_batch
from skyrl_isoexec_b200.train.config import SkyRLTrainConfig, validate_cfg
from skyrl_isoexec_b200.train.trainer import RayPPOTrainer


# ------------------------------------------------------------------ algorithms
def test_grpo_advantage_groups_and_single_sample():
    rewards = torch.zeros(5, 3)
    rewards[:, 2] = torch.tensor([1.0, 3.0, 2.0, 6.0, 5.0])
    mask = torch.ones(5, 3)
    adv, ret = alg.grpo_advantage(rewards, mask, ["a", "a", "b", "b", "c"])
    s = torch.tensor([1.0, 3.0]).std()
    assert torch.allclose(adv[0], torch.full((3,), float((1 - 2) / (s + 1e-6))))
    assert torch.allclose(adv[1], -adv[0]) and torch.allclose(adv[4], torch.full((3,), 5.0))   # single-sample group: mean 0, std 1
    adv2, _ = alg.grpo_advantage(rewards, mask, ["a", "a", "b", "b", "c"], grpo_norm_by_std=False)
    assert torch.allclose(adv2[3], torch.full((3,), 2.0))


def test_rloo_maxrl_reinforcepp_gae():
    r = torch.zeros(4, 2)
    r[:, 1] = torch.tensor([1.0, 2.0, 3.0, 6.0])
    m = torch.ones(4, 2)
    adv, _ = alg.rloo_advantage(r, m, ["a", "a", "a", "b"])
    assert torch.allclose(adv[0, 0], torch.tensor(1.0 - 2.5)) and adv[3, 0] == 0.0     # a group of one: advantage 0
    adv, _ = alg.maxrl_advantage(r, m, ["a", "a", "a", "b"])
    assert torch.allclose(adv[2, 0], torch.tensor((3.0 - 2.0) / (2.0 + 1e-6)))
    adv, ret = alg.reinforce_pp_advantage(r, m, gamma=1.0)
    assert torch.allclose(ret[:, 0], r[:, 1]) and abs(float((adv * m).sum())) < 1e-4
    adv, ret = alg.gae_advantage(r, m, values=torch.zeros(4, 2), gamma=1.0, lambd=1.0)
    assert torch.allclose(ret[:, 0], r[:, 1])


def test_policy_loss_regular_and_dual_clip_match_definition():
    torch.manual_seed(0)
    cfg = alg.AlgorithmConfig()
    lp = (torch.randn(4, 9) * 0.5).requires_grad_()
    old = lp.detach() + torch.randn(4, 9) * 0.4
    adv, mask = torch.randn(4, 9), (torch.rand(4, 9) > 0.3).float()
    loss, m = alg.ppo_policy_loss(lp, old, adv, cfg, loss_mask=mask)
    ratio = torch.exp(lp - old)
    ref = -torch.min(ratio * adv, ratio.clamp(0.8, 1.2) * adv)
    assert torch.allclose(loss, (ref * mask).sum(), atol=1e-5)
    loss2, _ = alg.dual_clip_policy_loss(lp, old, adv, cfg, loss_mask=mask)
    ref2 = torch.where(adv < 0, torch.min(-adv * 3.0, ref), ref)
    assert torch.allclose(loss2, (ref2 * mask).sum(), atol=1e-5)
    for name in ("sapo", "gspo", "cispo", "cross_entropy", "importance_sampling"):
        l, _ = alg.get_policy_loss(name)(lp, old, adv, cfg, loss_mask=mask, rollout_logprobs=old)
        (g,) = torch.autograd.grad(l, lp)
        assert torch.isfinite(l) and torch.isfinite(g).all()
    with pytest.raises(KeyError):
        alg.get_policy_loss("nope")


def test_on_policy_gradient_is_the_policy_gradient():
    lp = torch.randn(3, 5, requires_grad=True)
    adv, mask = torch.randn(3, 5), torch.ones(3, 5)
    loss, _ = alg.ppo_policy_loss(lp, lp.detach(), adv, alg.AlgorithmConfig(), loss_mask=mask)
    (g,) = torch.autograd.grad(loss, lp)
    assert torch.allclose(g, -adv)


def test_loss_reductions_and_kl():
    adv, mask = torch.ones(4, 6), torch.ones(4, 6)
    mask[0, 3:] = 0
    assert torch.allclose(alg.apply_loss_reduction_to_advantages(adv, mask, "token_mean") * mask, mask / mask.sum())
    sm = alg.apply_loss_reduction_to_advantages(adv, mask, "sequence_mean")
    assert torch.allclose((sm * mask).sum(), torch.tensor(1.0))
    assert torch.allclose(alg.apply_loss_reduction_to_advantages(adv, mask, "seq_mean_token_sum_norm", max_seq_len=6), adv / 24)
    pm = alg.apply_loss_reduction_to_advantages(adv, mask, "prompt_mean", prompt_boundaries=[(0, 2), (2, 4)])
    assert torch.allclose((pm * mask).sum(), torch.tensor(1.0))
    a, b = torch.randn(3, 4), torch.randn(3, 4)
    assert torch.allclose(alg.compute_approx_kl(a, b, kl_estimator_type="k1"), a - b)
    assert (alg.compute_approx_kl(a, b, kl_estimator_type="k3") >= 0).all()
    ctl = alg.AdaptiveKLController(0.1, 0.05, 100)
    ctl.update(0.2, 10)
    assert ctl.value > 0.1


def test_off_policy_correction():
    opc = alg.OffPolicyCorrection(tis_ratio_type="token", token_tis_ratio_clip_high=2.0, sequence_mask_metric="geometric")
    old = torch.zeros(2, 4)
    ro = torch.zeros(2, 4)
    ro[1] = -1.0
    w, mask, m = alg.compute_off_policy_correction(old, ro, torch.ones(2, 4), opc)
    assert torch.allclose(w[0], torch.ones(4)) and torch.allclose(w[1], torch.full((4,), 2.0))
    assert mask[0].sum() == 4 and mask[1].sum() == 0 and m["off_policy_masked_frac"] == 0.5


# ------------------------------------------------------------------ containers / config
def test_tensor_batch_ops_and_padding():
    b = TrainingInputBatch({"sequences": torch.arange(12).view(6, 2), "loss_mask": torch.ones(6, 2), "values": None})
    b.metadata["uids"] = list("abcdef")
    assert len(b) == 6 and [len(c) for c in b.chunk(3)] == [2, 2, 2]
    assert TensorBatch.cat(b.chunk(2))["sequences"].equal(b["sequences"])
    import pickle
    b2 = pickle.loads(pickle.dumps(b))
    assert b2["sequences"].equal(b["sequences"]) and b2.metadata["uids"] == list("abcdef") and b2["values"] is None
    p = pad_training_input_batch(b, 4)
    assert len(p) == 8 and p.metadata["pad_size"] == 2 and p["loss_mask"][6:].sum() == 0
    with pytest.raises(ValueError):
        TensorBatch({"a": torch.zeros(2), "b": torch.zeros(3)})
    seq, att, rm = build_sequences([[1, 2, 3], [4]], [[9], [8, 7]], pad_id=0)
    assert seq.tolist() == [[1, 2, 3, 9, 0], [0, 0, 4, 8, 7]] and att.sum(1).tolist() == [4, 3] and rm.tolist() == [[1, 0], [1, 1]]


def test_config_overrides_and_validation():
    cfg = SkyRLTrainConfig.from_cli_overrides(["trainer.algorithm.eps_clip_high=0.28", "generator.n_samples_per_prompt=8",
                                               "trainer.policy.model=qwen3-8b", "trainer.isoexec.enabled=false",
                                               "generator.sampling_params.temperature=0.7", "trainer.policy.model_overrides={\"num_layers\": 2}"])
    assert cfg.trainer.algorithm.eps_clip_high == 0.28 and cfg.generator.n_samples_per_prompt == 8
    assert cfg.trainer.policy.model_overrides == {"num_layers": 2}
    validate_cfg(cfg)
    with pytest.raises(KeyError):
        SkyRLTrainConfig.from_cli_overrides(["trainer.nonexistent=1"])
    with pytest.raises(ValueError):
        SkyRLTrainConfig.from_cli_overrides(["+trainer.x=1"])
    bad = SkyRLTrainConfig.from_cli_overrides(["generator.sampling_params.temperature=0.7"])
    with pytest.raises(ValueError, match="isoexec"):
        validate_cfg(bad)
    with pytest.raises(ValueError):
        isoexec_sampling_constraints(SamplingParams(top_k=50))


# ------------------------------------------------------------------ engine scheduling
def test_scheduler_preempts_and_recomputes_with_identical_logprobs():
    cfg = get_config("tiny-qwen3")
    model = DecoderLM(cfg)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (100,), generator=g).tolist() for _ in range(4)]
    sp = SamplingParams(max_generate_length=60, ignore_eos=True)
    roomy = LLMEngine(model, EngineConfig(max_num_seqs=8, num_kv_pages=16, seed=11))
    tight = LLMEngine(model, EngineConfig(max_num_seqs=8, num_kv_pages=5, seed=11, max_num_batched_tokens=64))
    a = roomy.generate(prompts, sp)
    b = tight.generate(prompts, sp)
    assert tight.cache.allocator.num_free == 5 and roomy.cache.allocator.num_free == 16
    assert tight.scheduler.preemptions > 0 and roomy.scheduler.preemptions == 0
    assert all(len(o.response_ids) == 60 and len(o.response_logprobs) == 60 for o in a + b)
    # a preempted sequence is recomputed from its tokens; the logprobs it reported before and after
    # the preemption must all equal what a clean scoring forward gives, bit for bit
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    worker = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=4096))
    for outs in (a, b):
        seq, att, rmask = build_sequences([o.prompt_ids for o in outs], [o.response_ids for o in outs])
        lp = worker.forward(TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask}))
        ro = torch.tensor([o.response_logprobs for o in outs])
        assert torch.equal(lp.view(torch.int32), ro.view(torch.int32))


# ------------------------------------------------------------------ full loop + checkpoints
def _cfg(tmp, steps, extra=()):
    return SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
        "generator.n_samples_per_prompt=4", "generator.sampling_params.max_generate_length=24",
        "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=16", "data.synthetic_prompts=32",
        "trainer.max_prompt_length=16", "generator.inference_engine.num_kv_pages=32",
        "trainer.policy.optimizer_config.lr=1e-3", f"trainer.num_steps={steps}", f"trainer.ckpt_path={tmp}",
        "trainer.ckpt_interval=2", "trainer.logger=jsonl", *extra])


def test_grpo_loop_is_bitwise_on_policy_and_resumes(tmp_path):
    d = str(tmp_path / "ck")
    tr = RayPPOTrainer(_cfg(d, 3), device="cpu")
    tr.train()
    assert tr.global_step == 3
    assert tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0
    assert tr.all_metrics["policy/grad_norm"] > 0
    assert sorted(os.listdir(d + "/global_step_2")) == ["data.pt", "policy", "trainer_state.pt"]
    assert open(d + "/latest_ckpt_global_step.txt").read() == "2"
    assert {"metadata.json", "__0_0.distcp"} <= set(os.listdir(d + "/global_step_2/policy"))
    assert os.path.exists(d + "/enforcement.trainer.r0.json") and os.path.exists(d + "/enforcement.engine.r0.json")
    # resume picks up step 2 and continues to 3 with the same parameters as the uninterrupted run had at step 2
    tr2 = RayPPOTrainer(_cfg(d, 3), device="cpu")
    tr2.build_models()
    assert tr2.load_checkpoints() == 2 and tr2.policy.opt.step_count == 2
    ref = torch.load(d + "/global_step_2/policy/__0_0.distcp", weights_only=False)["model"]
    for name, t in tr2.policy.model.named_weights():
        assert torch.equal(t, ref[name])


def test_checkpoint_helpers(tmp_path):
    d = str(tmp_path)
    assert ckpt.resolve_resume_path(d, "latest") is None and ckpt.resolve_resume_path(d, "none") is None
    with pytest.raises(ValueError):
        ckpt.resolve_resume_path(d, "from_path", d + "/not_a_step_dir")
    for s in (1, 2, 3):
        os.makedirs(f"{d}/global_step_{s}")
    assert ckpt.list_checkpoints(d) == [1, 2, 3]
    assert ckpt.cleanup_old_checkpoints(d, 2) == [1] and ckpt.list_checkpoints(d) == [2, 3]
    with pytest.raises(FileNotFoundError):
        ckpt.validate_checkpoint_dir(f"{d}/global_step_3")


def test_engine_stop_strings_end_a_sequence_at_the_first_match():
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import SamplingParams
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM

    assert SamplingParams.from_dict({"stop": "END"}).stop == ("END",) and SamplingParams.from_dict({"stop": None}).stop == ()
    prompt = [5, 6, 7, 8]

    def fresh():
        eng = LLMEngine(DecoderLM(get_config("tiny-qwen3"), seed=0), EngineConfig(max_num_seqs=4, num_kv_pages=16, seed=11))
        eng.detokenize = lambda ids: "".join(f"<{i}>" for i in ids)
        return eng

    free = fresh().generate([prompt], SamplingParams(max_generate_length=12, ignore_eos=True))[0]
    assert len(free.response_ids) == 12 and free.stop_reason == "length"
    target = free.response_ids[4]
    first = free.response_ids.index(target)
    out = fresh().generate([prompt], SamplingParams(max_generate_length=12, ignore_eos=True, stop=(f"<{target}>", "<never>")))[0]
    assert out.stop_reason == "stop" and out.response_ids == free.response_ids[:first + 1]      # same samples, cut at the match
    assert out.response_logprobs == free.response_logprobs[:first + 1]
    # without a detokenizer stop strings cannot be matched and are ignored
    eng = fresh()
    eng.detokenize = None
    assert len(eng.generate([prompt], SamplingParams(max_generate_length=6, ignore_eos=True, stop=(f"<{target}>",)))[0].response_ids) == 6


def test_forward_gate_ignores_observation_tokens_of_a_multi_turn_rollout(tmp_path):
    """Observation tokens sit inside response_mask with a placeholder rollout logprob of 0 and loss mask 0
    (train/generator.py agent_loop); the rollout-vs-train gate and its metrics must look at trained tokens only."""
    tr = RayPPOTrainer(_cfg(str(tmp_path / "ck"), 1, ["trainer.ckpt_interval=0"]), device="cpu")
    tr.build_models()
    tr.sync_weights()
    tr.engine.wake_up()
    gi, uids = tr.prepare_generator_input(next(iter(tr.loader)))
    go = tr.generate(gi)
    tr.engine.sleep()
    # splice an "observation" into the middle of every response: the tokens stay, their rollout logprob becomes the
    # placeholder 0.0 and their loss mask 0, exactly what the multi-turn loop emits
    for i in range(len(go["response_ids"])):
        for j in range(5, 9):
            go["loss_masks"][i][j] = 0
            go["rollout_logprobs"][i][j] = 0.0
    batch = tr.convert_to_training_input(go, uids)
    tr.global_step = 1
    batch = tr.fwd_logprobs_values_reward(batch)         # strict gate: would raise ForwardGateError on a mismatch
    m = tr.all_metrics
    assert m["policy/rollout_train_logprob_bit_mismatches"] == 0 and m["policy/rollout_train_logprobs_abs_diff_max"] == 0.0
    # all-masked batch: nothing to compare, nothing refuses
    batch["loss_mask"].zero_()
    tr.fwd_logprobs_values_reward(batch)
    assert tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0
    # the training-forward variant of the gate (scoring forward skipped) masks the same way
    batch = tr.convert_to_training_input(go, uids)
    batch["action_log_probs"] = batch["rollout_logprobs"].clone()
    batch["advantages"] = torch.zeros_like(batch["rollout_logprobs"])
    batch.metadata["check_rollout_bits"] = True
    out = tr.policy.forward_backward(batch)
    assert out["rollout_bits"]["mismatches"] == 0 and out["rollout_bits"]["tokens"] == float((batch["loss_mask"] > 0).sum())


def test_trainer_exports_a_dcp_checkpoint_and_resumes_from_it(tmp_path):
    """``trainer.dcp_save_interval`` writes a torch.distributed.checkpoint directory; ``resume_mode=from_path`` on it brings
    back the weights, the optimizer state and the step counter."""
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    ov = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
          "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8", "data.synthetic_prompt_len=12",
          "trainer.num_steps=2", "trainer.logger=jsonl", f"trainer.export_path={tmp_path}/export", "trainer.dcp_save_interval=2",
          f"trainer.ckpt_path={tmp_path}/ckpt", "trainer.ckpt_interval=0", "environment.env_class=even_tokens"]
    tr = RayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(ov), device="cpu")
    tr.build_models()
    tr.train()
    d = tmp_path / "export" / "global_step_2" / "dcp"
    assert (d / ".metadata").exists()
    tr2 = RayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(ov + ["trainer.resume_mode=from_path", f"trainer.resume_path={d}",
                                                                  "trainer.policy.seed=99"]), device="cpu")
    tr2.build_models()
    assert tr2.load_checkpoints() == 2 and tr2.policy.opt.step_count == tr.policy.opt.step_count
    for (n, a), (_, b) in zip(tr.policy.model.named_weights(), tr2.policy.model.named_weights()):
        assert torch.equal(a, b), n
    assert torch.equal(tr.policy.opt.exp_avg_sq, tr2.policy.opt.exp_avg_sq)


def test_reference_config_keys_are_wired_or_refused(tmp_path):
    """Keys carried over from the reference's config either do something or are refused: the contract artifact, the batch
    dump, per-mini-batch old logprobs, the debug trace; values that would be silently ignored raise."""
    import json

    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig, validate_cfg
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    base = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=2",
            "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=6", "data.synthetic_prompt_len=10",
            "trainer.num_steps=1", "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}/ckpt", "trainer.ckpt_interval=0",
            "environment.env_class=even_tokens"]
    ov = base + [f"trainer.isoexec.contract_path={tmp_path}/contract.json", "trainer.dump_data_batch=true",
                 "trainer.recompute_old_logprobs_per_minibatch=true", f"trainer.isoexec.debug_trace={tmp_path}/trace"]
    tr = RayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(ov), device="cpu")
    tr.build_models()
    calls = []
    real = tr.dispatch.forward
    tr.dispatch.forward = lambda name, b: (calls.append((name, b.batch_size)), real(name, b))[1]
    tr.train()
    from skyrl_isoexec_b200.debug import trace as _trace

    _trace.uninstall()
    doc = json.loads((tmp_path / "contract.json").read_text())
    assert doc and tr.adapter_trainer.contract is not None
    dumped = torch.load(tmp_path / "ckpt" / "dumped_data" / "global_step_1_rank0.pt", weights_only=False)
    assert dumped["tensors"]["sequences"].shape[0] == 8 and len(dumped["uids"]) == 8
    # two mini-batches: the batch is scored once, and the second mini-batch is re-scored under the moved policy
    assert calls == [("policy", 8), ("policy", 4)]
    assert any((tmp_path / "trace").iterdir())
    for bad in (["trainer.policy.parallel.sequence_parallel=true", "trainer.policy.parallel.context_parallel_size=2"],
                ["generator.inference_engine.data_parallel_size=2"],
                ["generator.inference_engine.run_engines_locally=false"], ["generator.use_conversation_multi_turn=false"]):
        with pytest.raises(ValueError):
            validate_cfg(SkyRLTrainConfig.from_cli_overrides(base + bad), 1)
    with pytest.raises(ValueError):
        validate_cfg(SkyRLTrainConfig.from_cli_overrides(base + ["trainer.placement.policy_num_gpus_per_node=4",
                                                                 "trainer.policy.parallel.tensor_model_parallel_size=1"]), 2)


def test_post_update_drift_metrics_are_zero_on_policy_and_positive_after_a_step(tmp_path):
    """With one mini-batch per batch the training forward IS the rollout policy: the drift metrics are exactly 0. With two
    mini-batches the second one is trained after an optimizer step and shows a positive drift."""
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    def run(mini):
        ov = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", f"trainer.policy_mini_batch_size={mini}",
              "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8", "data.synthetic_prompt_len=12",
              "trainer.num_steps=1", "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}/c{mini}", "trainer.ckpt_interval=0",
              "environment.env_class=even_tokens", "trainer.policy.optimizer_config.lr=1e-2"]
        tr = RayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(ov), device="cpu")
        tr.build_models()
        tr.train()
        return tr.all_metrics

    m = run(4)
    assert m["policy/post_update_rollout_logprobs_abs_diff_mean"] == 0.0 and m["policy/post_update_rollout_logprobs_abs_diff_max"] == 0.0
    m2 = run(2)
    assert m2["policy/post_update_rollout_logprobs_abs_diff_max"] > 0.0 and m2["policy/post_update_rollout_logprobs_abs_diff_std"] >= 0.0
