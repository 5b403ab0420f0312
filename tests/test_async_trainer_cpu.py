"""One-step-off-policy pipelining on CPU: the first batch is on-policy, every later batch is exactly one version old, the
generator never runs two batches ahead, and the command-line entry point builds both asynchronous trainers."""
import pytest
import torch

from skyrl_isoexec_b200.train.callbacks import TrainingCallback
from skyrl_isoexec_b200.train.config import SkyRLTrainConfig


def _cfg(tmp, steps, extra=()):
    return SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=6", "generator.sampling_params.ignore_eos=true",
        "data.synthetic_prompt_len=8", "data.synthetic_prompts=16", "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16",
        "generator.inference_engine.own_weights=true", f"trainer.num_steps={steps}", "trainer.logger=jsonl", f"trainer.ckpt_path={tmp}",
        "trainer.resume_mode=none", "trainer.policy.optimizer_config.lr=1e-3", *extra])


def test_one_step_off_trainer_trains_on_rollouts_one_version_old(tmp_path):
    from skyrl_isoexec_b200.train.async_trainer import AsyncRayPPOTrainer

    seen = []

    class Spy(TrainingCallback):
        def on_step_end(self, trainer, inp, control):
            m = inp.metrics
            seen.append((trainer.global_step, m["async/staleness"], m["policy/rollout_train_logprob_bit_mismatches"], trainer.policy_version))

    tr = AsyncRayPPOTrainer(_cfg(tmp_path, 4, ["trainer.eval_interval=2", "generator.eval_sampling_params.max_generate_length=4",
                                              "generator.eval_sampling_params.ignore_eos=true", "trainer.eval_batch_size=2"]),
                            device="cpu", callbacks=[Spy()])
    tr.train()
    assert tr.global_step == 4 and tr.policy_version == 4
    assert [s[1] for s in seen] == [0, 1, 1, 1]                          # the first batch is fresh, the others one step old
    assert seen[0][2] == 0                                                # the fresh batch scores to the rollout's bits
    assert any(s[2] > 0 for s in seen[1:])                                # a stale batch does not (the weights moved), and nothing refused it
    assert tr.separate_engine and torch.equal(tr.engine.model.store.flat, tr.policy.model.store.flat)     # the last sync published the last update
    assert tr.last_eval                                                   # evaluation ran between batches
    # refusals
    with pytest.raises(ValueError, match="own_weights"):
        AsyncRayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(["trainer.policy.model=tiny-qwen3"]), device="cpu")
    with pytest.raises(ValueError, match="model-parallel"):
        AsyncRayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(["trainer.policy.model=tiny-qwen3", "generator.inference_engine.own_weights=true",
                                                                "trainer.policy.parallel.tensor_model_parallel_size=2"]), device="cpu")


def test_generator_thread_failure_ends_training_with_its_error(tmp_path):
    from skyrl_isoexec_b200.train.async_trainer import AsyncRayPPOTrainer

    tr = AsyncRayPPOTrainer(_cfg(tmp_path, 3), device="cpu")
    tr.build_models()
    real, calls = tr.generate, []

    def flaky(gi):
        calls.append(1)
        if len(calls) == 2:
            raise RuntimeError("engine fell over")
        return real(gi)

    tr.generate = flaky
    with pytest.raises(RuntimeError, match="generation thread failed") as e:
        tr.train()
    assert "engine fell over" in str(e.value.__cause__) and tr.global_step <= 1      # it fails as soon as the trainer looks at the buffer


def test_async_entry_point_runs_both_modes(tmp_path):
    from skyrl_isoexec_b200.train.async_trainer import AsyncRayPPOTrainer
    from skyrl_isoexec_b200.train.entrypoints import main_async
    from skyrl_isoexec_b200.train.fully_async_trainer import FullyAsyncTrainer

    base = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2", "generator.n_samples_per_prompt=2",
            "generator.sampling_params.max_generate_length=4", "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8",
            "data.synthetic_prompts=8", "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.num_steps=2",
            "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}", "trainer.resume_mode=none"]
    tr = main_async.main(base + ["generator.inference_engine.own_weights=true"])
    assert isinstance(tr, AsyncRayPPOTrainer) and tr.global_step == 2
    tr = main_async.main(["--mode", "fully_async", "--max-staleness-steps", "2", "--generation-workers", "2"] + base)
    assert isinstance(tr, FullyAsyncTrainer) and tr.global_step == 2 and tr.acfg.max_staleness_steps == 2


def test_reference_config_keys_are_translated_accepted_or_refused_with_a_reason():
    from skyrl_isoexec_b200.train import config as C

    cfg = C.SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-qwen3", "trainer.policy.megatron_config.tensor_model_parallel_size=2", "trainer.algorithm.kl_ctrl.type=adaptive",
        "trainer.algorithm.dynamic_sampling.type=filter", "trainer.algorithm.use_tis=true", "trainer.algorithm.tis_imp_ratio_cap=3.0",
        "trainer.policy.optimizer_config.adam_betas=[0.9,0.95]", "trainer.gradient_checkpointing=false", "trainer.policy.fsdp_config.cpu_offload=true",
        "environment.skyrl_gym.search.search_url=http://127.0.0.1:8000/retrieve", "environment.skyrl_gym.search.topk=5", "trainer.rope_theta=500000",
        "generator.chat_template.source=name", "generator.chat_template.name_or_path=qwen3_with_thinking", "trainer.max_training_steps=7",
        "trainer.critic.optimizer_config.lr=1e-5", "trainer.fully_async.max_staleness_steps=2", "trainer.policy.model.lora.rank=0",
        "trainer.policy.model.lora.alpha=16", "generator.vision_language_generator=false", "data.train_data=none", "trainer.policy.sequence_parallel_size=1"])
    t = cfg.trainer
    assert (t.policy.model, t.policy.parallel.tensor_model_parallel_size, t.algorithm.kl_ctrl_type, t.algorithm.dynamic_sampling_type) == ("tiny-qwen3", 2, "adaptive", "filter")
    assert t.algorithm.off_policy_correction.tis_ratio_type == "token" and t.algorithm.off_policy_correction.token_tis_ratio_clip_high == 3.0
    assert t.policy.optimizer_config.beta2 == 0.95 and t.policy.keep_last_layers == -1 and t.num_steps == 7 and cfg.data.train_data == []
    assert cfg.environment.env_kwargs == {"search_url": "http://127.0.0.1:8000/retrieve", "topk": 5} and t.policy.model_overrides == {"rope_theta": 500000}
    assert cfg.generator.chat_template == {"source": "name", "name_or_path": "qwen3_with_thinking"}
    assert t.critic.optimizer_config.lr == 1e-5 and t.fully_async.max_staleness_steps == 2
    assert any("fsdp_config.cpu_offload" in n for n in C.COMPAT_NOTES)
    assert C.SkyRLTrainConfig.from_cli_overrides(["trainer.policy.model.lora.rank=8"]).trainer.policy.lora.rank == 8
    for bad, why in (("trainer.ref.model.lora.rank=8", "LoRA"), ("generator.inference_engine.num_prefill=2", "disaggregation"),
                     ("generator.inference_engine.enable_pd=true", "disaggregation"), ("trainer.policy.megatron_config.expert_tensor_parallel_size=2", "expert parallelism only")):
        with pytest.raises(ValueError, match=why):
            C.SkyRLTrainConfig.from_cli_overrides([bad])
    with pytest.raises(KeyError):
        C.SkyRLTrainConfig.from_cli_overrides(["trainer.nope=1"])
    # the same through a YAML file in the reference's nesting
    import yaml

    tree = {"trainer": {"policy": {"model": {"path": "tiny-qwen3", "lora": {"rank": 0}}, "fsdp_config": {"cpu_offload": False, "mixed_precision": {"param_dtype": "bf16"}}},
                        "algorithm": {"kl_ctrl": {"type": "fixed", "kl_target": 0.2}, "sapo": {"tau_pos": 1.5}}, "fully_async": {"enabled": False}},
            "generator": {"inference_engine": {"vllm_v1_disable_multiproc": True, "engine_init_kwargs": {"a": 1}}},
            "environment": {"skyrl_gym": {"max_env_workers": 8, "text2sql": {"db_path": "/data/sql"}}}}
    import tempfile

    with tempfile.NamedTemporaryFile("w", suffix=".yaml", delete=False) as f:
        yaml.safe_dump(tree, f)
    cfg = C.SkyRLTrainConfig.from_file(f.name)
    assert cfg.trainer.algorithm.kl_target == 0.2 and cfg.trainer.algorithm.sapo_tau_pos == 1.5 and cfg.environment.env_kwargs == {"db_path": "/data/sql"}


def test_critic_has_its_own_config_and_the_plain_entry_point_honours_fully_async(tmp_path):
    from skyrl_isoexec_b200.train.entrypoints import main_base
    from skyrl_isoexec_b200.train.fully_async_trainer import FullyAsyncTrainer
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    base = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2", "generator.n_samples_per_prompt=2",
            "generator.sampling_params.max_generate_length=4", "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8",
            "data.synthetic_prompts=8", "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.num_steps=1",
            "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}", "trainer.resume_mode=none"]
    cfg = SkyRLTrainConfig.from_cli_overrides(base + ["trainer.algorithm.advantage_estimator=gae", "trainer.critic.optimizer_config.lr=3e-4",
                                                      'trainer.critic.model_overrides={"num_layers": 1}', "trainer.critic_mini_batch_size=1",
                                                      "trainer.logprobs_chunk_size=16"])
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.train()
    assert tr.critic.cfg.optimizer.lr == 3e-4 and tr.policy.cfg.optimizer.lr != 3e-4 and tr.critic.model.cfg.num_layers == 1
    assert tr.policy.cfg.logprob_chunk_rows == 16 and tr.critic.opt.step_count == 2            # two critic mini-batches of one prompt each
    exp = main_base.BasePPOExp(SkyRLTrainConfig.from_cli_overrides(base + ["trainer.fully_async.enabled=true", "trainer.fully_async.max_staleness_steps=3",
                                                                           "trainer.fully_async.num_parallel_generation_workers=2"]))
    trainer = exp.get_trainer()
    assert isinstance(trainer, FullyAsyncTrainer) and trainer.acfg.max_staleness_steps == 3 and trainer.acfg.num_parallel_generation_workers == 2


def test_batch_normalised_advantages_zero_variance_filter_and_reference_refresh(tmp_path):
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    base = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2", "generator.n_samples_per_prompt=2",
            "generator.sampling_params.max_generate_length=4", "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8",
            "data.synthetic_prompts=4", "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.epochs=2",
            "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}", "trainer.resume_mode=none", "trainer.policy.optimizer_config.lr=1e-3"]
    cfg = SkyRLTrainConfig.from_cli_overrides(base + ["trainer.algorithm.advantage_batch_normalize=true", "trainer.algorithm.zero_variance_filter=true",
                                                      "trainer.algorithm.use_kl_loss=true", "trainer.update_ref_every_epoch=true"])
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.all_metrics = {}
    rm = torch.ones(4, 3)
    rewards = torch.zeros(4, 3)
    rewards[0, 2], rewards[1, 2] = 1.0, 0.0            # prompt a: the two samples differ
    rewards[2, 2], rewards[3, 2] = 1.0, 1.0            # prompt b: no variance
    b = TrainingInputBatch({"rewards": rewards, "response_mask": rm, "loss_mask": rm.clone()})
    b.metadata = {"uids": ["a", "a", "b", "b"]}
    out = tr.compute_advantages_and_returns(b)
    adv = out["advantages"]
    assert abs(float(adv.mean())) < 1e-6 and abs(float(adv.pow(2).mean()) - 1.0) < 1e-4           # z-scored over all response tokens
    assert out["loss_mask"][:2].sum() == 6 and out["loss_mask"][2:].sum() == 0 and tr.all_metrics["reward/num_zero_variance_filtered"] == 1
    # two epochs of two steps: after each epoch the reference is the policy of that moment
    tr.train()
    assert tr.global_step == 4
    assert torch.equal(tr.ref.model.store.flat, tr.policy.model.store.flat)


def test_rl_with_lora_adapters_moves_only_the_factors_and_resumes(tmp_path):
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    base = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4", "generator.n_samples_per_prompt=4",
            "generator.sampling_params.max_generate_length=12", "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8",
            "data.synthetic_prompts=16", "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=32",
            "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}", "trainer.ckpt_interval=2", "trainer.policy.optimizer_config.lr=1e-2",
            "trainer.policy.model.lora.rank=4", "trainer.policy.model.lora.alpha=8", "trainer.policy.model.lora.dropout=0.0"]      # the reference's key names
    cfg = SkyRLTrainConfig.from_cli_overrides(base + ["trainer.num_steps=2", "trainer.resume_mode=none"])
    assert cfg.trainer.policy.lora.rank == 4 and cfg.trainer.policy.lora.alpha == 8
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.build_models()
    w0 = {n: t.clone() for n, t in tr.policy.model.named_weights()}
    tr.train()
    ad = tr.lora_store.adapters["policy"]
    assert tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0            # the engine reads the merged weights
    assert any(float(b.abs().sum()) > 0 for b in ad.B.values())                           # the factors moved
    assert tr.policy.opt.step_count == 0 and float(tr.policy.opt.exp_avg.abs().sum()) == 0      # the base optimizer never stepped
    for n, t in tr.policy.model.named_weights():
        if n in ad.A:
            assert torch.allclose(t, w0[n] + ad.delta(n), atol=1e-6) and not torch.equal(t, w0[n])
        else:
            assert torch.equal(t, w0[n]), n                                               # embeddings, norms: untouched
    # resume: merged weights, factors, base rows and the adapter's optimizer state come back
    tr2 = RayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(base + ["trainer.num_steps=3", "trainer.resume_mode=latest"]), device="cpu")
    tr2.build_models()
    assert tr2.load_checkpoints() == 2
    ad2 = tr2.lora_store.adapters["policy"]
    assert all(torch.equal(ad2.B[k], ad.B[k]) and torch.equal(ad2.A[k], ad.A[k]) for k in ad.A)
    assert all(torch.equal(t, dict(tr.policy.model.named_weights())[n]) for n, t in tr2.policy.model.named_weights())
    assert all(torch.equal(tr2.lora_store._base[k], w0[k]) for k in ad.A)
    from skyrl_isoexec_b200.train.config import validate_cfg

    with pytest.raises(ValueError, match="lora"):
        validate_cfg(SkyRLTrainConfig.from_cli_overrides(base + ["trainer.policy.parallel.tensor_model_parallel_size=2"]), world_size=2)


def test_training_temperature_scales_the_logits_the_logprobs_are_taken_from(tmp_path):
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.config import validate_cfg
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    m = DecoderLM(get_config("tiny-qwen3"), seed=0)
    g = torch.Generator().manual_seed(0)
    p, r = torch.randint(5, 500, (12,), generator=g).tolist(), torch.randint(5, 500, (6,), generator=g).tolist()
    seq, att, rmask = build_sequences([p], [r])
    b = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask})
    lp1 = PolicyWorker(m, WorkerConfig()).forward(b)[0]
    lp2 = PolicyWorker(m, WorkerConfig(temperature=2.0)).forward(b)[0]
    # the same numbers from the definition: log softmax(logits / T) at the response tokens
    from skyrl_isoexec_b200.models.decoder import ForwardCtx
    from skyrl_isoexec_b200.ops import functional as F

    ids = torch.tensor(p + r)
    fc = ForwardCtx(positions=torch.arange(len(ids), dtype=torch.int32), meta=F.AttnMeta.packed([len(ids)], m.hq, m.hkv, "cpu"), site="trainer_score")
    with torch.no_grad():
        logits = m.logits(m(ids, fc)).float()
    want = torch.log_softmax(logits / 2.0, -1)[torch.arange(len(p) - 1, len(ids) - 1), torch.tensor(r)]
    assert torch.allclose(lp2, want, atol=1e-5) and not torch.allclose(lp1, lp2, atol=1e-3)
    ov = ["trainer.policy.model=tiny-qwen3", "generator.sampling_params.temperature=0.7"]
    with pytest.raises(ValueError, match="isoexec.enabled=false"):
        validate_cfg(SkyRLTrainConfig.from_cli_overrides(ov + ["trainer.isoexec.enabled=true", "trainer.algorithm.temperature=0.7"]))
    validate_cfg(SkyRLTrainConfig.from_cli_overrides(ov + ["trainer.isoexec.enabled=false"]))


def test_moe_balance_term_reaches_the_router_gradient_through_recomputed_layers(tmp_path):
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.ops import moe as moe_ops
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    # the injected gradient equals d(coeff * scale * aux) / d(logits) computed by plain autograd
    torch.manual_seed(0)
    logits = torch.randn(12, 8, requires_grad=True)
    idx, w = moe_ops.route(logits, 2, None, False, True)
    moe_ops.AUX_LOSS.update(coeff=0.5, scale=0.25, sum=0.0, layers=0)
    w2 = moe_ops._with_aux_loss(logits, idx, w, get_config("tiny-moe"))
    (w2 * 0.0).sum().backward()                                  # nothing but the injection reaches the logits
    f = torch.zeros(8).index_add_(0, idx.reshape(-1).long(), torch.ones(idx.numel())) / idx.numel()
    lg = logits.detach().clone().requires_grad_(True)
    (0.5 * 0.25 * 8 * (f * torch.softmax(lg, -1).mean(0)).sum()).backward()
    assert torch.allclose(logits.grad, lg.grad, atol=1e-7) and float(logits.grad.abs().sum()) > 0
    moe_ops.AUX_LOSS.update(coeff=0.0)
    # with zero advantages the policy gradient vanishes; what is left on the router is the balance term, also with every
    # layer recomputed in the backward
    m = DecoderLM(get_config("tiny-moe"), seed=0)
    g = torch.Generator().manual_seed(1)
    seq, att, rmask = build_sequences([torch.randint(5, 500, (10,), generator=g).tolist() for _ in range(3)],
                                      [torch.randint(5, 500, (6,), generator=g).tolist() for _ in range(3)])
    def batch():
        b = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                "advantages": torch.zeros_like(rmask)})
        b.metadata["aux_loss_scale"] = 1.0 / float(rmask.sum())
        return b

    def router_grad(worker):
        s = worker.model.store.specs["layers.0.moe.router.weight"]
        n = s.shape[0] * s.shape[1]
        return worker.opt.main_grad[s.offset:s.offset + n].clone()

    w0 = PolicyWorker(m, WorkerConfig(max_tokens_per_microbatch=4096))
    w0.forward_backward(batch())
    assert float(router_grad(w0).abs().sum()) == 0.0
    w1 = PolicyWorker(DecoderLM(get_config("tiny-moe"), seed=0), WorkerConfig(max_tokens_per_microbatch=4096, moe_aux_loss_coeff=0.1, checkpoint_layers=True))
    out = w1.forward_backward(batch())
    assert float(router_grad(w1).abs().sum()) > 0 and out["moe_aux_loss"] >= 1.0 - 1e-6          # E * sum f P >= 1, = 1 when balanced
    w2_ = PolicyWorker(DecoderLM(get_config("tiny-moe"), seed=0), WorkerConfig(max_tokens_per_microbatch=4096, moe_aux_loss_coeff=0.1, keep_last_layers=2))
    w2_.forward_backward(batch())
    assert torch.allclose(router_grad(w2_), router_grad(w1), atol=1e-7)                            # recomputed or kept: the same gradient
    cfg = SkyRLTrainConfig.from_cli_overrides(["trainer.policy.model=tiny-moe", "trainer.policy.megatron_config.moe_aux_loss_coeff=0.01"])
    assert cfg.trainer.policy.moe_aux_loss_coeff == 0.01 and RayPPOTrainer is not None


def test_frozen_moe_router_does_not_move_while_the_experts_train(tmp_path):
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    ov = ["trainer.policy.model=tiny-moe", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4", "generator.n_samples_per_prompt=4",
          "generator.sampling_params.max_generate_length=8", "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8",
          "data.synthetic_prompts=16", "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=32", "trainer.num_steps=2",
          "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}", "trainer.resume_mode=none", "trainer.ckpt_interval=0",
          "trainer.policy.optimizer_config.lr=1e-2", "trainer.policy.megatron_config.freeze_moe_router=true",
          "trainer.policy.megatron_config.moe_aux_loss_coeff=0.01"]
    tr = RayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(ov), device="cpu")
    tr.build_models()
    w0 = {n: t.clone() for n, t in tr.policy.model.named_weights()}
    tr.train()
    moved = {n for n, t in tr.policy.model.named_weights() if not torch.equal(t, w0[n])}
    assert not any(".moe.router." in n for n in moved) and any(".moe.experts." in n for n in moved)
    assert tr.all_metrics["policy/moe_aux_loss"] >= 1.0 - 1e-6 and tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0
