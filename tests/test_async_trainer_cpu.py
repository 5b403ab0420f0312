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
