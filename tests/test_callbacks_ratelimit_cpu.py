"""Trainer callbacks (events, control flags, log mutation, early stop) and the trajectory rate / concurrency limiter."""

import asyncio
import json
import os

import pytest

from skyrl_isoexec_b200.train.callbacks import CallbackHandler, TrainingCallback
from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
from skyrl_isoexec_b200.train.trainer import RayPPOTrainer
from skyrl_isoexec_b200.utils.rate_limiter import (AsyncRateLimiter, NoOpRateLimiter, RateLimiterConfig, create_rate_limiter)


def _cfg(tmp, steps, *extra):
    return SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=4",
        "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=16",
        "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", f"trainer.num_steps={steps}",
        f"trainer.ckpt_path={tmp}", "trainer.ckpt_interval=0", "trainer.logger=jsonl", "trainer.eval_batch_size=2",
        "generator.eval_sampling_params.max_generate_length=4", "generator.eval_sampling_params.ignore_eos=true", *extra])


class _Recorder(TrainingCallback):
    def __init__(self):
        self.events = []

    def on_train_start(self, trainer, ci, control):
        self.events.append(("train_start", ci.global_step, ci.total_steps))

    def on_epoch_start(self, trainer, ci, control):
        self.events.append(("epoch_start", ci.epoch))

    def on_step_start(self, trainer, ci, control):
        assert ci.batch is not None and ci.metrics is None
        self.events.append(("step_start", ci.global_step))

    def on_step_end(self, trainer, ci, control):
        assert "policy/grad_norm" in ci.metrics
        self.events.append(("step_end", ci.global_step))
        if ci.global_step == 1:
            control.should_save = control.should_evaluate = True     # neither is scheduled by the config
        if ci.global_step == 2:
            control.should_stop = True

    def on_eval_start(self, trainer, ci, control):
        self.events.append(("eval_start", ci.global_step))

    def on_eval_end(self, trainer, ci, control):
        assert "eval/num_prompts" in ci.metrics
        self.events.append(("eval_end", ci.global_step))

    def on_save(self, trainer, ci, control):
        assert os.path.isdir(ci.ckpt_path)
        self.events.append(("save", ci.global_step))

    def on_log(self, trainer, ci, control):
        ci.logs["custom/seen_by_callback"] = float(ci.global_step)

    def on_train_end(self, trainer, ci, control):
        self.events.append(("train_end", ci.global_step))


def test_trainer_fires_callbacks_and_honours_control_flags(tmp_path):
    rec, other = _Recorder(), TrainingCallback()
    tr = RayPPOTrainer(_cfg(str(tmp_path), 5), device="cpu", callbacks=[CallbackHandler([rec]), other])   # handlers nest
    tr.train()
    assert tr.global_step == 2, "should_stop ends the run after step 2 although five steps were configured"
    assert rec.events == [("train_start", 0, 5), ("epoch_start", 0), ("step_start", 0), ("step_end", 1), ("save", 1),
                          ("eval_start", 1), ("eval_end", 1), ("step_start", 1), ("step_end", 2), ("train_end", 2)]
    assert not tr.control.should_save and not tr.control.should_evaluate
    assert tr.all_metrics["custom/seen_by_callback"] == 2.0
    logged = [json.loads(ln) for ln in open(_jsonl(tr))]
    assert any(r.get("custom/seen_by_callback") == 1.0 for r in logged), "the field a callback added reaches the tracker"


def _jsonl(tr):
    return tr.tracker.loggers["jsonl"].f.name


def test_rate_limiter_config_and_factory():
    with pytest.raises(ValueError):
        RateLimiterConfig(True, 0.5, None)
    with pytest.raises(ValueError):
        AsyncRateLimiter(None, 0)
    assert isinstance(create_rate_limiter(None), NoOpRateLimiter)
    assert isinstance(create_rate_limiter({"enabled": False, "max_concurrency": 2}), NoOpRateLimiter)
    assert isinstance(create_rate_limiter({"enabled": True}), NoOpRateLimiter)
    lim = create_rate_limiter(RateLimiterConfig(True, 2.0, 3))
    assert isinstance(lim, AsyncRateLimiter) and lim.rate == 2.0 and lim.max_concurrency == 3


def test_rate_limiter_token_bucket_on_virtual_time_and_concurrency_cap():
    now = [0.0]

    async def fake_sleep(dt):
        now[0] += dt
        await asyncio.sleep(0)

    async def run():
        lim = AsyncRateLimiter(rate=4.0, clock=lambda: now[0], sleep=fake_sleep)
        stamps = []
        for _ in range(10):
            await lim.acquire()
            stamps.append(now[0])
            lim.release()
        # a full bucket lets four through at once, then one start every quarter second
        assert stamps[:4] == [0.0] * 4
        assert [round(s, 6) for s in stamps[4:]] == [0.25, 0.5, 0.75, 1.0, 1.25, 1.5]

        cap = AsyncRateLimiter(max_concurrency=3)
        live = [0]

        async def traj():
            async with cap:
                live[0] += 1
                assert live[0] <= 3
                await asyncio.sleep(0.001)
                live[0] -= 1

        await asyncio.gather(*[traj() for _ in range(12)])
        assert cap.peak_in_flight == 3 and cap.in_flight == 0 and cap.started == 12

        # an exception inside the bracket still frees the slot
        with pytest.raises(RuntimeError):
            async with cap:
                raise RuntimeError("trajectory failed")
        assert cap.in_flight == 0

    asyncio.run(run())


def test_generator_brackets_multi_turn_trajectories_with_the_limiter(tmp_path):
    tr = RayPPOTrainer(_cfg(str(tmp_path), 1, "generator.batched=false", "generator.rate_limit.enabled=true",
                            "generator.rate_limit.max_concurrency=2"), device="cpu")
    tr.build_models()
    tr.sync_weights()
    m = tr.train_step(next(iter(tr.loader)))
    lim = tr.generator.rate_limiter
    assert isinstance(lim, AsyncRateLimiter) and lim.started == 4 and lim.peak_in_flight <= 2 and lim.in_flight == 0
    assert m["policy/rollout_train_logprob_bit_mismatches"] == 0


def test_archives_round_trip_and_shared_filesystem_probe(tmp_path):
    from skyrl_isoexec_b200.utils import io as xio

    dest = str(tmp_path / "out" / "ckpt.tar.gz")
    with xio.pack_and_upload(dest) as d:
        os.makedirs(os.path.join(d, "sub"))
        open(os.path.join(d, "sub", "a.bin"), "wb").write(b"\x00\x01" * 1000)
        open(os.path.join(d, "meta.json"), "w").write("{}")
    with xio.download_and_unpack(dest) as d:
        assert open(os.path.join(d, "sub", "a.bin"), "rb").read() == b"\x00\x01" * 1000 and os.path.exists(os.path.join(d, "meta.json"))
    assert xio.download_file(dest).read(2) == b"\x1f\x8b"                       # a gzip stream
    # shared filesystem (probe file present): ranks other than 0 leave the archive alone
    other = str(tmp_path / "shared.tar.gz")
    open(other + ".probe", "w").close()
    with xio.pack_and_upload(other, rank=1) as d:
        open(os.path.join(d, "x"), "w").write("1")
    assert not os.path.exists(other)
    with xio.pack_and_upload(other, rank=0) as d:
        open(os.path.join(d, "x"), "w").write("1")
    assert os.path.exists(other)
    # a failure inside the block writes nothing
    bad = str(tmp_path / "bad.tar.gz")
    with pytest.raises(RuntimeError):
        with xio.pack_and_upload(bad) as d:
            raise RuntimeError("save failed")
    assert not os.path.exists(bad)


def test_log_example_formats_reward_and_colours(tmp_path, capsys):
    import io

    from skyrl_isoexec_b200.utils.tracking import log_example

    buf = io.StringIO()
    text = log_example([{"role": "user", "content": "2+2?"}], "line one\nline two", [0.0, 1.0], stream=buf, color=True)
    assert buf.getvalue() == text and "Total Reward: 1.0000" in text
    assert text.count("\033[32m") == 2 and "\033[36m" in text                     # both response lines green, prompt cyan
    text = log_example("p", "r", None, stream=buf, color=False)
    assert "Total Reward: N/A" in text and "\033[" not in text
    assert "\033[33m" in log_example("p", "r", -1.0, stream=buf, color=True)     # non-positive reward: yellow
    tr = RayPPOTrainer(_cfg(str(tmp_path), 1, "trainer.log_example_interval=1"), device="cpu")
    tr.train()
    assert "Example:\n  Input: " in capsys.readouterr().out


def test_simulated_async_trainer_builds_no_trainer_state_and_keeps_the_generation_dynamics(tmp_path):
    from skyrl_isoexec_b200.train.fully_async_trainer import AsyncConfig, FullyAsyncTrainerSim

    cfg = _cfg(str(tmp_path), 3)
    with pytest.raises(AssertionError):
        FullyAsyncTrainerSim(cfg, AsyncConfig(mini_batch_prompts=2), device="cpu")          # simulate_training is off
    with pytest.raises(AssertionError):
        FullyAsyncTrainerSim(_cfg(str(tmp_path), 3, "trainer.ckpt_interval=1"),
                             AsyncConfig(mini_batch_prompts=2, simulate_training=True), device="cpu")
    ac = AsyncConfig(max_staleness_steps=1, num_parallel_generation_workers=3, mini_batch_prompts=2, simulate_training=True,
                     simulate_training_step_seconds=0.01, simulate_weight_sync_seconds=0.005)
    tr = FullyAsyncTrainerSim(cfg, ac, device="cpu")
    tr.train()
    assert tr.policy is None and tr.global_step == 3 and len(tr.sim_steps) == 3
    assert all(s["num_sequences"] == 4 and s["response_tokens"] == 16 for s in tr.sim_steps)   # 2 prompts x 2 samples x 4 tokens
    assert tr.stale.version == 3 and 0 <= tr.all_metrics["async/staleness_max"] <= 2
    assert tr.all_metrics["sim/response_tokens"] == 16
    assert not any(p.requires_grad for p in tr.engine.model.parameters())

    class StopAfterTwo(TrainingCallback):
        seen = []

        def on_train_start(self, trainer, ci, control):
            self.seen.append("start")

        def on_step_end(self, trainer, ci, control):
            self.seen.append(ci.global_step)
            control.should_stop = ci.global_step >= 2

        def on_log(self, trainer, ci, control):
            ci.logs["custom/async"] = 1.0

        def on_train_end(self, trainer, ci, control):
            self.seen.append("end")

    tr = FullyAsyncTrainerSim(_cfg(str(tmp_path), 5), ac, device="cpu", callbacks=[StopAfterTwo()])
    tr.train()
    assert StopAfterTwo.seen == ["start", 1, 2, "end"] and tr.global_step == 2 and tr.all_metrics["custom/async"] == 1.0


def test_step_wise_trajectories_train_each_turn_with_the_trajectory_advantage(tmp_path):
    import torch

    from skyrl_isoexec_b200.train.config import validate_cfg

    with pytest.raises(ValueError):
        validate_cfg(_cfg(str(tmp_path), 1, "generator.step_wise_trajectories=true"))                     # batched single turn
    with pytest.raises(ValueError):
        validate_cfg(_cfg(str(tmp_path), 1, "generator.step_wise_trajectories=true", "generator.batched=false",
                          "trainer.algorithm.advantage_estimator=gae"))
    cfg = _cfg(str(tmp_path), 1, "generator.step_wise_trajectories=true", "generator.batched=false", "generator.max_turns=3",
               "environment.env_class=even_tokens_turns", "generator.inference_engine.num_kv_pages=32", "trainer.max_prompt_length=24",
               "generator.eval_n_samples_per_prompt=2", "generator.eval_sampling_params.temperature=1.0")
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.build_models()
    tr.sync_weights()
    rows = next(iter(tr.loader))
    gi, uids = tr.prepare_generator_input(rows)
    tr.engine.wake_up()
    go = tr.generate(gi)
    tr.engine.sleep()
    # 2 prompts x 2 samples = 4 trajectories of 3 turns: 12 rows, turns adjacent, the third of each closes the trajectory
    assert len(go["response_ids"]) == 12 and go["is_last_step"] == [False, False, True] * 4
    assert go["step_source"] == [0] * 3 + [1] * 3 + [2] * 3 + [3] * 3
    for k in range(0, 12, 3):
        p0, p1, p2 = (go["prompt_token_ids"][k + j] for j in range(3))
        assert p1 == p0 + go["response_ids"][k] and p2 == p1 + go["response_ids"][k + 1], "a step's prompt is the whole context so far"
        assert sum(go["rewards"][k]) == 0 and sum(go["rewards"][k + 1]) == 0          # the outcome reward arrives with the last turn
    assert go["rollout_metrics"]["generate/steps_per_trajectory"] == 3.0
    batch = tr.convert_to_training_input(go, uids)
    assert batch.metadata["uids"] == [uids[i] for i in go["step_source"]] and batch.batch_size == 12
    tr.all_metrics = {}
    batch = tr.compute_advantages_and_returns(batch)
    adv, rm = batch["advantages"], batch["response_mask"]
    for k in range(0, 12, 3):
        vals = [adv[k + j][rm[k + j].bool()] for j in range(3)]
        assert all(torch.equal(v, vals[2][:1].expand_as(v)) for v in vals), "every turn carries its trajectory's one advantage"
    # the group baseline is over trajectories (last steps), not over rows: two trajectories per prompt sum to zero
    a_traj = torch.stack([adv[k + 2][0] for k in range(0, 12, 3)])
    assert abs(float(a_traj[0] + a_traj[1])) < 1e-5 and abs(float(a_traj[2] + a_traj[3])) < 1e-5
    # and the whole step runs through the trainer with the forward gate on
    m = tr.train_step(next(iter(tr.loader)))
    assert m["policy/rollout_train_logprob_bit_mismatches"] == 0 and m["policy/grad_norm"] > 0
    # evaluation scores TRAJECTORIES (last steps), not rows: 2 prompts x 2 samples, each 3 turns of 4 tokens
    ev = tr.eval()
    assert ev["eval/num_prompts"] == 2 and ev["eval/avg_response_length"] == 12.0 and 0.0 <= ev["eval/avg_reward"] <= 1.0


def test_on_policy_distillation_rewards_are_the_teacher_gap_and_pull_the_student_toward_the_teacher(tmp_path):
    import torch

    from skyrl_isoexec_b200.train.distill import OnPolicyDistillationTrainer

    cfg = _cfg(str(tmp_path), 3, "trainer.ref.model=tiny-qwen3", "trainer.ref.seed=7", "trainer.policy.optimizer_config.lr=1e-3",
               "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4", "generator.sampling_params.max_generate_length=8",
               "data.synthetic_prompts=64")
    tr = OnPolicyDistillationTrainer(cfg, device="cpu")
    assert cfg.trainer.algorithm.advantage_estimator == "no_op" and cfg.trainer.algorithm.use_kl_in_reward
    tr.build_models()
    assert tr.ref is not None and not torch.equal(tr.ref.model.store.flat, tr.policy.model.store.flat), "the teacher has its own weights"
    tr.sync_weights()
    rows = next(iter(tr.loader))
    gi, uids = tr.prepare_generator_input(rows)
    tr.engine.wake_up()
    go = tr.generate(gi)
    tr.engine.sleep()
    tr.all_metrics = {}
    batch = tr.fwd_logprobs_values_reward(tr.convert_to_training_input(go, uids))
    want = -(batch["action_log_probs"] - batch["base_action_log_probs"]) * batch["loss_mask"]
    assert torch.equal(batch["rewards"], want) and float(want.abs().sum()) > 0
    batch = tr.compute_advantages_and_returns(batch)
    assert torch.equal(batch["advantages"], want * batch["response_mask"]), "no_op: the dense rewards are the advantages"
    assert tr.all_metrics["distill/reverse_kl"] > 0
    # one update on this batch moves the student the right way: tokens the teacher likes more than the student (positive
    # advantage) gain probability, the others lose it -- to first order sum(adv * delta logprob) > 0
    before, adv, mask = batch["action_log_probs"].clone(), batch["advantages"].clone(), batch["response_mask"]
    tr.train_critic_and_policy(batch)
    after = tr.policy.forward(batch)
    assert float((adv * (after - before) * mask).sum()) > 0
    tr.sync_weights()
    tr.train()
    assert tr.global_step == 3 and tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0
    assert tr.all_metrics["distill/reverse_kl"] == tr.all_metrics["distill/reverse_kl"]          # finite, logged every step


def test_tracking_backends_against_fake_clients(tmp_path, monkeypatch, capsys):
    """Every tracker backend, driven through stand-ins for the client packages (none of which is installed here): each gets
    the run's identity at construction, scalar metrics per step and a closing call; unknown names and missing packages fail
    at construction, not at the first log call; a crash report reaches every backend."""
    import sys
    import types

    from skyrl_isoexec_b200.utils.tracking import Tracking

    calls = []

    def fake(name, **fns):
        m = types.ModuleType(name)
        for k, f in fns.items():
            setattr(m, k, f)
        monkeypatch.setitem(sys.modules, name, m)

    fake("wandb", init=lambda **kw: calls.append(("wandb.init", kw["project"], kw["name"])),
         log=lambda d, step: calls.append(("wandb.log", dict(d), step)), finish=lambda: calls.append(("wandb.finish",)))
    fake("mlflow", set_experiment=lambda p: calls.append(("mlflow.exp", p)), start_run=lambda run_name: calls.append(("mlflow.run", run_name)),
         log_params=lambda p: calls.append(("mlflow.params", p)), log_metrics=lambda d, step: calls.append(("mlflow.log", dict(d), step)),
         end_run=lambda: calls.append(("mlflow.end",)))
    fake("swanlab", init=lambda **kw: calls.append(("swanlab.init", kw["experiment_name"])),
         log=lambda d, step: calls.append(("swanlab.log", dict(d), step)), finish=lambda: calls.append(("swanlab.finish",)))
    tr = Tracking("proj", "run1", "['wandb', 'mlflow', 'swanlab', 'console', 'jsonl']", config={"lr": 1e-6, "nested": {"a": 1}},
                  log_dir=str(tmp_path))
    assert list(tr.loggers) == ["wandb", "mlflow", "swanlab", "console", "jsonl"]
    tr.log({"loss": 0.5, "note": "text", "n": 3}, step=7)
    assert ("wandb.log", {"loss": 0.5, "note": "text", "n": 3}, 7) in calls
    assert ("mlflow.log", {"loss": 0.5, "n": 3.0}, 7) in calls and ("swanlab.log", {"loss": 0.5, "n": 3}, 7) in calls   # scalars only
    assert ("mlflow.params", {"lr": "1e-06", "nested": "{'a': 1}"}) in calls
    assert "[step 7]" in capsys.readouterr().out
    try:
        raise RuntimeError("boom")
    except RuntimeError as e:
        tr.log_exception(e, step=8)
    crash = [c for c in calls if c[0] == "wandb.log" and "crash/traceback" in c[1]]
    assert crash and "RuntimeError: boom" in crash[0][1]["crash/traceback"] and crash[0][1]["crash/type"] == "RuntimeError"
    tr.finish()
    assert all(c in calls for c in (("wandb.finish",), ("mlflow.end",), ("swanlab.finish",)))
    lines = [json.loads(ln) for ln in open(tmp_path / "proj" / "run1.jsonl")]
    assert lines[0]["step"] == 7 and lines[0]["loss"] == 0.5 and lines[1]["crash/type"] == "RuntimeError"
    with pytest.raises(ValueError):
        Tracking("p", "r", "console,comet")
    monkeypatch.setitem(sys.modules, "wandb", None)                          # "import wandb" now fails
    with pytest.raises(ImportError):
        Tracking("p", "r", "wandb")


def test_step_wise_rollouts_can_be_merged_back_into_one_row_per_trajectory(tmp_path):
    cfg = _cfg(str(tmp_path), 1, "generator.step_wise_trajectories=true", "generator.merge_stepwise_output=true", "generator.batched=false",
               "generator.max_turns=3", "environment.env_class=even_tokens_turns", "generator.inference_engine.num_kv_pages=32",
               "trainer.max_prompt_length=24")
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.build_models()
    tr.sync_weights()
    rows = next(iter(tr.loader))
    gi, uids = tr.prepare_generator_input(rows)
    tr.engine.wake_up()
    go = tr.generate(gi)
    tr.engine.sleep()
    assert len(go["response_ids"]) == 12
    batch = tr.convert_to_training_input(go, uids)
    assert batch.batch_size == 4 and batch.metadata["uids"] == [uids[0], uids[1], uids[2], uids[3]]
    # a merged row is the first step's prompt followed by all three turns; every generated token keeps loss and logprob
    first_prompt = go["prompt_token_ids"][0]
    joined = go["response_ids"][0] + go["response_ids"][1] + go["response_ids"][2]
    n = int(batch["response_mask"][0].sum())
    assert n == len(joined) and int(batch["loss_mask"][0].sum()) == len(joined)
    assert batch["sequences"][0][batch["attention_mask"][0].bool()].tolist() == first_prompt + joined
    m = tr.train_step(next(iter(tr.loader)))
    assert m["policy/rollout_train_logprob_bit_mismatches"] == 0
