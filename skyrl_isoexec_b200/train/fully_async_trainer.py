"""Fully asynchronous RL: rollout generation runs continuously in the background and the trainer
consumes finished prompt groups, with bounded staleness (reference: R/train/fully_async_trainer.py:104-399).

Pieces (same roles as the reference's):
  * ``AsyncPromptSource``    hands out prompts one group at a time, resumable (consumed uids are checkpointed);
  * ``StalenessManager``     admits a new rollout only while (in-flight + buffered groups) stay within
                             ``(max_staleness_steps + 1) * mini_batch_size``, so no sample can be trained on more than
                             ``max_staleness_steps`` policy versions after the one that generated it;
  * ``GenerationGroupQueue`` finished groups, each stamped with the policy version that produced it;
  * ``FullyAsyncTrainer``    a generation thread (its own event loop) + the training loop; a weight sync pauses
                             generation between engine steps, swaps weights, bumps the version and resumes.

Because trainer and engine share one flat parameter buffer when colocated, the weight "swap" is the
optimizer step itself; the pause is what keeps an engine step from reading half-updated weights, and it then covers the
whole scoring + update. With ``generator.inference_engine.own_weights=true`` the engine reads a copy of its own:
generation overlaps scoring and update, and pauses only for the copy of the new weights.
Samples generated under an older version are off-policy: their rollout logprobs are kept and the
configured off-policy correction (TIS / masks) applies. The bitwise gate only covers version-matched samples.
"""

from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass


from ..engine.sampler import SamplingParams
from .trainer import RayPPOTrainer


@dataclass
class AsyncConfig:
    max_staleness_steps: int = 1
    num_parallel_generation_workers: int = 4      # prompt groups in flight
    mini_batch_prompts: int = 8
    # simulated trainer (FullyAsyncTrainerSim): no trainer components, sleeps stand in for the update and the weight sync
    simulate_training: bool = False
    simulate_training_step_seconds: float = 0.0
    simulate_weight_sync_seconds: float = 0.0


class AsyncPromptSource:
    def __init__(self, dataset, seed: int = 0):
        self.ds, self.consumed, self.cursor, self.epoch, self.seed = dataset, set(), 0, 0, seed
        self._lock = threading.Lock()

    def next(self):
        with self._lock:
            n = len(self.ds)
            if self.cursor >= n:
                self.cursor, self.epoch = 0, self.epoch + 1
            row = self.ds[self.cursor]
            self.cursor += 1
            return row

    def mark_consumed(self, uid) -> None:
        self.consumed.add(uid)

    def state_dict(self):
        return {"cursor": self.cursor, "epoch": self.epoch, "consumed": sorted(self.consumed)}

    def load_state_dict(self, sd):
        self.cursor, self.epoch, self.consumed = sd["cursor"], sd["epoch"], set(sd["consumed"])


class StalenessManager:
    def __init__(self, max_staleness_steps: int, mini_batch_prompts: int):
        self.capacity = (max_staleness_steps + 1) * mini_batch_prompts
        self.in_flight = 0
        self.buffered = 0
        self.version = 0
        self._cv = threading.Condition()

    def acquire(self, timeout: float | None = None) -> bool:
        """Block until a new rollout group may start."""
        with self._cv:
            ok = self._cv.wait_for(lambda: self.in_flight + self.buffered < self.capacity, timeout)
            if ok:
                self.in_flight += 1
            return ok

    def finished(self) -> None:
        with self._cv:
            self.in_flight -= 1
            self.buffered += 1
            self._cv.notify_all()

    def consumed(self, n: int) -> None:
        with self._cv:
            self.buffered -= n
            self._cv.notify_all()

    def bump_version(self) -> int:
        with self._cv:
            self.version += 1
            self._cv.notify_all()
            return self.version


class GenerationGroupQueue:
    def __init__(self):
        self.q: deque = deque()
        self.failed = False
        self._cv = threading.Condition()

    def put(self, group) -> None:
        with self._cv:
            self.q.append(group)
            self._cv.notify_all()

    def get_many(self, n: int, timeout: float | None = None) -> list:
        with self._cv:
            if not self._cv.wait_for(lambda: len(self.q) >= n or self.failed, timeout):
                raise TimeoutError(f"only {len(self.q)} of {n} rollout groups arrived")
            if len(self.q) < n:
                return []
            return [self.q.popleft() for _ in range(n)]

    def put_error(self) -> None:
        with self._cv:
            self.failed = True
            self._cv.notify_all()

    def __len__(self):
        return len(self.q)


class FullyAsyncTrainer(RayPPOTrainer):
    def __init__(self, cfg, async_cfg: AsyncConfig | None = None, **kw):
        super().__init__(cfg, **kw)
        self.acfg = async_cfg or AsyncConfig(mini_batch_prompts=cfg.trainer.policy_mini_batch_size)
        self.stale = StalenessManager(self.acfg.max_staleness_steps, self.acfg.mini_batch_prompts)
        self.groups = GenerationGroupQueue()
        self._stop = threading.Event()
        self._engine_lock = threading.Lock()       # held by an engine step or by a weight update, never both
        self._gen_error: BaseException | None = None

    # ------------------------------------------------------------------ generation side
    def _admit_group(self, row) -> dict:
        gi, _ = self.prepare_generator_input([row])
        sp = SamplingParams.from_dict(gi["sampling_params"])
        prompt = list(row["prompt"])
        seqs = [self.engine.add_request(prompt, sp, i) for i in range(len(gi["prompts"]))]
        return {"row": row, "version": self.stale.version, "seqs": seqs}

    def _finish_group(self, g) -> dict:
        from .. import gym

        row, seqs = g["row"], g["seqs"]
        rewards = []
        for s in seqs:
            env = gym.make(row["env_class"], self.cfg.environment.env_kwargs, row.get("env_extras") or {})
            env.init(row["prompt"])
            rewards.append(float(env.step(s.output_ids)["reward"]))
        return {"uid": row["uid"], "version": g["version"], "prompt_token_ids": [list(row["prompt"])] * len(seqs),
                "response_ids": [list(s.output_ids) for s in seqs], "rewards": rewards,
                "loss_masks": [[1] * len(s.output_ids) for s in seqs], "rollout_logprobs": [list(s.logprobs) for s in seqs]}

    def _generation_loop(self) -> None:
        """Continuous batching across prompt groups: up to ``num_parallel_generation_workers`` groups share the
        engine's running batch; a new group is admitted as soon as the staleness budget allows."""
        active: list[dict] = []
        try:
            while not self._stop.is_set():
                while len(active) < self.acfg.num_parallel_generation_workers and self.stale.acquire(timeout=0.0):
                    active.append(self._admit_group(self.source.next()))
                if not active:
                    time.sleep(0.002)
                    continue
                with self._engine_lock:             # a weight update can slip in between two engine steps
                    self.engine.step()
                still = []
                for g in active:
                    if all(s.finished for s in g["seqs"]):
                        self.groups.put(self._finish_group(g))
                        self.stale.finished()
                    else:
                        still.append(g)
                active = still
        except BaseException as e:  # noqa: BLE001
            self._gen_error = e
            self.groups.put_error()

    # ------------------------------------------------------------------ training side
    def _run_training(self, batch, fresh: bool) -> None:
        """Scoring forward, advantages and the policy update on one mini-batch of finished groups."""
        iso = self.cfg.trainer.isoexec
        strict_before = iso.strict
        if not fresh:
            iso.strict = False          # stale samples are off-policy by construction
        try:
            batch = self.fwd_logprobs_values_reward(batch)
        finally:
            iso.strict = strict_before
        batch = self.compute_advantages_and_returns(batch)
        self.train_critic_and_policy(batch)

    def _publish_weights(self) -> None:
        self.sync_weights()

    def train(self) -> None:
        if self.engine is None:
            self.build_models()
        self.source = AsyncPromptSource(self.dataset, self.cfg.trainer.seed)
        self._publish_weights()
        self.engine.wake_up()
        th = threading.Thread(target=self._generation_loop, daemon=True)
        th.start()
        n_steps = self.cfg.trainer.num_steps if self.cfg.trainer.num_steps > 0 else 1
        self._fire("on_train_start")
        try:
            for _ in range(n_steps):
                t0 = time.perf_counter()
                groups = self.groups.get_many(self.acfg.mini_batch_prompts, timeout=600)
                if self._gen_error is not None:
                    raise RuntimeError("the generation thread failed") from self._gen_error
                self.stale.consumed(len(groups))
                go = {k: [x for g in groups for x in g[k]] for k in ("prompt_token_ids", "response_ids", "rewards", "loss_masks",
                                                                      "rollout_logprobs")}
                uids = [g["uid"] for g in groups for _ in g["response_ids"]]
                self.global_step += 1
                self.all_metrics = {}
                batch = self.convert_to_training_input(go, uids)
                staleness = [self.stale.version - g["version"] for g in groups]
                if getattr(self, "separate_engine", False):
                    # the engine has weights of its own (generator.inference_engine.own_weights): generation goes on during
                    # scoring and the update, and stops only while the new weights are copied in
                    self._run_training(batch, all(s == 0 for s in staleness))
                    with self._engine_lock:
                        self._publish_weights()
                        self.stale.bump_version()
                else:
                    with self._engine_lock:         # scoring + update exclude engine steps: one flat buffer, one writer
                        self._run_training(batch, all(s == 0 for s in staleness))
                        self._publish_weights()
                        self.stale.bump_version()
                for g in groups:
                    self.source.mark_consumed(g["uid"])
                self.all_metrics.update({"async/staleness_max": max(staleness), "async/staleness_mean": sum(staleness) / len(staleness),
                                         "async/buffered_groups": len(self.groups), "timing/step": time.perf_counter() - t0})
                self._fire("on_step_end", metrics=dict(self.all_metrics))
                self._fire("on_log", logs=self.all_metrics)
                if self.tracker is not None:
                    self.tracker.log(self.all_metrics, self.global_step)
                self.control.reset()
                if self.control.should_stop:
                    break
            self._fire("on_train_end")
        finally:
            self._stop.set()
            th.join(timeout=30)


class FullyAsyncTrainerSim(FullyAsyncTrainer):
    """The fully-async loop with a SIMULATED trainer (reference: R/train/fully_async_trainer_sim.py:55-115): the engine,
    the generation thread, the staleness budget and the pause around a weight update are real; the update itself is a
    sleep of ``simulate_training_step_seconds`` and the weight sync a sleep of ``simulate_weight_sync_seconds`` during
    which generation is paused. No policy worker, optimizer state, reference or critic model is built, so the
    generation side can be measured at a model size whose training state would not fit. Evaluation, checkpoints and
    exports are refused; nothing is resumed."""

    def __init__(self, cfg, async_cfg: AsyncConfig | None = None, **kw):
        super().__init__(cfg, async_cfg, **kw)
        t = self.cfg.trainer
        assert self.acfg.simulate_training, "FullyAsyncTrainerSim needs AsyncConfig.simulate_training=True"
        assert t.eval_interval <= 0 and t.ckpt_interval <= 0 and t.hf_save_interval <= 0, \
            "the simulated trainer has no model state: evaluation, checkpoints and exports must be off (it never resumes)"

    def build_models(self) -> None:
        """Engine side only: the model's parameters (random init or whatever the caller loads into them), the engine and
        the generator."""
        from ..engine.interface import NativeInferenceEngine
        from ..engine.llm_engine import EngineConfig, LLMEngine
        from ..models.config import get_config
        from ..models.decoder import DecoderLM
        from .generator import SkyRLGymGenerator
        from .trainer import PromptDataLoader, SyntheticPromptDataset

        t, g = self.cfg.trainer, self.cfg.generator
        mcfg = get_config(t.policy.model, **t.policy.model_overrides)
        model = DecoderLM(mcfg, self.ps, self.device, seed=t.policy.seed)
        for p in model.parameters():
            p.requires_grad_(False)
        ie = g.inference_engine
        ecfg = EngineConfig(max_num_seqs=ie.max_num_seqs, max_num_batched_tokens=ie.max_num_batched_tokens,
                            num_kv_pages=ie.num_kv_pages, gpu_memory_utilization=ie.gpu_memory_utilization,
                            seed=t.seed + 7919 * self.ps.dp_rank, enable_prefix_caching=ie.enable_prefix_caching,
                            use_cuda_graph=not ie.enforce_eager, share_prompt_pages=ie.share_prompt_pages, share_recurrent_state=ie.share_recurrent_state,
                            max_model_len=min(mcfg.max_position, t.max_prompt_length + g.sampling_params.max_generate_length + 1))
        self.engine = LLMEngine(model, ecfg)
        self.infer = NativeInferenceEngine(self.engine, self.tokenizer)
        self.generator = SkyRLGymGenerator(self.infer, self.tokenizer, max_turns=g.max_turns, batched=g.batched,
                                           env_config=self.cfg.environment.env_kwargs)
        if self.dataset is None:
            d = self.cfg.data
            self.dataset = SyntheticPromptDataset(d.synthetic_prompts or t.train_batch_size * 4, d.synthetic_prompt_len,
                                                  mcfg.vocab_size, t.seed, self.cfg.environment.env_class)
        self.loader = PromptDataLoader(self.dataset, t.train_batch_size, t.seed)
        self.sim_steps: list[dict] = []

    def convert_to_training_input(self, go, uids):
        return {"num_sequences": len(go["response_ids"]), "response_tokens": sum(len(r) for r in go["response_ids"])}

    def _run_training(self, batch, fresh: bool) -> None:
        time.sleep(self.acfg.simulate_training_step_seconds)
        self.sim_steps.append({"step": self.global_step, "fresh": fresh, **batch})
        self.all_metrics.update({"sim/step_seconds": self.acfg.simulate_training_step_seconds,
                                 "sim/response_tokens": batch["response_tokens"]})

    def _publish_weights(self) -> None:
        """Called with the engine lock held (generation is paused), as a real weight update would be."""
        if self.acfg.simulate_weight_sync_seconds > 0:
            time.sleep(self.acfg.simulate_weight_sync_seconds)
