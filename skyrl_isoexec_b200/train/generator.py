"""Generators turn prompts into trajectories by driving an inference engine and environments.

Data contracts are the reference's (R/train/generators/base.py:27-79): ``GeneratorInput`` =
{prompts, env_classes, env_extras, sampling_params, trajectory_ids, batch_metadata} and
``GeneratorOutput`` = {prompt_token_ids, response_ids, rewards, loss_masks, stop_reasons,
rollout_metrics, rollout_logprobs, trajectory_ids, ...}; ``generate`` is async and
order-preserving. ``SkyRLGymGenerator`` implements single-turn batched generation and the
multi-turn agent loop (R/train/generators/skyrl_gym_generator.py:273,713,808).
"""

from __future__ import annotations

from ..utils.tokenizer import chat_ids, chat_ids_continuation

import asyncio
import time
from abc import ABC, abstractmethod
from typing import Any, TypedDict

from .. import gym
from ..engine.interface import InferenceEngineInterface


class GeneratorInput(TypedDict, total=False):
    prompts: list                 # token-id lists, strings, or chat message lists
    env_classes: list[str]
    env_extras: list[dict] | None
    sampling_params: dict | None
    trajectory_ids: list | None
    batch_metadata: dict | None


class GeneratorOutput(TypedDict, total=False):
    prompt_token_ids: list[list[int]]
    response_ids: list[list[int]]
    rewards: list                 # per-sequence float or per-token list
    loss_masks: list[list[int]]
    stop_reasons: list[str] | None
    rollout_metrics: dict | None
    rollout_logprobs: list[list[float]] | None
    trajectory_ids: list | None
    trajectory_generation_times: list[float] | None
    rollout_expert_indices: Any
    is_last_step: list[bool] | None
    step_source: list[int] | None
    env_metrics: list[dict] | None


class GeneratorInterface(ABC):
    @abstractmethod
    async def generate(self, input_batch: GeneratorInput) -> GeneratorOutput: ...


def get_rollout_metrics(response_ids, rewards, env_metrics=None) -> dict:
    lens = [len(r) for r in response_ids]
    scalar = [float(sum(r)) if isinstance(r, (list, tuple)) else float(r) for r in rewards]
    n = max(1, len(lens))
    m = {
        "generate/min_num_tokens": min(lens) if lens else 0,
        "generate/max_num_tokens": max(lens) if lens else 0,
        "generate/avg_num_tokens": sum(lens) / n,
        "generate/avg_reward": sum(scalar) / n,
        "generate/pass_rate": sum(1 for s in scalar if s > 0) / n,
    }
    if env_metrics:
        for k, v in gym.Env.aggregate_metrics(env_metrics).items():
            m[f"environment/{k}"] = v
    return m


def concatenate_generator_outputs(outs: list[GeneratorOutput]) -> GeneratorOutput:
    res: GeneratorOutput = {}
    for k in ("prompt_token_ids", "response_ids", "rewards", "loss_masks", "stop_reasons", "rollout_logprobs",
              "trajectory_ids", "trajectory_generation_times", "is_last_step", "env_metrics"):
        vals = [o.get(k) for o in outs]
        res[k] = None if any(v is None for v in vals) else [x for v in vals for x in v]
    res["rollout_metrics"] = get_rollout_metrics(res["response_ids"], res["rewards"], res.get("env_metrics"))
    res["rollout_expert_indices"] = None
    return res


class SkyRLGymGenerator(GeneratorInterface):
    def __init__(self, engine: InferenceEngineInterface, tokenizer=None, max_turns: int = 1, batched: bool = True,
                 max_input_length: int = 1 << 30, env_config: dict | None = None, zero_reward_on_non_stop: bool = False,
                 apply_overlong_filtering: bool = False, rate_limit=None, step_wise: bool = False):
        from ..utils.rate_limiter import create_rate_limiter

        self.rate_limiter = create_rate_limiter(rate_limit)      # brackets every multi-turn trajectory (start rate, in flight)
        # step-wise trajectories (R/train/generators/skyrl_gym_generator.py:361-580): every model turn of a multi-turn
        # trajectory becomes a training sample of its own (prompt = the whole context before the turn, response = the turn)
        self.step_wise = step_wise
        if step_wise and batched and max_turns == 1:
            raise ValueError("step-wise trajectories need the multi-turn agent loop: set generator.batched=false")
        self.engine = engine
        self.tokenizer = tokenizer
        self.max_turns = max_turns
        self.batched = batched
        self.max_input_length = max_input_length
        self.env_config = env_config or {}
        self.zero_reward_on_non_stop = zero_reward_on_non_stop
        self.apply_overlong_filtering = apply_overlong_filtering
        self.chat_template_kwargs: dict = {}                     # extra arguments of the tokenizer's chat template (the trainer sets them)

    # ------------------------------------------------------------------ helpers
    def _encode_prompt(self, prompt) -> list[int]:
        if isinstance(prompt, (list, tuple)) and (len(prompt) == 0 or isinstance(prompt[0], int)):
            return list(prompt)
        if self.tokenizer is None:
            raise ValueError("string / chat prompts need a tokenizer")
        if isinstance(prompt, str):
            return list(self.tokenizer.encode(prompt))
        return chat_ids(self.tokenizer, prompt, **self.chat_template_kwargs)

    def _decode(self, ids: list[int]) -> str:
        return self.tokenizer.decode(ids) if self.tokenizer is not None else ""

    # ------------------------------------------------------------------ single turn, whole batch in one engine call
    async def generate_batched(self, input_batch: GeneratorInput) -> GeneratorOutput:
        prompts = input_batch["prompts"]
        n = len(prompts)
        env_classes = input_batch["env_classes"]
        extras = input_batch.get("env_extras") or [{}] * n
        envs = [gym.make(c, self.env_config, e) for c, e in zip(env_classes, extras)]
        prompt_ids = [self._encode_prompt(env.init(p)[0]) for env, p in zip(envs, prompts)]
        t0 = time.time()
        out = await self.engine.generate({"prompt_token_ids": prompt_ids, "sampling_params": input_batch.get("sampling_params")})
        dt = time.time() - t0
        rewards, env_metrics, loss_masks = [], [], []
        for env, rid, stop in zip(envs, out["response_ids"], out["stop_reasons"]):
            step = env.step(rid if env.accepts_tokens else self._decode(rid))
            r = float(step["reward"])
            if self.zero_reward_on_non_stop and stop != "stop":
                r = 0.0
            rewards.append(r)
            env_metrics.append(env.get_metrics())
            mask = [1] * len(rid)
            if self.apply_overlong_filtering and stop == "length":
                mask = [0] * len(rid)
            loss_masks.append(mask)
            env.close()
        return {
            "prompt_token_ids": prompt_ids, "response_ids": out["response_ids"], "rewards": rewards,
            "loss_masks": loss_masks, "stop_reasons": out["stop_reasons"],
            "rollout_metrics": get_rollout_metrics(out["response_ids"], rewards, env_metrics),
            "rollout_logprobs": out.get("response_logprobs"), "trajectory_ids": input_batch.get("trajectory_ids"),
            "trajectory_generation_times": [dt] * n, "rollout_expert_indices": None, "is_last_step": [True] * n,
            "env_metrics": env_metrics,
        }

    # ------------------------------------------------------------------ multi-turn, one trajectory
    async def agent_loop(self, prompt, env_class: str, env_extras: dict, sampling_params: dict | None):
        """Alternate model turns and environment observations. Observation tokens are appended to
        the context with loss mask 0 and logprob 0; per-token rewards put each turn's reward on the
        turn's last generated token."""
        extras = dict(env_extras or {})
        extras.setdefault("max_turns", self.max_turns)
        env = gym.make(env_class, self.env_config, extras)
        prompt, _ = env.init(prompt)
        prompt_ids = self._encode_prompt(prompt)
        ctx = list(prompt_ids)
        resp, mask, lps, rew = [], [], [], []
        steps: list[dict] = []
        stop = "stop"
        t0 = time.time()
        for _turn in range(self.max_turns):
            if len(ctx) >= self.max_input_length:
                stop = "length"
                break
            out = await self.engine.generate({"prompt_token_ids": [ctx], "sampling_params": sampling_params})
            rid = out["response_ids"][0]
            rlp = (out.get("response_logprobs") or [[0.0] * len(rid)])[0]
            stop = out["stop_reasons"][0]
            step = env.step(rid if env.accepts_tokens else self._decode(rid))
            if self.step_wise and rid:
                steps.append({"prompt": list(ctx), "response": list(rid), "logprobs": list(rlp), "stop": stop,
                              "rewards": [0.0] * (len(rid) - 1) + [float(step["reward"])]})
            resp += rid
            mask += [1] * len(rid)
            lps += rlp
            rew += [0.0] * (len(rid) - 1) + [float(step["reward"])] if rid else []
            ctx += rid
            if step["done"]:
                break
            obs = step.get("observations") or []
            if obs:
                if self.tokenizer is None:
                    raise ValueError("text observations need a tokenizer")
                obs_ids = chat_ids_continuation(self.tokenizer, obs, **self.chat_template_kwargs)
                resp += obs_ids
                mask += [0] * len(obs_ids)
                lps += [0.0] * len(obs_ids)
                rew += [0.0] * len(obs_ids)
                ctx += obs_ids
        metrics = env.get_metrics()
        env.close()
        if self.step_wise:
            return steps, time.time() - t0, metrics
        return prompt_ids, resp, rew, mask, stop, lps, time.time() - t0, metrics

    def _flatten_steps(self, res, input_batch: GeneratorInput) -> GeneratorOutput:
        """One row per model turn, the turns of a trajectory adjacent and in order; ``is_last_step`` marks a trajectory's
        final turn and ``step_source`` gives the index of the trajectory (the row of the generator input) a step came from."""
        keys = ("prompt_token_ids", "response_ids", "rewards", "loss_masks", "stop_reasons", "rollout_logprobs", "is_last_step",
                "step_source", "trajectory_generation_times", "env_metrics")
        out: GeneratorOutput = {k: [] for k in keys}
        tids = input_batch.get("trajectory_ids")
        out["trajectory_ids"] = [] if tids is not None else None
        for i, (steps, secs, metrics) in enumerate(res):
            for j, st in enumerate(steps):
                out["prompt_token_ids"].append(st["prompt"])
                out["response_ids"].append(st["response"])
                out["rewards"].append(st["rewards"])
                out["loss_masks"].append([1] * len(st["response"]))
                out["stop_reasons"].append(st["stop"])
                out["rollout_logprobs"].append(st["logprobs"])
                out["is_last_step"].append(j == len(steps) - 1)
                out["step_source"].append(i)
                out["trajectory_generation_times"].append(secs)
                out["env_metrics"].append(metrics)
                if tids is not None:
                    out["trajectory_ids"].append(tids[i])
        out["rollout_expert_indices"] = None
        last = [k for k, f in enumerate(out["is_last_step"]) if f]
        out["rollout_metrics"] = get_rollout_metrics([out["response_ids"][k] for k in last], [out["rewards"][k] for k in last],
                                                     [out["env_metrics"][k] for k in last])
        out["rollout_metrics"]["generate/steps_per_trajectory"] = len(out["is_last_step"]) / max(1, len(last))
        return out

    async def generate(self, input_batch: GeneratorInput) -> GeneratorOutput:
        n = len(input_batch["prompts"])
        if self.batched and self.max_turns == 1:
            return await self.generate_batched(input_batch)
        extras = input_batch.get("env_extras") or [{}] * n
        async def one(i):
            async with self.rate_limiter:
                return await self.agent_loop(input_batch["prompts"][i], input_batch["env_classes"][i], extras[i],
                                             input_batch.get("sampling_params"))

        res = await asyncio.gather(*[one(i) for i in range(n)])
        if self.step_wise:
            return self._flatten_steps(res, input_batch)
        out: GeneratorOutput = {
            "prompt_token_ids": [r[0] for r in res], "response_ids": [r[1] for r in res], "rewards": [r[2] for r in res],
            "loss_masks": [r[3] for r in res], "stop_reasons": [r[4] for r in res], "rollout_logprobs": [r[5] for r in res],
            "trajectory_generation_times": [r[6] for r in res], "env_metrics": [r[7] for r in res],
            "trajectory_ids": input_batch.get("trajectory_ids"), "rollout_expert_indices": None, "is_last_step": [True] * n,
        }
        out["rollout_metrics"] = get_rollout_metrics(out["response_ids"], out["rewards"], out["env_metrics"])
        return out
