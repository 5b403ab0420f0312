"""Multi-turn generator for vision-language policies (reference: R/train/generators/skyrl_vlm_generator.py).

The CONVERSATION is the source of truth: messages may hold images (in the prompt and in every observation an environment
returns), and before each model turn the whole conversation is rendered again (``engine/renderer.py``) into token ids in
which an image is a run of placeholder tokens, plus the images' patches. Generated tokens keep the logprobs the engine
reported; the tokens of an observation are what the next render appends behind the previous context (loss mask 0,
logprob 0), which is exact when rendering is prefix-stable and is CHECKED here: a render that does not extend the
context of the previous turn ends the trajectory with an error instead of training on misaligned tokens.

Besides the usual per-trajectory lists the output carries, per trajectory, ``pixel_values`` (all patches of all its
images, in order), ``image_grid_thw`` and ``mm_positions`` (where the placeholder tokens are, counted from the first
prompt token over prompt + response), which the trainer puts into the batch so that its forward splices the same
vision rows the engine used.

Not supported, as in the reference: single-call batched generation and step-wise trajectories.
"""

from __future__ import annotations

import asyncio
import copy
import time
from uuid import uuid4

import torch

from .. import gym
from .generator import GeneratorInput, GeneratorOutput, SkyRLGymGenerator, get_rollout_metrics


class SkyRLVLMGymGenerator(SkyRLGymGenerator):
    def __init__(self, engine, tokenizer=None, max_turns: int = 1, batched: bool = False, append_eos_after_stop_str: bool = False, **kw):
        if batched:
            raise ValueError("the vision-language generator renders every trajectory on its own: set generator.batched=false")
        if kw.get("step_wise"):
            raise ValueError("the vision-language generator does not produce step-wise trajectories")
        super().__init__(engine, tokenizer, max_turns=max_turns, batched=False, **kw)
        self.append_eos_after_stop_str = append_eos_after_stop_str

    async def _render(self, conversation: list[dict]) -> tuple[list[int], dict | None]:
        r = await self.engine.render_chat_completion({"json": {"messages": conversation}})
        return list(r["token_ids"]), r.get("features")

    async def agent_loop(self, prompt, env_class: str, env_extras: dict, sampling_params: dict | None, trajectory_id=None):
        t0 = time.time()
        session = f"{trajectory_id}" if trajectory_id is not None else uuid4().hex
        extras = dict(env_extras or {})
        extras.setdefault("max_turns", self.max_turns)
        env = gym.make(env_class, self.env_config, extras)
        conversation = copy.deepcopy(prompt)
        conversation, _ = env.init(conversation)
        prompt_ids, features = await self._render(conversation)
        resp, mask, lps = [], [], []
        step_rewards: list[tuple[float, int]] = []
        stop, done = "stop", False
        pending_obs_at: int | None = None          # where, in context coordinates, the last observation's tokens start
        stops = (sampling_params or {}).get("stop")
        eos = getattr(self.tokenizer, "eos_token_id", None)
        turns = 0
        while not done and turns < self.max_turns:
            turns += 1
            input_ids, features = await self._render(conversation)
            if input_ids[:len(prompt_ids) + len(resp)] != prompt_ids + resp:
                raise RuntimeError("rendering the conversation again did not reproduce the tokens generated so far: the chat "
                                   "template is not prefix-stable (for instance it strips earlier reasoning), which this "
                                   "generator cannot train on")
            if pending_obs_at is not None:
                obs = input_ids[pending_obs_at:]
                resp += obs
                mask += [0] * len(obs)
                lps += [0.0] * len(obs)
                pending_obs_at = None
            if len(input_ids) > self.max_input_length:
                stop = "length"
                break
            out = await self.engine.generate({"prompt_token_ids": [input_ids], "sampling_params": sampling_params,
                                              "session_ids": [session], "mm_features": [features] if features is not None else None})
            gen = list(out["response_ids"][0])
            glp = list((out.get("response_logprobs") or [[0.0] * len(gen)])[0])
            text = out["responses"][0] if out.get("responses") and out["responses"][0] else self._decode(gen)
            stop = out["stop_reasons"][0]
            added_eos = False
            if stops and self.append_eos_after_stop_str and eos is not None and gen and gen[-1] != eos and text.endswith(tuple(stops)):
                gen.append(eos)
                glp.append(0.0)
                added_eos = True
            step = env.step(text)
            done = bool(step["done"])
            conversation.append({"role": "assistant", "content": text})
            resp += gen
            mask += [1] * (len(gen) - 1) + [0] if added_eos else [1] * len(gen)
            lps += glp
            if gen:
                step_rewards.append((float(step["reward"]), len(resp) - 1))
            if not done:
                conversation.extend(step.get("observations") or [])
                pending_obs_at = len(input_ids) + len(gen)
        rewards = [0.0] * len(resp)
        for r, idx in step_rewards:
            rewards[idx] = r
        metrics = env.get_metrics()
        env.close()
        # the latest render covers every image of the trajectory that lies inside prompt + response (an observation
        # appended after the last model turn was never rendered, and is not part of the tokens either)
        n_tok = len(prompt_ids) + len(resp)
        if features is not None:
            pos = [p for p in features["positions"] if p < n_tok]
            if len(pos) != len(features["positions"]):
                raise RuntimeError("an image of the conversation lies behind the last trained token")   # cannot happen: renders precede turns
            pv, grid = features["pixel_values"], features["image_grid_thw"]
        else:
            pos, pv, grid = [], None, None
        return {"prompt_ids": prompt_ids, "response_ids": resp, "rewards": rewards, "loss_mask": mask, "stop_reason": stop,
                "logprobs": lps, "seconds": time.time() - t0, "env_metrics": metrics, "pixel_values": pv, "image_grid_thw": grid,
                "mm_positions": pos}

    async def generate(self, input_batch: GeneratorInput) -> GeneratorOutput:
        n = len(input_batch["prompts"])
        extras = input_batch.get("env_extras") or [{}] * n
        tids = input_batch.get("trajectory_ids")

        async def one(i):
            async with self.rate_limiter:
                return await self.agent_loop(input_batch["prompts"][i], input_batch["env_classes"][i], extras[i],
                                             input_batch.get("sampling_params"), tids[i] if tids is not None else None)

        res = await asyncio.gather(*[one(i) for i in range(n)])
        dim = next((r["pixel_values"].shape[1] for r in res if r["pixel_values"] is not None), 0)
        out: GeneratorOutput = {
            "prompt_token_ids": [r["prompt_ids"] for r in res], "response_ids": [r["response_ids"] for r in res],
            "rewards": [r["rewards"] for r in res], "loss_masks": [r["loss_mask"] for r in res],
            "stop_reasons": [r["stop_reason"] for r in res], "rollout_logprobs": [r["logprobs"] for r in res],
            "trajectory_generation_times": [r["seconds"] for r in res], "env_metrics": [r["env_metrics"] for r in res],
            "trajectory_ids": tids, "rollout_expert_indices": None, "is_last_step": [True] * n,
        }
        if dim:
            # a trajectory without images gets zero-row tensors, so that the three lists stay aligned with the samples
            out["pixel_values"] = [r["pixel_values"] if r["pixel_values"] is not None else torch.zeros(0, dim) for r in res]
            out["image_grid_thw"] = [r["image_grid_thw"] if r["image_grid_thw"] is not None else torch.zeros(0, 3, dtype=torch.int64) for r in res]
            out["mm_positions"] = [torch.tensor(r["mm_positions"], dtype=torch.int64) for r in res]
        out["rollout_metrics"] = get_rollout_metrics(out["response_ids"], out["rewards"], out["env_metrics"])
        return out
