"""Generator for REPL environments whose code blocks query the policy itself (reference: examples/train/rlm/rlm_generator.py
``RLMGymGenerator``): for every trajectory in an RLM-shaped environment it puts two callables into the environment's
extras before the environment is made,

* ``lm_callback(prompts) -> answers``: one plain completion of the CURRENT policy per prompt, through the same engine the
  rollout uses (chat template, the trajectory's sampling parameters with ``lm_max_tokens``);
* ``subcall_fn(prompt, context=None) -> answer``: a CHILD trajectory: a fresh environment of the same class on the sub-task,
  with ``context`` as its REPL context, run through the same agent loop one level deeper (children of children up to
  ``max_depth``; past it the call degrades to a plain completion). The child's final answer is what the parent's block
  gets back.

Children are real rollouts of the policy. With ``train_children=True`` every child trajectory is appended to the
generator's output as a sample of its own, rewarded with its ROOT trajectory's final reward (the children contributed to
that outcome), with ``trajectory_ids`` ``"<root>/c<k>"`` so that a group-relative estimator can tell them from the roots;
``step_source`` maps every row to the input row it came from. Without it they are only counted in the rollout metrics.

The callables are synchronous (they are called from inside ``exec``), while the engine interface is asynchronous: a call
made while an event loop is running in this thread is carried out on a helper thread with a loop of its own.
"""

from __future__ import annotations

from ..utils.tokenizer import chat_ids

import asyncio
import threading

from .generator import GeneratorInput, GeneratorOutput, SkyRLGymGenerator, get_rollout_metrics


def _run_sync(coro):
    try:
        asyncio.get_running_loop()
    except RuntimeError:
        return asyncio.run(coro)
    box: dict = {}

    def work():
        try:
            box["v"] = asyncio.run(coro)
        except BaseException as e:  # noqa: BLE001 - re-raised in the caller's thread
            box["e"] = e

    t = threading.Thread(target=work, daemon=True)
    t.start()
    t.join()
    if "e" in box:
        raise box["e"]
    return box["v"]


class RLMGymGenerator(SkyRLGymGenerator):
    RLM_ENV_CLASSES = {"rlm"}

    def __init__(self, engine, tokenizer=None, max_turns: int = 8, max_depth: int = 1, lm_max_tokens: int = 256,
                 train_children: bool = False, **kw):
        if tokenizer is None:
            raise ValueError("the RLM generator renders text prompts: it needs a tokenizer")
        kw["batched"] = False
        super().__init__(engine, tokenizer, max_turns=max_turns, **kw)
        self.max_depth, self.lm_max_tokens, self.train_children = max_depth, lm_max_tokens, train_children
        self._children: dict = {}            # root key -> [child trajectory tuples]

    # ------------------------------------------------------------------ callables handed to the environment
    def _complete(self, prompts: list[str], sampling_params: dict | None) -> list[str]:
        sp = dict(sampling_params or {})
        sp["max_generate_length"] = self.lm_max_tokens
        ids = [chat_ids(self.tokenizer, [{"role": "user", "content": p}])
               for p in prompts]
        out = _run_sync(self.engine.generate({"prompt_token_ids": ids, "sampling_params": sp}))
        return [self._decode(r) for r in out["response_ids"]]

    def _make_callbacks(self, env_class: str, extras: dict, sampling_params: dict | None, root, depth: int):
        def lm_callback(prompts):
            return self._complete(list(prompts), sampling_params)

        def subcall_fn(prompt, context=None):
            if depth >= self.max_depth:
                return lm_callback([prompt])[0]
            child_extras = {k: v for k, v in extras.items() if k not in ("lm_callback", "subcall_fn", "context", "extra_info", "reward_spec")}
            child_extras["context"] = context if context is not None else prompt
            child_extras["result_box"] = box = {}
            res = _run_sync(self._loop_at(prompt_of(prompt), env_class, child_extras, sampling_params, root, depth + 1))
            self._children.setdefault(root, []).append(res)
            return box.get("final") or ""

        def prompt_of(text):
            return [{"role": "user", "content": str(text)}]

        return lm_callback, subcall_fn

    async def _loop_at(self, prompt, env_class, extras, sampling_params, root, depth):
        ex = dict(extras or {})
        if env_class in self.RLM_ENV_CLASSES:
            ex["lm_callback"], ex["subcall_fn"] = self._make_callbacks(env_class, ex, sampling_params, root, depth)
        res = await SkyRLGymGenerator.agent_loop(self, prompt, env_class, ex, sampling_params)
        return res

    async def agent_loop(self, prompt, env_class: str, env_extras: dict, sampling_params: dict | None, root=None):
        return await self._loop_at(prompt, env_class, env_extras, sampling_params, root if root is not None else id(prompt), 0)

    # ------------------------------------------------------------------ output
    async def generate(self, input_batch: GeneratorInput) -> GeneratorOutput:
        n = len(input_batch["prompts"])
        extras = input_batch.get("env_extras") or [{}] * n
        self._children = {}

        async def one(i):
            async with self.rate_limiter:
                return await self.agent_loop(input_batch["prompts"][i], input_batch["env_classes"][i], extras[i],
                                             input_batch.get("sampling_params"), root=i)

        res = await asyncio.gather(*[one(i) for i in range(n)])
        tids = input_batch.get("trajectory_ids") or list(range(n))
        rows, source, ids = list(res), list(range(n)), list(tids)
        n_children = sum(len(v) for v in self._children.values())
        if self.train_children:
            for i in range(n):
                root_reward = sum(res[i][2]) if isinstance(res[i][2], list) else float(res[i][2])
                for k, ch in enumerate(self._children.get(i, [])):
                    ch = list(ch)
                    ch[2] = [0.0] * (len(ch[1]) - 1) + [root_reward] if ch[1] else []        # the root's outcome, on the child's last token
                    rows.append(tuple(ch))
                    source.append(i)
                    ids.append(f"{tids[i]}/c{k}")
        out: GeneratorOutput = {
            "prompt_token_ids": [r[0] for r in rows], "response_ids": [r[1] for r in rows], "rewards": [r[2] for r in rows],
            "loss_masks": [r[3] for r in rows], "stop_reasons": [r[4] for r in rows], "rollout_logprobs": [r[5] for r in rows],
            "trajectory_generation_times": [r[6] for r in rows], "env_metrics": [r[7] for r in rows],
            "trajectory_ids": ids, "rollout_expert_indices": None, "is_last_step": [True] * len(rows),
        }
        if self.train_children:
            out["step_source"] = source
        out["rollout_metrics"] = get_rollout_metrics(out["response_ids"][:n], out["rewards"][:n], out["env_metrics"][:n])
        out["rollout_metrics"]["generate/child_trajectories"] = n_children
        return out
