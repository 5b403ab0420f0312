"""Inference-engine API: the verbs and payloads of the reference's ``InferenceEngineInterface``
(B/inference_engines/base.py:25-201) on top of the native engine, plus a client that fans a
batch out over several engines (data-parallel rollout).

Payloads are plain dicts (``InferenceEngineInput`` / ``InferenceEngineOutput``) so they cross
process boundaries (HTTP, pipes, gloo object collectives) unchanged.
"""

from __future__ import annotations

import asyncio
from abc import ABC, abstractmethod
from typing import Any, TypedDict

from ..utils.tokenizer import chat_ids
from .llm_engine import EngineConfig, LLMEngine
from .sampler import SamplingParams


class InferenceEngineInput(TypedDict, total=False):
    prompts: list | None
    prompt_token_ids: list[list[int]] | None
    sampling_params: dict | None
    session_ids: list | None
    mm_features: Any


class InferenceEngineOutput(TypedDict, total=False):
    responses: list[str]
    response_ids: list[list[int]]
    stop_reasons: list[str]
    response_logprobs: list[list[float]] | None
    prompt_logprobs: Any
    rollout_expert_indices: Any


class InferenceEngineInterface(ABC):
    @abstractmethod
    async def generate(self, input_batch: InferenceEngineInput) -> InferenceEngineOutput: ...

    async def sample(self, prompt_token_ids: list[int], num_samples: int, sampling_params: dict) -> InferenceEngineOutput:
        """n samples of one prompt (Tinker-style)."""
        return await self.generate({"prompt_token_ids": [prompt_token_ids] * num_samples, "sampling_params": sampling_params})

    async def chat_completion(self, request_payload: dict) -> dict:
        raise NotImplementedError("chat_completion needs a tokenizer; use engine.server.OpenAIServer")

    async def completion(self, request_payload: dict) -> dict:
        raise NotImplementedError("completion needs a tokenizer; use engine.server.OpenAIServer")

    async def render_chat_completion(self, request_payload: dict) -> dict:
        """``{"json": {"messages": [...]}}`` -> ``{"token_ids", "features"}`` (``engine/renderer.py``): the ids the engine
        would be given for that conversation, with every image a run of placeholder tokens, and the images' patches."""
        raise NotImplementedError("rendering needs a tokenizer and a model configuration")

    @abstractmethod
    async def wake_up(self, *a, **kw): ...

    @abstractmethod
    async def sleep(self, *a, **kw): ...

    @abstractmethod
    async def init_weight_update_communicator(self, init_info): ...

    @abstractmethod
    async def update_named_weights(self, request): ...

    async def teardown(self):
        pass

    async def reset_prefix_cache(self):
        pass

    async def pause_generation(self):
        pass

    async def resume_generation(self):
        pass

    def tp_size(self) -> int:
        return 1

    def pp_size(self) -> int:
        return 1

    def dp_size(self) -> int:
        return 1


class NativeInferenceEngine(InferenceEngineInterface):
    """In-process engine over ``LLMEngine``."""

    def __init__(self, llm: LLMEngine, tokenizer=None):
        self.llm = llm
        self.tokenizer = tokenizer
        if tokenizer is not None and llm.detokenize is None:
            llm.detokenize = tokenizer.decode          # stop strings are matched on decoded text
        eos = getattr(tokenizer, "eos_token_id", None)
        if eos is not None and llm.cfg.eos_token_id is None:
            llm.cfg.eos_token_id = int(eos)            # a sequence ends at the tokenizer's end-of-sequence token (unless ignore_eos)
        self.receiver = None

    async def generate(self, input_batch: InferenceEngineInput) -> InferenceEngineOutput:
        ids = input_batch.get("prompt_token_ids")
        if ids is None:
            if self.tokenizer is None:
                raise ValueError("text prompts need a tokenizer; pass prompt_token_ids")
            ids = [self.tokenizer.encode(p) if isinstance(p, str) else
                   chat_ids(self.tokenizer, p)
                   for p in input_batch["prompts"]]
        sp = SamplingParams.from_dict(input_batch.get("sampling_params"))
        mm = input_batch.get("mm_features")
        if mm is not None:
            from .renderer import decode_features

            mm = [decode_features(f) for f in mm]
        outs = self.llm.generate(ids, sp, mm=mm)
        texts = [self.tokenizer.decode(o.response_ids) if self.tokenizer is not None else "" for o in outs]
        return {"responses": texts, "response_ids": [o.response_ids for o in outs],
                "stop_reasons": [o.stop_reason for o in outs],
                "response_logprobs": [o.response_logprobs for o in outs],
                "prompt_logprobs": [o.prompt_logprobs for o in outs] if sp.prompt_logprobs is not None else None,
                "rollout_expert_indices": None}

    async def render_chat_completion(self, request_payload: dict) -> dict:
        from .renderer import render_conversation

        if self.tokenizer is None:
            raise ValueError("rendering a conversation needs a tokenizer")
        body = request_payload.get("json", request_payload)
        return render_conversation(body["messages"], self.tokenizer, self.llm.mcfg, body.get("add_generation_prompt", True))

    async def wake_up(self, *a, tags=None, **kw):
        self.llm.wake_up(tags)

    async def sleep(self, *a, tags=None, **kw):
        self.llm.sleep(tags)

    async def init_weight_update_communicator(self, init_info):
        from ..sync.strategies import create_receiver

        self.receiver = create_receiver(init_info, self.llm.model)
        return True

    async def update_named_weights(self, request):
        if self.receiver is None:
            raise RuntimeError("update_named_weights before init_weight_update_communicator")
        from ..sync.strategies import load_weights

        load_weights(self.llm.model, self.receiver.receive_weights(request))
        self.llm.reset_prefix_cache()
        return True

    async def reset_prefix_cache(self):
        self.llm.reset_prefix_cache()

    async def pause_generation(self):
        self.llm.pause_generation()

    async def resume_generation(self):
        self.llm.resume_generation()

    def tp_size(self) -> int:
        return self.llm.model.ps.tp


class InferenceEngineClient(InferenceEngineInterface):
    """Routes a batch over several engines: prompts with a ``session_id`` stick to
    ``hash(session) % n``; the rest are split into contiguous, near-equal shards. Control-plane
    verbs fan out to every engine."""

    def __init__(self, engines: list[InferenceEngineInterface]):
        assert engines
        self.engines = engines

    def _route(self, n: int, session_ids):
        k = len(self.engines)
        if session_ids is not None:
            return [hash(str(s)) % k for s in session_ids]
        per = (n + k - 1) // k
        return [min(i // per, k - 1) for i in range(n)]

    async def generate(self, input_batch: InferenceEngineInput) -> InferenceEngineOutput:
        ids = input_batch.get("prompt_token_ids")
        prompts = input_batch.get("prompts")
        n = len(ids if ids is not None else prompts)
        route = self._route(n, input_batch.get("session_ids"))
        shards: dict[int, list[int]] = {}
        for i, e in enumerate(route):
            shards.setdefault(e, []).append(i)

        async def run(e, idx):
            sub: InferenceEngineInput = {"sampling_params": input_batch.get("sampling_params")}
            if ids is not None:
                sub["prompt_token_ids"] = [ids[i] for i in idx]
            else:
                sub["prompts"] = [prompts[i] for i in idx]
            if input_batch.get("mm_features") is not None:
                sub["mm_features"] = [input_batch["mm_features"][i] for i in idx]
            return idx, await self.engines[e].generate(sub)

        results = await asyncio.gather(*[run(e, idx) for e, idx in shards.items()])
        out: InferenceEngineOutput = {"responses": [None] * n, "response_ids": [None] * n, "stop_reasons": [None] * n,
                                      "response_logprobs": [None] * n, "prompt_logprobs": None,
                                      "rollout_expert_indices": None}
        for idx, r in results:
            for j, i in enumerate(idx):
                out["responses"][i] = r["responses"][j]
                out["response_ids"][i] = r["response_ids"][j]
                out["stop_reasons"][i] = r["stop_reasons"][j]
                out["response_logprobs"][i] = r["response_logprobs"][j] if r.get("response_logprobs") else None
        return out

    async def render_chat_completion(self, request_payload: dict) -> dict:
        return await self.engines[0].render_chat_completion(request_payload)       # a pure function of the conversation

    async def _all(self, name, *a, **kw):
        return await asyncio.gather(*[getattr(e, name)(*a, **kw) for e in self.engines])

    async def wake_up(self, *a, **kw):
        return await self._all("wake_up", *a, **kw)

    async def sleep(self, *a, **kw):
        return await self._all("sleep", *a, **kw)

    async def init_weight_update_communicator(self, init_info):
        return await asyncio.gather(*[e.init_weight_update_communicator(init_info.for_engine(i, e.tp_size(), e.pp_size(), e.dp_size())
                                                                        if hasattr(init_info, "for_engine") else init_info)
                                      for i, e in enumerate(self.engines)])

    async def update_named_weights(self, request):
        return await self._all("update_named_weights", request)

    async def reset_prefix_cache(self):
        return await self._all("reset_prefix_cache")

    async def pause_generation(self):
        return await self._all("pause_generation")

    async def resume_generation(self):
        return await self._all("resume_generation")

    async def teardown(self):
        return await self._all("teardown")

    def tp_size(self):
        return self.engines[0].tp_size()

    def dp_size(self):
        return len(self.engines)
