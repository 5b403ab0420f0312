"""Engines the agents can talk to besides the in-process one (reference: skyrl-agent/skyrl_agent/integrations/{tinker,
skyrl_train}). An agent only needs ``await engine.generate({"prompt_token_ids": [...], "sampling_params": {...}})``
returning ``response_ids`` / ``response_logprobs`` / ``stop_reasons``; these adapters give that face to

  * a Tinker-style training service (``tinker/api.py``): sampling goes through its ``asample`` verb and futures, so the
    SAME model that the service is training serves the agent's turns, and the finished trajectories go back as
    ``forward_backward`` data (``trajectories_to_tinker_batch``);
  * an HTTP inference server group (``engine/server.py::RemoteInferenceClient`` already has this face).
"""

from __future__ import annotations

import asyncio

from .react import Trajectory


class TinkerSamplingEngine:
    def __init__(self, client, model_id: str):
        self.client, self.model_id = client, model_id
        self.calls = 0

    async def generate(self, batch: dict) -> dict:
        sp = dict(batch.get("sampling_params") or {})
        loop = asyncio.get_running_loop()

        def one(prompt):
            return self.client.call("asample", model_id=self.model_id, prompt_ids=list(prompt), num_samples=1, sampling_params=sp)

        outs = await asyncio.gather(*[loop.run_in_executor(None, one, p) for p in batch["prompt_token_ids"]])
        self.calls += len(outs)
        seqs = [o["sequences"][0] for o in outs]
        return {"response_ids": [s["tokens"] for s in seqs], "response_logprobs": [s["logprobs"] for s in seqs],
                "stop_reasons": [s["stop_reason"] for s in seqs]}


def trajectories_to_tinker_batch(trajs: list[Trajectory], advantages: list[float] | None = None) -> dict:
    """The ``data`` of a ``forward_backward`` request: one datum per trajectory with per-token loss weights (0 on
    observation tokens), the rollout logprobs and one advantage per trajectory broadcast over its model tokens (by
    default the trajectory's reward minus the mean reward of the batch)."""
    if advantages is None:
        mean = sum(t.reward for t in trajs) / max(1, len(trajs))
        advantages = [t.reward - mean for t in trajs]
    data = []
    for t, a in zip(trajs, advantages):
        data.append({"prompt_ids": list(t.prompt_ids), "response_ids": list(t.response_ids), "loss_mask": [float(m) for m in t.loss_mask],
                     "logprobs": list(t.logprobs), "advantages": [a * float(m) for m in t.loss_mask]})
    return {"data": data}
