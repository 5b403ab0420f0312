"""A synthetic multi-turn VISUAL environment for vision-language policies (the reference exercises its VLM generator with
image observations from gym environments, tests/train/generators/test_skyrl_vlm_generator.py): the prompt shows an image
with ``k`` bright squares on a dark ground and asks how many there are; a wrong answer gets a fresh image of the same
count (squares at other places) as the next observation and another turn. Images are made from a seed, so a dataset row
only has to carry ``{"count": k, "seed": s}``."""

from __future__ import annotations

import re

import torch

from ..core import BaseTextEnv, register


def squares_image(count: int, seed: int, size: int = 64, cell: int = 16) -> torch.Tensor:
    """uint8 [3, size, size]: ``count`` bright cells of a (size / cell)^2 grid."""
    g = torch.Generator().manual_seed(int(seed))
    n = size // cell
    img = torch.full((3, size, size), 16, dtype=torch.uint8)
    for idx in torch.randperm(n * n, generator=g)[:count].tolist():
        r, c = divmod(idx, n)
        img[:, r * cell:(r + 1) * cell, c * cell:(c + 1) * cell] = 235
    return img


class VisualCountEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        spec = self.extras.get("reward_spec") or {}
        self.count = int(spec.get("count", self.extras.get("count", 1)))
        self.seed = int(self.extras.get("seed", 0))
        self.size = int(self.env_config.get("image_size", 64))

    def _image_message(self, text: str, seed: int) -> dict:
        return {"role": "user", "content": [{"type": "text", "text": text},
                                            {"type": "image", "image": squares_image(self.count, seed, self.size)}]}

    def init(self, prompt):
        """A prompt that already holds an image is kept; otherwise the question and the first image are appended."""
        has_image = any(isinstance(m.get("content"), (list, tuple)) and any(isinstance(p, dict) and p.get("type") in ("image", "image_url")
                                                                             for p in m["content"]) for m in prompt)
        if not has_image:
            prompt = list(prompt) + [self._image_message("How many bright squares are in this picture? Answer with a number.", self.seed)]
        return prompt, {}

    def step(self, action: str):
        self.turns += 1
        m = re.search(r"-?\d+", action)
        ok = m is not None and int(m.group(0)) == self.count
        done = ok or self.turns >= self.max_turns
        if done:
            return {"observations": [], "reward": 1.0 if ok else 0.0, "done": True, "metadata": {"answer": m.group(0) if m else None}}
        return {"observations": [self._image_message("Not right. Look at this one, it has as many:", self.seed + self.turns)],
                "reward": 0.0, "done": False, "metadata": {}}

    def get_metrics(self) -> dict:
        return {"turns": self.turns}


register("visual_count", lambda c, e: VisualCountEnv(c, e))
