"""MoE training utilities: length-balanced data-parallel striping and rollout routing replay (reference:
B/utils/ep_balance.py DP row striping by length; B/utils/replay_utils.py rollout router replay).
"""

from __future__ import annotations

import torch


def balanced_dp_assignment(lengths: list[int], dp: int) -> list[list[int]]:
    """Sequences -> DP ranks so that every rank gets the same COUNT (needed by fixed micro-batching) and nearly the
    same token total: sort by length, deal out in a serpentine (0..dp-1, dp-1..0, ...)."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    out = [[] for _ in range(dp)]
    for j, i in enumerate(order):
        r = j % dp
        if (j // dp) % 2:
            r = dp - 1 - r
        out[r].append(i)
    return out


def imbalance(lengths: list[int], assignment: list[list[int]]) -> float:
    loads = [sum(lengths[i] for i in a) for a in assignment]
    return max(loads) / max(1e-9, sum(loads) / len(loads))


class RouterReplay:
    """Records the experts the ROLLOUT picked for every (layer, token) and makes the trainer's forward use the same
    picks, so that a routing flip caused by any numeric difference cannot turn into a large logprob difference.
    Under the bitwise contract the replayed picks equal the trainer's own (checked by ``mismatches``)."""

    def __init__(self):
        self.store: dict[int, torch.Tensor] = {}
        self.mode = "off"                      # off | record | replay
        self.flips = 0

    def record(self, layer: int, idx: torch.Tensor) -> None:
        self.store[layer] = idx.detach().to("cpu", copy=True) if layer not in self.store else torch.cat([self.store[layer], idx.detach().cpu()])

    def take(self, layer: int, start: int, n: int, device) -> torch.Tensor:
        return self.store[layer][start:start + n].to(device)

    def route(self, layer: int, idx_now: torch.Tensor, start: int = 0) -> torch.Tensor:
        """Called where the router's top-k has just been computed. Returns the indices to use."""
        if self.mode == "record":
            self.record(layer, idx_now)
            return idx_now
        if self.mode == "replay":
            want = self.take(layer, start, idx_now.shape[0], idx_now.device)
            self.flips += int((want.sort(-1).values != idx_now.sort(-1).values).any(-1).sum())
            return want
        return idx_now

    def clear(self) -> None:
        self.store.clear()
        self.flips = 0
