"""Datasets and batching utilities (reference: R/train/dataset/*.py).

* ``PromptDataset``: rows {prompt (chat messages | string | token ids), env_class, reward_spec/extras} from
  JSONL or Parquet files, filtered by prompt length;
* sequence packing: first-fit-decreasing and balanced bin packing of sequences into token-budgeted bins;
* ``ReplayBuffer``: bounded FIFO of trajectories with staleness bookkeeping (used by the async trainer);
* prompt / mini-batch boundary helpers.
"""

from __future__ import annotations

from ..utils.tokenizer import chat_ids

import json
import random
from collections import deque


class PromptDataset:
    def __init__(self, paths, tokenizer=None, max_prompt_length: int = 1 << 30, env_class: str = "gsm8k",
                 prompt_key: str = "prompt", env_class_key: str = "env_class"):
        self.rows = []
        self.tokenizer = tokenizer
        for path in ([paths] if isinstance(paths, str) else list(paths)):
            for raw in self._read(path):
                prompt = raw.get(prompt_key)
                if prompt is None:
                    raise KeyError(f"{path}: row without {prompt_key!r}")
                if not self._prompt_not_too_long(prompt, max_prompt_length):
                    continue
                extras = {k: v for k, v in raw.items() if k not in (prompt_key, env_class_key)}
                self.rows.append({"prompt": prompt, "env_class": raw.get(env_class_key, env_class), "env_extras": extras,
                                  "uid": raw.get("uid", f"{len(self.rows)}")})

    @staticmethod
    def _read(path: str):
        if path.endswith(".jsonl"):
            with open(path) as f:
                for line in f:
                    if line.strip():
                        yield json.loads(line)
        elif path.endswith(".json"):
            with open(path) as f:
                yield from json.load(f)
        elif path.endswith(".parquet"):
            import pandas as pd

            yield from pd.read_parquet(path).to_dict("records")
        else:
            raise ValueError(f"unsupported dataset file {path!r} (jsonl | json | parquet)")

    def _prompt_not_too_long(self, prompt, limit: int) -> bool:
        if isinstance(prompt, (list, tuple)) and prompt and isinstance(prompt[0], int):
            return len(prompt) <= limit
        if self.tokenizer is None:
            return True
        if isinstance(prompt, str):
            return len(self.tokenizer.encode(prompt)) <= limit
        if any(isinstance(m.get("content"), (list, tuple)) for m in prompt):
            # multimodal messages: the text parts are measured here; the images' placeholder tokens depend on the model and
            # are counted by the generator against its max_input_length
            prompt = [dict(m, content="".join(p if isinstance(p, str) else p.get("text", "") for p in m["content"]))
                      if isinstance(m.get("content"), (list, tuple)) else m for m in prompt]
        return len(chat_ids(self.tokenizer, prompt)) <= limit

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]


# ------------------------------------------------------------------ packing
def pack_first_fit_decreasing(lengths: list[int], capacity: int) -> list[list[int]]:
    """Bins of sequence indices whose total length fits ``capacity`` (FFD). A sequence longer than the
    capacity gets a bin of its own."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins, room = [], []
    for i in order:
        n = lengths[i]
        for b, r in enumerate(room):
            if n <= r:
                bins[b].append(i)
                room[b] -= n
                break
        else:
            bins.append([i])
            room.append(max(0, capacity - n))
    return bins


def pack_balanced(lengths: list[int], num_bins: int) -> list[list[int]]:
    """``num_bins`` bins with near-equal total length (longest-first into the lightest bin): the
    length-balanced DP striping that removes the straggler tax of skewed micro-batches."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins = [[] for _ in range(num_bins)]
    load = [0] * num_bins
    for i in order:
        b = min(range(num_bins), key=lambda j: (load[j], j))
        bins[b].append(i)
        load[b] += lengths[i]
    return bins


def compute_prompt_boundaries(uids: list) -> list[tuple[int, int]]:
    """(start, end) slices of consecutive rows that share a uid."""
    out, lo = [], 0
    for i in range(1, len(uids) + 1):
        if i == len(uids) or uids[i] != uids[lo]:
            out.append((lo, i))
            lo = i
    return out


def compute_prompt_mini_batch_boundaries(uids: list, prompts_per_mini_batch: int) -> list[tuple[int, int]]:
    pb = compute_prompt_boundaries(uids)
    return [(pb[i][0], pb[min(i + prompts_per_mini_batch, len(pb)) - 1][1]) for i in range(0, len(pb), prompts_per_mini_batch)]


# ------------------------------------------------------------------ replay buffer
class ReplayBuffer:
    """Bounded FIFO of (item, policy_version) with staleness filtering."""

    def __init__(self, capacity: int, max_staleness: int | None = None, seed: int = 0):
        self.capacity, self.max_staleness = capacity, max_staleness
        self.items: deque = deque()
        self.rng = random.Random(seed)
        self.dropped_stale = 0

    def __len__(self):
        return len(self.items)

    def add(self, item, version: int) -> None:
        if len(self.items) >= self.capacity:
            self.items.popleft()
        self.items.append((item, version))

    def evict_stale(self, current_version: int) -> int:
        if self.max_staleness is None:
            return 0
        keep = deque(x for x in self.items if current_version - x[1] <= self.max_staleness)
        n = len(self.items) - len(keep)
        self.items = keep
        self.dropped_stale += n
        return n

    def pop_batch(self, n: int, current_version: int | None = None) -> list:
        if current_version is not None:
            self.evict_stale(current_version)
        n = min(n, len(self.items))
        return [self.items.popleft() for _ in range(n)]

    def sample(self, n: int) -> list:
        return self.rng.sample(list(self.items), min(n, len(self.items)))
