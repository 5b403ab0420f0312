"""Batch containers exchanged between the controller and the workers.

``TensorBatch`` is a dict of tensors sharing dim 0 plus free-form metadata; it can be
sliced, chunked, concatenated, moved and pickled (tensors travel as CPU tensors). The field
names of ``TrainingInputBatch`` are the reference's (B/training_batch.py:463-480) so data
written by either framework reads in the other.

Sequence layout: ``sequences[b] = [PAD.. prompt | response ..PAD]`` with the prompt
left-padded to ``max_prompt`` and the response right-padded to ``max_response``;
response-level tensors are ``[B, max_response]``.
"""

from __future__ import annotations

import io
import pickle
from typing import Any, Iterable

import torch


class TensorBatch(dict):
    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.metadata: dict[str, Any] = {}
        self._check()

    def _check(self):
        n = None
        for k, v in self.items():
            if v is None:
                continue
            if not torch.is_tensor(v):
                raise TypeError(f"field {k!r} is {type(v).__name__}, expected a tensor")
            if n is None:
                n = v.shape[0]
            elif v.shape[0] != n:
                raise ValueError(f"field {k!r} has batch size {v.shape[0]}, expected {n}")

    @property
    def batch_size(self) -> int:
        for v in self.values():
            if v is not None:
                return v.shape[0]
        return 0

    def __len__(self) -> int:  # number of samples, like the reference's container
        return self.batch_size

    def to(self, device=None, dtype=None, non_blocking=False) -> "TensorBatch":
        out = type(self)({k: (None if v is None else v.to(device=device, non_blocking=non_blocking)) for k, v in self.items()})
        out.metadata = dict(self.metadata)
        return out

    def pin_memory(self) -> "TensorBatch":
        out = type(self)({k: (None if v is None else v.contiguous().pin_memory()) for k, v in self.items()})
        out.metadata = dict(self.metadata)
        return out

    def slice(self, lo: int, hi: int) -> "TensorBatch":
        out = type(self)({k: (None if v is None else v[lo:hi]) for k, v in self.items()})
        out.metadata = dict(self.metadata)
        return out

    def select(self, idx) -> "TensorBatch":
        idx = torch.as_tensor(idx, dtype=torch.long)
        out = type(self)({k: (None if v is None else v[idx]) for k, v in self.items()})
        out.metadata = dict(self.metadata)
        if "uids" in out.metadata and out.metadata["uids"] is not None:
            out.metadata["uids"] = [self.metadata["uids"][i] for i in idx.tolist()]
        return out

    def chunk(self, n: int) -> list["TensorBatch"]:
        B = self.batch_size
        if B % n:
            raise ValueError(f"batch size {B} is not divisible into {n} chunks")
        s = B // n
        return [self.slice(i * s, (i + 1) * s) for i in range(n)]

    @classmethod
    def cat(cls, batches: Iterable["TensorBatch"]) -> "TensorBatch":
        batches = list(batches)
        keys = list(batches[0].keys())
        out = cls({k: (None if batches[0][k] is None else torch.cat([b[k] for b in batches], 0)) for k in keys})
        out.metadata = dict(batches[0].metadata)
        return out

    def __getstate__(self):
        buf = io.BytesIO()
        torch.save({k: (None if v is None else v.detach().cpu()) for k, v in self.items()}, buf)
        return {"tensors": buf.getvalue(), "metadata": self.metadata}

    def __setstate__(self, st):
        self.clear()
        self.update(torch.load(io.BytesIO(st["tensors"]), weights_only=True))
        self.metadata = st["metadata"]

    def __reduce__(self):
        return (type(self), (), self.__getstate__())

    def dumps(self) -> bytes:
        return pickle.dumps(self)


class TrainingInputBatch(TensorBatch):
    """Fields: sequences, attention_mask, loss_mask, response_mask, action_log_probs,
    base_action_log_probs, values, returns, advantages, kl, rewards, rollout_logprobs."""


def pad_training_input_batch(batch: TrainingInputBatch, multiple: int) -> TrainingInputBatch:
    """Pad the batch to a multiple of ``multiple`` by cloning row 0 with a zero loss mask (the
    clones contribute nothing to any loss); records ``pad_size`` in the metadata."""
    B = batch.batch_size
    pad = (-B) % multiple
    if pad == 0:
        batch.metadata.setdefault("pad_size", 0)
        return batch
    out = {}
    for k, v in batch.items():
        if v is None:
            out[k] = None
            continue
        rep = v[:1].expand(pad, *v.shape[1:]).clone()
        if k in ("loss_mask", "response_mask"):
            rep.zero_()
        out[k] = torch.cat([v, rep], 0)
    nb = TrainingInputBatch(out)
    nb.metadata = dict(batch.metadata)
    nb.metadata["pad_size"] = pad
    if nb.metadata.get("uids") is not None:
        nb.metadata["uids"] = list(nb.metadata["uids"]) + [f"__pad{i}" for i in range(pad)]
    return nb


def build_sequences(prompts: list[list[int]], responses: list[list[int]], pad_id: int = 0,
                    max_prompt: int | None = None, max_response: int | None = None):
    """[PAD.. prompt | response ..PAD] tensors. Returns (sequences, attention_mask, response_mask)."""
    P = max_prompt or max(len(p) for p in prompts)
    R = max_response or max(1, max(len(r) for r in responses))
    B = len(prompts)
    seq = torch.full((B, P + R), pad_id, dtype=torch.long)
    att = torch.zeros(B, P + R, dtype=torch.long)
    rmask = torch.zeros(B, R, dtype=torch.float32)
    for i, (p, r) in enumerate(zip(prompts, responses)):
        p, r = p[-P:], r[:R]
        seq[i, P - len(p):P] = torch.tensor(p, dtype=torch.long)
        seq[i, P:P + len(r)] = torch.tensor(r, dtype=torch.long)
        att[i, P - len(p):P + len(r)] = 1
        rmask[i, :len(r)] = 1
    return seq, att, rmask
