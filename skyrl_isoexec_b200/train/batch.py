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


class TensorList:
    """One tensor per sample, shapes free (``pixel_values[i]`` is ``[patches of sample i, dim]``; a sample without any is a
    tensor with zero rows). Behaves like a batch-major tensor for the container's slicing, selection, concatenation,
    device moves and pickling (reference: B/training_batch.py:50-130)."""

    def __init__(self, tensors: list[torch.Tensor]):
        self.tensors = list(tensors)
        for t in self.tensors:
            if not torch.is_tensor(t):
                raise TypeError(f"a TensorList holds tensors, got {type(t).__name__}")

    @property
    def shape(self) -> tuple:
        return (len(self.tensors),)

    def __len__(self) -> int:
        return len(self.tensors)

    def __iter__(self):
        return iter(self.tensors)

    def __getitem__(self, index):
        if isinstance(index, slice):
            return TensorList(self.tensors[index])
        if torch.is_tensor(index):
            if index.ndim == 0:
                return self.tensors[int(index)]
            index = index.tolist()
        if isinstance(index, (list, tuple)):
            return TensorList([self.tensors[int(i)] for i in index])
        return self.tensors[index]

    def to(self, device=None, dtype=None, non_blocking=False) -> "TensorList":
        return TensorList([t.to(device=device, non_blocking=non_blocking) for t in self.tensors])

    def contiguous(self) -> "TensorList":
        return TensorList([t.contiguous() for t in self.tensors])

    def pin_memory(self) -> "TensorList":
        return TensorList([t.pin_memory() if t.numel() else t for t in self.tensors])

    def detach(self) -> "TensorList":
        return TensorList([t.detach() for t in self.tensors])

    def cpu(self) -> "TensorList":
        return TensorList([t.cpu() for t in self.tensors])

    def expand_first(self, n: int) -> "TensorList":
        return TensorList([self.tensors[0].clone() for _ in range(n)])

    @staticmethod
    def cat(lists: list["TensorList"]) -> "TensorList":
        return TensorList([t for tl in lists for t in tl.tensors])

    def __eq__(self, other) -> bool:
        return isinstance(other, TensorList) and len(self) == len(other) and all(
            a.shape == b.shape and torch.equal(a, b) for a, b in zip(self.tensors, other.tensors))

    def __repr__(self) -> str:
        return f"TensorList({[tuple(t.shape) for t in self.tensors]})"


def _is_field(v) -> bool:
    return torch.is_tensor(v) or isinstance(v, TensorList)


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
            if not _is_field(v):
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
        join = lambda vs: TensorList.cat(vs) if isinstance(vs[0], TensorList) else torch.cat(vs, 0)
        out = cls({k: (None if batches[0][k] is None else join([b[k] for b in batches])) for k in keys})
        out.metadata = dict(batches[0].metadata)
        return out

    def __getstate__(self):
        buf = io.BytesIO()
        lists = sorted(k for k, v in self.items() if isinstance(v, TensorList))
        torch.save({k: (None if v is None else (v.detach().cpu().tensors if k in lists else v.detach().cpu())) for k, v in self.items()}, buf)
        return {"tensors": buf.getvalue(), "metadata": self.metadata, "lists": lists}

    def __setstate__(self, st):
        self.clear()
        d = torch.load(io.BytesIO(st["tensors"]), weights_only=True)
        for k in st.get("lists", ()):
            d[k] = TensorList(d[k])
        self.update(d)
        self.metadata = st["metadata"]

    def __reduce__(self):
        return (type(self), (), self.__getstate__())

    def dumps(self) -> bytes:
        return pickle.dumps(self)


class TrainingInputBatch(TensorBatch):
    """Fields: sequences, attention_mask, loss_mask, response_mask, action_log_probs,
    base_action_log_probs, values, returns, advantages, kl, rewards, rollout_logprobs; vision-language batches add
    ``pixel_values`` and ``image_grid_thw`` as ``TensorList`` fields (per sample: all patches / all grids of its images)."""


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
        if isinstance(v, TensorList):
            out[k] = TensorList.cat([v, v.expand_first(pad)])
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
