"""Paged KV cache: a pool of 128-slot pages per attention layer plus a page allocator.

One page == one key block of the attention kernel (ops/functional.PAGE), so a block table
row is exactly the list of TMA row coordinates the kernel walks. Pools are zero-initialised
and re-zeroed on wake-up: a masked key still enters P*V with weight 0, so stale bytes must be
finite (csrc/attention_tcgen05.cu).
"""

from __future__ import annotations

import torch

from ..models.config import ModelConfig
from ..ops.functional import PAGE


class PageAllocator:
    """Free list with reference counts: a page shared by several sequences (the common prompt of the samples of one
    request group) returns to the free list when its last holder releases it."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.free = list(range(num_pages - 1, -1, -1))
        self.refs = [0] * num_pages

    def can_alloc(self, n: int) -> bool:
        return len(self.free) >= n

    def alloc(self, n: int) -> list[int]:
        if len(self.free) < n:
            raise RuntimeError(f"out of KV pages: want {n}, have {len(self.free)}")
        out = [self.free.pop() for _ in range(n)]
        for p in out:
            self.refs[p] = 1
        return out

    def share(self, pages: list[int]) -> None:
        for p in pages:
            assert self.refs[p] > 0, f"page {p} is not in use"
            self.refs[p] += 1

    def release(self, pages: list[int]) -> None:
        for p in reversed(pages):
            self.refs[p] -= 1
            assert self.refs[p] >= 0, f"page {p} released twice"
            if self.refs[p] == 0:
                self.free.append(p)

    @property
    def num_free(self) -> int:
        return len(self.free)


class KVCache:
    """Per attention layer (k_pool, v_pool), each [num_pages*PAGE, Hkv_local, D]; GDN layers get
    ``None`` here (their state lives in ``engine.gdn_state``)."""

    def __init__(self, cfg: ModelConfig, num_pages: int, device, tp: int = 1, layer_ids: list[int] | None = None):
        self.cfg = cfg
        self.num_pages = num_pages
        self.device = torch.device(device)
        self.hkv = max(1, cfg.num_kv_heads // tp)
        self.layer_ids = list(layer_ids if layer_ids is not None else range(cfg.num_layers))
        self.allocator = PageAllocator(num_pages)
        self.pools: list | None = None
        self.invalidations = {"weight_sync": 0, "sleep_wake": 0}     # how often each lifecycle event really emptied the cache
        self.wake()

    @staticmethod
    def bytes_per_page(cfg: ModelConfig, tp: int = 1) -> int:
        n_attn = sum(1 for i in range(cfg.num_layers) if cfg.layer_type(i) == "attn")
        elt = 2 if cfg.dtype == "bfloat16" else 4
        return n_attn * 2 * PAGE * max(1, cfg.num_kv_heads // tp) * cfg.head_dim * elt

    def wake(self) -> None:
        if self.pools is not None:
            return
        dt = self.cfg.torch_dtype
        shape = (self.num_pages * PAGE, self.hkv, self.cfg.head_dim)
        self.pools = [
            (torch.zeros(shape, dtype=dt, device=self.device), torch.zeros(shape, dtype=dt, device=self.device))
            if self.cfg.layer_type(i) == "attn" else None
            for i in self.layer_ids
        ]

    def sleep(self) -> None:
        """Drop the pools (their memory returns to the allocator for the trainer); contents are
        never needed after a rollout phase ends."""
        self.pools = None
        self.allocator = PageAllocator(self.num_pages)
        self.invalidations["sleep_wake"] += 1

    def invalidate(self, event: str) -> bool:
        """A weight sync makes every cached key and value stale. Cached prefixes are dropped by the engine before this is
        called, so the cache is clean exactly when no page is in use at that moment. Returns whether it was, and counts clean invalidations so that
        the contract ledger sees that the event really emptied the cache instead of taking it on trust. (A sync while
        paused requests keep their pages, the in-flight update mode, is counted under ``stale_syncs``.)"""
        assert event in self.invalidations
        clean = self.pools is None or self.allocator.num_free == self.num_pages
        if clean:
            self.invalidations[event] += 1
        else:
            self.stale_syncs = getattr(self, "stale_syncs", 0) + 1
        return clean

    def slots_for(self, pages: list[int], start: int, n: int) -> list[int]:
        """Slots of positions start .. start+n-1 of a sequence whose pages are ``pages``."""
        return [pages[p // PAGE] * PAGE + p % PAGE for p in range(start, start + n)]
