"""CUDA-graph replay of the decode step.

A decode-only step (one token per running sequence) is launch-bound when run eagerly: ~10
kernels per layer, each a few microseconds. The step is therefore captured once per batch size
into a CUDA graph over STATIC buffers and replayed: per step the host writes one packed pinned
staging buffer (token ids, positions, KV slots, attention work items, block table), issues ONE
host-to-device copy, and launches the graph, which ends with the logits of every row.

What is static: all device addresses (inputs, KV pools, weights, outputs), the batch size and
the block-table width. What changes per step lives in the packed buffer. TMA tensor maps are
encoded on the host at capture time over those static addresses and travel in the kernel
parameters that the graph records. The contract's ``engine_decode`` case names exactly these
constraints (``cudagraph_capturable``, ``host_free``, ``address_stable``).
"""

from __future__ import annotations

import numpy as np
import torch

from ..models.decoder import ForwardCtx
from ..ops import functional as F


class DecodeGraph:
    def __init__(self, engine, batch: int, bt_width: int):
        self.engine, self.B, self.W = engine, batch, bt_width
        dev = engine.device
        B, W = batch, bt_width
        # packed layout, in int32 words: slots (int64 -> 2 words each) | ids | positions | items[B,8] | bt[B,W]
        self.o_slots, self.o_ids, self.o_pos, self.o_items, self.o_bt = 0, 2 * B, 3 * B, 4 * B, 12 * B
        self.words = 12 * B + B * W
        self.host = torch.zeros(self.words, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.words, dtype=torch.int32, device=dev)
        d = self.dev
        self.slots = d[self.o_slots:self.o_ids].view(torch.int64)
        self.ids = d[self.o_ids:self.o_pos]
        self.pos = d[self.o_pos:self.o_items]
        self.items = d[self.o_items:self.o_bt].view(B, 8)
        self.bt = d[self.o_bt:].view(B, W)
        self.graph = None
        self.logits = None

    def _forward(self):
        eng = self.engine
        fc = ForwardCtx(positions=self.pos, meta=F.AttnMeta(self.items, self.bt), slots=self.slots, kv=eng.cache.pools,
                        site="engine_decode")
        hidden = eng.model(self.ids, fc)
        return eng.model.logits(hidden)

    def capture(self):
        # warm-up on a side stream (sets function attributes, fills allocator pools), then capture
        s = torch.cuda.Stream(device=self.engine.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s), torch.no_grad():
            self._forward()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.logits = self._forward()

    def fill(self, ids, pos, slots, items, bt_rows):
        h = self.host_np
        B, W = self.B, self.W
        h[self.o_slots:self.o_ids].view(np.int64)[:] = slots
        h[self.o_ids:self.o_pos] = ids
        h[self.o_pos:self.o_items] = pos
        h[self.o_items:self.o_bt].reshape(B, 8)[:] = items
        btv = h[self.o_bt:].reshape(B, W)
        for i, r in enumerate(bt_rows):
            btv[i, :len(r)] = r

    def run(self) -> torch.Tensor:
        self.dev.copy_(self.host, non_blocking=True)
        self.engine.stats["h2d_bytes"] += self.words * 4
        self.graph.replay()
        return self.logits
