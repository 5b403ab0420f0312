"""CUDA-graph replay of the decode step.

A decode-only step (one token per running sequence) is launch-bound when run eagerly: ~10
kernels per layer, each a few microseconds. The step is therefore captured once per batch size
into a CUDA graph over STATIC buffers and replayed: per step the host writes one packed pinned
staging buffer (positions, KV slots, attention work items, block table, token ids), issues ONE
host-to-device copy, and launches the graph, which ends with the logits of every row. When the
engine runs one step ahead of the host, the token ids are not copied: the previous step's sampler
left them in the graph's id buffer.

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
        # packed layout, in int32 words: slots (int64 -> 2 words each) | positions | items[B,8] | bt[B,W] | ids.
        # The ids come last so that a step whose input tokens are already on the device (written there by the previous
        # step's sampler) copies only the words before them.
        self.o_slots, self.o_pos, self.o_items, self.o_bt = 0, 2 * B, 3 * B, 11 * B
        self.o_ids = 11 * B + B * W
        self.words = self.o_ids + B
        # two pinned staging buffers: the host may fill the next step's while the previous copy has not run yet
        self.hosts = [torch.zeros(self.words, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.hosts_np = [h.numpy() for h in self.hosts]
        self.parity = 0
        self.dev = torch.zeros(self.words, dtype=torch.int32, device=dev)
        d = self.dev
        self.slots = d[self.o_slots:self.o_pos].view(torch.int64)
        self.pos = d[self.o_pos:self.o_items]
        self.items = d[self.o_items:self.o_bt].view(B, 8)
        self.bt = d[self.o_bt:self.o_ids].view(B, W)
        self.ids = d[self.o_ids:]
        self.graph = None
        self.logits = None
        self.tp_calls = 0

    @property
    def host(self):
        return self.hosts[self.parity]

    def _forward(self):
        eng = self.engine
        fc = ForwardCtx(positions=self.pos, meta=F.AttnMeta(self.items, self.bt), slots=self.slots, kv=eng.cache.pools,
                        site="engine_decode")
        hidden = eng.model(self.ids, fc)
        return eng.model.logits(hidden)

    def _fused_tp(self):
        """The engine's fused tensor-parallel runtime, if its row-parallel GEMMs run as GEMM -> all-reduce kernels."""
        ps = self.engine.model.ps
        if ps.tp == 1:
            return None
        from ..parallel import tp_fused

        return tp_fused.get(ps.tp_group)

    def capture(self):
        # warm-up on a side stream (sets function attributes, fills allocator pools, runs the per-shape admission probes
        # of the fused tensor-parallel kernels, which compare on the host), then capture
        s = torch.cuda.Stream(device=self.engine.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s), torch.no_grad():
            self._forward()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        rt = self._fused_tp()
        self.graph = torch.cuda.CUDAGraph()
        if rt is not None:
            rt.begin_capture()       # calls are recorded with their epoch read from a device word
        try:
            with torch.cuda.graph(self.graph), torch.no_grad():
                self.logits = self._forward()
        finally:
            self.tp_calls = rt.end_capture() if rt is not None else 0

    def fill(self, ids, pos, slots, items, bt_rows):
        """Write the next step's inputs into the free staging buffer. ``ids`` None: the tokens are on the device."""
        self.parity ^= 1
        h = self.hosts_np[self.parity]
        B, W = self.B, self.W
        h[self.o_slots:self.o_pos].view(np.int64)[:] = slots
        h[self.o_pos:self.o_items] = pos
        h[self.o_items:self.o_bt].reshape(B, 8)[:] = items
        btv = h[self.o_bt:self.o_ids].reshape(B, W)
        for i, r in enumerate(bt_rows):
            btv[i, :len(r)] = r
        if ids is not None:
            h[self.o_ids:] = ids
        self._with_ids = ids is not None

    def run(self) -> torch.Tensor:
        n = self.words if self._with_ids else self.o_ids
        self.dev[:n].copy_(self.hosts[self.parity][:n], non_blocking=True)
        self.engine.stats["h2d_bytes"] += n * 4
        if self.tp_calls:
            self._fused_tp().before_replay(self.tp_calls)
        self.graph.replay()
        return self.logits
