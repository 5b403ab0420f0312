"""Engine-side GatedDeltaNet state: a bounded pool of per-sequence rows holding, for every GDN
layer, the fp32 recurrent state [Hv, Dv, Dk] and the conv tail [C, W-1] (reference:
ISO/ops/gdn/gdn_recurrent_state.py:120-505). A sequence gets a row when it is first scheduled and
gives it back when it finishes; row 0 is a null lane that is never handed out. The state is not
checkpointed and is dropped on ``weight_sync`` and ``sleep_wake`` (the contract's state claim
``gdn_recurrent_state``): after either event every sequence restarts from position 0.
"""

from __future__ import annotations

import torch

from ..models.config import ModelConfig
from ..ops.gdn import GDNMeta


class GDNStatePool:
    def __init__(self, cfg: ModelConfig, max_seqs: int, device, tp: int = 1, layer_ids: list[int] | None = None):
        self.cfg, self.device = cfg, torch.device(device)
        self.rows = max_seqs + 1
        hk, hv, d = cfg.gdn_k_heads // tp, cfg.gdn_v_heads // tp, cfg.gdn_head_dim
        C, W = (2 * hk + hv) * d, cfg.gdn_conv_kernel
        self.layer_ids = list(layer_ids if layer_ids is not None else range(cfg.num_layers))
        dt = cfg.torch_dtype
        from ..ops.gdn import chunked_ok, new_chunk_buffers

        # per layer: conv tail, fp32 recurrent state at the sequence's last chunk boundary and, where the scan is the
        # chunked tensor-core form, the tokens of the sequence's open chunk (re-run in front of every new token)
        probe = torch.empty(0, dtype=dt, device=self.device)
        self.states = {
            i: (torch.zeros(self.rows, C, W - 1, dtype=dt, device=self.device),
                torch.zeros(self.rows, hv, d, d, dtype=torch.float32, device=self.device))
            + ((new_chunk_buffers(self.rows, hk, hv, d, dt, self.device),) if chunked_ok(probe, d) else ())
            for i in self.layer_ids if cfg.layer_type(i) == "gdn"
        }
        self.free = list(range(self.rows - 1, 0, -1))
        self.row_of: dict[int, int] = {}
        self.epoch = 0
        self.invalidations = {"weight_sync": 0, "sleep_wake": 0}
        # boundary states kept for the samples of one prompt: {leader seq id: [per-layer (conv tail, fp32 state), users left]}
        # (keyed by the request that computed the prefix, alive only while its siblings wait; the prefix-keyed store that
        # outlives requests is engine/prefix_cache.py::BoundaryStates)
        self.snapshots: dict[int, list] = {}

    def _row(self, seq_id: int) -> int:
        if seq_id not in self.row_of:
            if not self.free:
                raise RuntimeError("GDN state pool exhausted: raise max_num_seqs")
            self.row_of[seq_id] = self.free.pop()
        return self.row_of[seq_id]

    def release(self, seq_id: int) -> None:
        r = self.row_of.pop(seq_id, None)
        if r is not None:
            self.free.append(r)
        self.snapshots.pop(seq_id, None)

    # ------------------------------------------------------------------ boundary snapshots (samples of one prompt)
    def clone_row(self, seq_id: int) -> dict:
        """{layer: (conv tail, fp32 state)} of the sequence as they stand now. Meaningful as a resume point only when the
        sequence's open chunk is empty, i.e. right after a step that ended on a chunk boundary."""
        r = self.row_of[seq_id]
        return {i: (st[0][r].clone(), st[1][r].clone()) for i, st in self.states.items()}

    def load_row(self, seq_id: int, state: dict) -> None:
        """Start (or restart) ``seq_id`` from a cloned boundary state: its row gets the state's bits."""
        r = self._row(seq_id)
        for i, st in self.states.items():
            conv, ssm = state[i]
            st[0][r].copy_(conv)
            st[1][r].copy_(ssm)

    def snapshot(self, seq_id: int, users: int) -> None:
        """Copy the sequence's conv tail and fp32 state of every GDN layer as they stand now (called right after the step
        that brought its prefill to a chunk boundary, where its open chunk is empty)."""
        self.snapshots[seq_id] = [self.clone_row(seq_id), int(users)]

    def has_snapshot(self, seq_id: int) -> bool:
        return seq_id in self.snapshots

    def adopt(self, seq_id: int, leader_id: int) -> None:
        """Start ``seq_id`` from the leader's boundary state: its row gets the snapshot's bits."""
        snap = self.snapshots[leader_id]
        self.load_row(seq_id, snap[0])
        snap[1] -= 1
        if snap[1] <= 0:
            del self.snapshots[leader_id]

    def invalidate(self, event: str) -> None:
        """Drop every sequence's state (``weight_sync`` / ``sleep_wake``)."""
        assert event in ("weight_sync", "sleep_wake")
        self.free = list(range(self.rows - 1, 0, -1))
        self.row_of.clear()
        self.snapshots.clear()
        self.epoch += 1
        self.invalidations[event] += 1

    def step_meta(self, decode, prefill) -> GDNMeta:
        """Chunks in batch order: decode tokens first (one token each), then the prefill chunks. A chunk
        that starts at position 0 starts from a zero state; every chunk stores its final state."""
        chunks, tok = [], 0
        for s in decode:
            r = self._row(s.seq_id)
            p = s.length - 1
            chunks.append((tok, 1, p, r if p > 0 else -1, r))
            tok += 1
        for s, start, n in prefill:
            r = self._row(s.seq_id)
            chunks.append((tok, n, start, r if start > 0 else -1, r))
            tok += n
        return GDNMeta.build(chunks, self.device)

    def merge_into(self, kv_pools: list) -> list:
        """Per-layer state list for ``ForwardCtx.kv``: KV pools for attention layers, (conv, ssm) for GDN layers."""
        return [self.states[i] if self.cfg.layer_type(i) == "gdn" else kv_pools[j] for j, i in enumerate(self.layer_ids)]
