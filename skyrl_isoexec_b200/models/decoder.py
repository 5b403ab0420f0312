"""The one model definition both runtimes execute.

The reference reaches "same function on both sides" by running Megatron's ``GPTModel`` inside
vLLM (ISO/runtimes/vllm/gptmodel_vllm.py:217-222,278-408). Here trainer and rollout engine
instantiate this class directly, so the unified model is structural: the forward below is
the only forward there is, and the only difference between the sites is where K/V live
(fresh packed tensors with autograd for ``trainer_fwd``; a paged slot pool for the engine
sites and for ``trainer_score`` when it chooses to).

Weights live in ONE flat buffer per rank (``ParamStore``), Megatron-style, so that the
optimizer, the DP gradient reduction and the trainer->rollout weight sync each work on a
single contiguous range instead of hundreds of tensors.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from ..core import observe as _obs
from ..debug import trace as _trace
from ..ops import functional as F
from ..ops import gdn as gdn_ops
from ..ops import moe as moe_ops
from ..parallel.state import ParallelState
from ..parallel import tp as tp_ops
from .config import ModelConfig


# ------------------------------------------------------------------------------------ parameters
@dataclass
class ParamSpec:
    name: str
    shape: tuple[int, ...]       # local (sharded) shape
    full_shape: tuple[int, ...]  # unsharded shape
    shard_dim: int | None        # dim split over TP (None = replicated)
    init_std: float | None       # None = ones (norm weights), 0.0 = zeros
    offset: int = 0
    ep_sharded: bool = False     # leading expert dim split over EP
    sections: tuple[int, ...] = ()  # sizes of the blocks on shard_dim that are each split over TP
    tp_grad_sum: bool = False    # replicated weight used by the LOCAL heads only: its gradient is summed over TP
    kv_rep: int = 1              # fused QKV when tp > num_kv_heads: kv_rep consecutive TP ranks share one KV head (each
                                 # holds a slice of its query heads plus a full copy of k and v)
    kv_layout: tuple[int, ...] = ()   # (Hkv, G, rows per query head, D) of the full fused QKV


class ParamStore:
    """Flat parameter storage. ``flat`` holds every local parameter back to back (each start
    aligned to 128 elements so TMA bases stay 16-byte aligned); ``views[name]`` are the tensors
    the model computes with."""

    ALIGN = 128

    def __init__(self, specs: list[ParamSpec], dtype: torch.dtype, device, alloc=None):
        """``alloc(numel, dtype, device)`` supplies the flat buffer (e.g. from symmetric memory, so that peers can read
        the weights during a resharding weight sync); default: an ordinary zero-filled tensor."""
        off = 0
        for s in specs:
            s.offset = off
            n = math.prod(s.shape)
            off += (n + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        self.specs = {s.name: s for s in specs}
        self.order = [s.name for s in specs]
        self.numel = off
        self.flat = alloc(off, dtype, device) if alloc is not None else torch.zeros(off, dtype=dtype, device=device)
        assert self.flat.numel() >= off and self.flat.dtype == dtype
        self.views = {s.name: self.flat[s.offset:s.offset + math.prod(s.shape)].view(s.shape) for s in specs}

    def init_weights(self, seed: int, tp_rank: int = 0, tp: int = 1, ep_rank: int = 0, ep: int = 1) -> None:
        """Deterministic init: every parameter is drawn at FULL shape from a generator seeded by
        (seed, parameter name) and then sliced, so any TP/EP/PP layout holds the same model."""
        import zlib

        for name in self.order:
            s = self.specs[name]
            v = self.views[name]
            if s.init_std is None:
                v.fill_(1.0)
                continue
            if s.init_std == 0.0:
                v.zero_()
                continue
            g = torch.Generator(device="cpu").manual_seed(seed * 1000003 + zlib.crc32(name.encode()))
            full = torch.empty(s.full_shape, dtype=torch.float32).normal_(0.0, s.init_std, generator=g)
            v.copy_(shard_of(full, s, tp_rank, tp, ep_rank, ep).to(v.dtype))


def kv_rows(s: ParamSpec) -> tuple[int, int]:
    """(first row, number of rows) of the replicated k|v block inside a local fused-QKV shard with ``kv_rep > 1``."""
    Hkv, G, qs, D = s.kv_layout
    return (G // s.kv_rep) * qs, 2 * D


def unshard_kv_rep(parts: list[torch.Tensor], s: ParamSpec) -> torch.Tensor:
    """Full fused QKV from the shards of all TP ranks (rank order) when KV heads are replicated: per KV group the query
    slices of its ``kv_rep`` ranks, then k|v taken from the first of them."""
    Hkv, G, qs, D = s.kv_layout
    rep = s.kv_rep
    q_rows = (G // rep) * qs
    out = []
    for g in range(Hkv):
        mine = parts[g * rep:(g + 1) * rep]
        out += [m[:q_rows] for m in mine] + [mine[0][q_rows:]]
    return torch.cat(out, dim=0)


def shard_of(full: torch.Tensor, s: ParamSpec, tp_rank: int, tp: int, ep_rank: int = 0, ep: int = 1) -> torch.Tensor:
    """Slice a full-shape tensor to the local shard described by ``s``."""
    t = full
    if s.kv_rep > 1 and tp > 1:
        Hkv, G, qs, D = s.kv_layout
        rep = s.kv_rep
        g, j, gl = tp_rank // rep, tp_rank % rep, G // rep
        grp = t.reshape(Hkv, G * qs + 2 * D, -1)[g]
        return torch.cat([grp[j * gl * qs:(j + 1) * gl * qs], grp[G * qs:]], dim=0)
    if s.ep_sharded and ep > 1:
        e = t.shape[0] // ep
        t = t[ep_rank * e:(ep_rank + 1) * e]
    if s.shard_dim is not None and tp > 1:
        secs = s.sections or (t.shape[s.shard_dim],)
        parts, lo = [], 0
        for sz in secs:
            parts.append(t.narrow(s.shard_dim, lo + tp_rank * (sz // tp), sz // tp))
            lo += sz
        t = parts[0] if len(parts) == 1 else torch.cat(parts, dim=s.shard_dim)
    return t


def _qkv_rows(cfg: ModelConfig) -> int:
    return (cfg.num_q_heads * (2 if cfg.attn_output_gate else 1) + 2 * cfg.num_kv_heads) * cfg.head_dim


def build_param_specs(cfg: ModelConfig, ps: ParallelState, layer_range: range | None = None) -> list[ParamSpec]:
    """Parameter inventory of this rank. Column-parallel weights are split on dim 0 by whole
    heads / FFN columns, row-parallel weights on dim 1; MoE experts on the leading expert dim."""
    tp, h = ps.tp, cfg.hidden_size
    std = 0.02
    out_std = 0.02 / math.sqrt(2 * cfg.num_layers)
    specs: list[ParamSpec] = []

    def add(name, full_shape, shard_dim, init_std, ep_sharded=False, sections=()):
        shape = list(full_shape)
        for sz in sections:
            assert sz % tp == 0, (name, sections, tp)
        if ep_sharded and ps.ep > 1:
            assert shape[0] % ps.ep == 0
            shape[0] //= ps.ep
        if shard_dim is not None and tp > 1:
            assert shape[shard_dim] % tp == 0, (name, full_shape, tp)
            shape[shard_dim] //= tp
        per_head = name.endswith(("q_norm.weight", "k_norm.weight", "gdn.out_norm.weight"))
        specs.append(ParamSpec(name, tuple(shape), tuple(full_shape), shard_dim, init_std, ep_sharded=ep_sharded,
                               sections=tuple(sections), tp_grad_sum=per_head))

    layers = layer_range if layer_range is not None else range(cfg.num_layers)
    if ps.is_first_pp or cfg.tie_embeddings:
        add("embed.weight", (cfg.vocab_size, h), None, std)
    for i in layers:
        p = f"layers.{i}."
        add(p + "ln1.weight", (h,), None, 0.0 if cfg.zero_centered_norm else None)
        if cfg.layer_type(i) == "attn" and cfg.is_mla:
            # latent attention: low-rank query and key/value projections. The down-projections and their norms are
            # replicated; the up-projections and the output projection are cut over TP by whole heads.
            H, D, dn, dr, dv = cfg.num_q_heads, cfg.head_dim, cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.v_head_dim
            assert cfg.num_kv_heads == H and 0 < dr < D and 0 < dv <= D and not cfg.qk_norm and not cfg.attn_output_gate, \
                "latent attention: one KV head per query head, qk_rope_dim < head_dim, v_head_dim <= head_dim, no QK-norm or gate"
            if cfg.q_lora_rank:
                add(p + "attn.q_a.weight", (cfg.q_lora_rank, h), None, std)
                add(p + "attn.q_a_norm.weight", (cfg.q_lora_rank,), None, None)
                add(p + "attn.q_b.weight", (H * D, cfg.q_lora_rank), 0, std)           # per head: [rotated dr | un-rotated dn]
            else:
                add(p + "attn.q_b.weight", (H * D, h), 0, std)
            add(p + "attn.kv_a.weight", (cfg.kv_lora_rank + dr, h), None, std)           # [latent | shared rotated key]
            add(p + "attn.kv_a_norm.weight", (cfg.kv_lora_rank,), None, None)
            add(p + "attn.kv_b.weight", (H * (dn + dv), cfg.kv_lora_rank), 0, std)       # per head: [un-rotated key dn | value dv]
            add(p + "attn.o.weight", (h, H * dv), 1, out_std)
        elif cfg.layer_type(i) == "attn":
            # stored head-major per KV group so a TP shard holds whole GQA groups: [q-block | k | v] per shard
            if tp > cfg.num_kv_heads:
                # more TP ranks than KV heads: tp / Hkv consecutive ranks share a KV head; each keeps a slice of the
                # group's query heads and a full copy of its k and v rows (their gradients are summed over those ranks)
                Hkv, D = cfg.num_kv_heads, cfg.head_dim
                G, qs = cfg.num_q_heads // Hkv, (2 * D if cfg.attn_output_gate else D)
                assert tp % Hkv == 0 and G % (tp // Hkv) == 0, f"tp={tp} cannot replicate {Hkv} KV heads of {G}-head groups"
                rep = tp // Hkv
                specs.append(ParamSpec(p + "attn.qkv.weight", ((G // rep) * qs + 2 * D, h), (_qkv_rows(cfg), h), 0, std,
                                       kv_rep=rep, kv_layout=(Hkv, G, qs, D)))
            else:
                add(p + "attn.qkv.weight", (_qkv_rows(cfg), h), 0, std)
            add(p + "attn.o.weight", (h, cfg.num_q_heads * cfg.head_dim), 1, out_std)
            if cfg.qk_norm:
                add(p + "attn.q_norm.weight", (cfg.head_dim,), None, 0.0 if cfg.zero_centered_norm else None)
                add(p + "attn.k_norm.weight", (cfg.head_dim,), None, 0.0 if cfg.zero_centered_norm else None)
        else:
            kd, vd = cfg.gdn_k_heads * cfg.gdn_head_dim, cfg.gdn_v_heads * cfg.gdn_head_dim
            # in_proj rows: [q(kd) | k(kd) | v(vd) | z(vd) | b(Hv) | a(Hv)], split over TP by head
            add(p + "gdn.in_proj.weight", (2 * kd + 2 * vd + 2 * cfg.gdn_v_heads, h), 0, std,
                sections=(kd, kd, vd, vd, cfg.gdn_v_heads, cfg.gdn_v_heads))
            add(p + "gdn.conv.weight", (2 * kd + vd, cfg.gdn_conv_kernel), 0, 0.2, sections=(kd, kd, vd))
            add(p + "gdn.A_log", (cfg.gdn_v_heads,), 0, 0.0)
            add(p + "gdn.dt_bias", (cfg.gdn_v_heads,), 0, 0.0)
            add(p + "gdn.out_norm.weight", (cfg.gdn_head_dim,), None, 0.0 if cfg.zero_centered_norm else None)
            add(p + "gdn.out_proj.weight", (h, vd), 1, out_std)
        add(p + "ln2.weight", (h,), None, 0.0 if cfg.zero_centered_norm else None)
        if cfg.has_moe:
            E, f = cfg.num_experts, cfg.moe_ffn_size
            add(p + "moe.router.weight", (E, h), None, std)
            if cfg.router == "sigmoid_bias":
                add(p + "moe.router.expert_bias", (E,), None, 0.0)
            add(p + "moe.experts.gate_up", (E, 2 * f, h), None, std, ep_sharded=True)
            add(p + "moe.experts.down", (E, h, f), None, out_std, ep_sharded=True)
            if cfg.shared_expert_ffn:
                add(p + "moe.shared.gate_up.weight", (2 * cfg.shared_expert_ffn, h), 0, std,
                    sections=(cfg.shared_expert_ffn, cfg.shared_expert_ffn))
                add(p + "moe.shared.down.weight", (h, cfg.shared_expert_ffn), 1, out_std)
                if cfg.shared_expert_gate:
                    add(p + "moe.shared.gate.weight", (1, h), None, std)
        else:
            add(p + "mlp.gate_up.weight", (2 * cfg.ffn_size, h), 0, std, sections=(cfg.ffn_size, cfg.ffn_size))
            add(p + "mlp.down.weight", (h, cfg.ffn_size), 1, out_std)
    if ps.is_last_pp:
        add("final_norm.weight", (h,), None, 0.0 if cfg.zero_centered_norm else None)
        if not cfg.tie_embeddings:
            add("lm_head.weight", (cfg.vocab_size, h), 0, std)
    return specs


# ------------------------------------------------------------------------------------ forward context
@dataclass
class ForwardCtx:
    """Per-call inputs of the forward. ``kv`` is None at the differentiable trainer site
    (K/V are fresh packed tensors) and a list of per-layer state at the engine sites."""

    positions: torch.Tensor            # int32 [T]
    meta: F.AttnMeta
    slots: torch.Tensor | None = None  # int64 [T] slot of each token in the KV pools
    kv: list | None = None             # per attention layer: (k_pool, v_pool); per GDN layer: GDN state handle
    gdn_meta: object | None = None     # sequence layout for GDN layers (see ops/gdn.py)
    site: str = "trainer_fwd"          # trainer_fwd | trainer_score | engine_prefill | engine_decode
    sp_T: int | None = None            # set by the forward when sequence parallelism is on: total rows of the micro-batch
    mm: tuple | None = None            # vision-language: (rows int64 [n], features [n, hidden]) that replace embedding rows


class DecoderLM(nn.Module):
    def __init__(self, cfg: ModelConfig, ps: ParallelState | None = None, device="cpu", seed: int = 0,
                 layer_range: range | None = None, init: bool = True, flat_alloc=None):
        super().__init__()
        self.cfg = cfg
        self.ps = ps or ParallelState.single()
        self.device_ = torch.device(device)
        self.layer_ids = list(layer_range if layer_range is not None else range(cfg.num_layers))
        specs = build_param_specs(cfg, self.ps, layer_range)
        self.store = ParamStore(specs, cfg.torch_dtype, self.device_, alloc=flat_alloc)
        if init:
            self.store.init_weights(seed, self.ps.tp_rank, self.ps.tp, self.ps.ep_rank, self.ps.ep)
        self.params = nn.ParameterDict()
        self._p: dict[str, nn.Parameter] = {}
        for name in self.store.order:
            p = nn.Parameter(self.store.views[name], requires_grad=True)
            self._p[name] = p
            self.params[name.replace(".", "/")] = p
        self.rope = F.RopeTable(cfg.rot_dim, cfg.max_position, cfg.rope_theta, self.device_, scaling=cfg.rope_scaling_dict)
        self.scale = F.softmax_scale(cfg.head_dim)
        self.vision = None
        if getattr(cfg, "vision_depth", 0) > 0 and self.ps.is_first_pp:
            from .vision import VisionTower

            self.vision = VisionTower(cfg, self.device_, seed)       # frozen; same seed, same bits on every rank and side
        tp = self.ps.tp
        assert cfg.num_kv_heads % tp == 0 or tp % cfg.num_kv_heads == 0, "TP must divide, or be a multiple of, the KV heads"
        self.hq, self.hkv = cfg.num_q_heads // tp, max(1, cfg.num_kv_heads // tp)
        self.kv_rep = max(1, tp // cfg.num_kv_heads)
        if self.kv_rep > 1 and any(t == "attn" for t in (cfg.layer_type(i) for i in self.layer_ids)):
            assert getattr(self.ps, "kvr_ranks", None) and len(self.ps.kvr_ranks) == self.kv_rep, \
                f"KV heads are replicated over {self.kv_rep} ranks: build the process groups with kv_rep={self.kv_rep}"

    # -------------------------------------------------------------------------------- helpers
    def p(self, name: str) -> torch.Tensor:
        return self._p[name]

    def named_weights(self):
        """(name, local tensor) in storage order, the unit of weight sync and checkpoints."""
        for name in self.store.order:
            yield name, self.store.views[name]

    def embed(self, input_ids: torch.Tensor, mm: tuple | None = None) -> torch.Tensor:
        """Token embeddings; ``mm = (rows, features)`` puts the vision tower's rows in place of the image placeholder
        tokens' embeddings (out of place: the other rows keep their gradient path, the features carry none)."""
        x = torch.nn.functional.embedding(input_ids, self.p("embed.weight"))
        if mm is not None and mm[0].numel():
            x = x.index_copy(0, mm[0], mm[1].to(x.dtype))
        return x

    def lm_head_weight(self) -> torch.Tensor:
        if self.cfg.tie_embeddings:
            w = self.p("embed.weight")
            if self.ps.tp > 1:
                return tp_ops.tied_head_slice(w, self.ps)
            return w
        return self.p("lm_head.weight")

    # -------------------------------------------------------------------------------- layers
    def _attn_block(self, i: int, y: torch.Tensor, fc: ForwardCtx, kv_idx: int) -> torch.Tensor:
        cfg, pfx = self.cfg, f"layers.{i}.attn."
        T = fc.sp_T if fc.sp_T is not None else y.shape[0]
        qkv = F.linear(tp_ops.copy_to_tp(y, self.ps, fc.sp_T), self.p(pfx + "qkv.weight"))
        qw = self.p(pfx + "q_norm.weight") if cfg.qk_norm else None
        kw = self.p(pfx + "k_norm.weight") if cfg.qk_norm else None
        if fc.kv is None:
            q, k, v = F.qk_norm_rope_train(qkv, fc.positions, self.rope, qw, kw, self.hq, self.hkv, cfg.head_dim,
                                           cfg.rms_eps, cfg.qk_norm, cfg.zero_centered_norm, cfg.attn_output_gate)
            if self.ps.cp > 1:
                # context parallelism: tokens are cut over the cp ranks; an all-to-all gives every rank all tokens of a
                # slice of the heads for the attention kernel and the inverse brings the result back (bytes only)
                from ..parallel import cp as cp_ops

                a = cp_ops.ulysses_attention(q, k, v, fc.meta, self.scale, self.ps)
            else:
                a = F.attention(q, k, v, fc.meta, self.scale)
        else:
            k_pool, v_pool = fc.kv[kv_idx]
            q = F.qk_norm_rope_fwd(qkv, fc.positions, fc.slots, self.rope, qw, kw, k_pool, v_pool, self.hq, self.hkv,
                                   cfg.head_dim, cfg.rms_eps, cfg.qk_norm, cfg.zero_centered_norm, cfg.attn_output_gate)
            a, _ = F.attention_fwd(q, k_pool, v_pool, fc.meta, self.scale)
        if cfg.attn_output_gate:
            a = _gate_attn(a, qkv, self.hq, self.hkv, cfg.head_dim)
        return tp_ops.row_parallel_linear(a.reshape(T, self.hq * cfg.head_dim), self.p(pfx + "o.weight"), self.ps, cfg,
                                          sp=fc.sp_T is not None)

    def _mla_block(self, i: int, y: torch.Tensor, fc: ForwardCtx, kv_idx: int) -> torch.Tensor:
        """Multi-head latent attention (reference model: R/tx/models/deepseekv3.py) in its materialised form: the latent
        is expanded to per-head keys and values, which are laid out as an ordinary fused [q | k | v] row per head
        (rotated dims first, values zero-padded to the query/key width), so rotary, KV pool and the attention kernels are
        the ones every other family uses. The padding contributes exact zeros to every dot product; the padded output
        columns are dropped before the output projection. The KV pool therefore holds full keys and values, not the latent."""
        cfg, pfx, ps = self.cfg, f"layers.{i}.attn.", self.ps
        T, H, D, dn, dr, dv, r = y.shape[0], self.hq, cfg.head_dim, cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.v_head_dim, cfg.kv_lora_rank
        if cfg.q_lora_rank:
            qa, _ = F.rmsnorm(F.linear(y, self.p(pfx + "q_a.weight")), self.p(pfx + "q_a_norm.weight"), cfg.rms_eps, False)
        else:
            qa = y
        q = F.linear(tp_ops.copy_to_tp(qa, ps), self.p(pfx + "q_b.weight")).view(T, H, D)
        kva = F.linear(y, self.p(pfx + "kv_a.weight"))
        c, _ = F.rmsnorm(kva[:, :r].contiguous(), self.p(pfx + "kv_a_norm.weight"), cfg.rms_eps, False)
        k_rot = tp_ops.copy_to_tp(kva[:, r:].contiguous(), ps)                  # one rotated key shared by all heads
        kvb = F.linear(tp_ops.copy_to_tp(c, ps), self.p(pfx + "kv_b.weight")).view(T, H, dn + dv)
        k = torch.cat([k_rot.unsqueeze(1).expand(T, H, dr), kvb[..., :dn]], dim=-1)
        v = kvb[..., dn:]
        if dv < D:
            v = torch.nn.functional.pad(v, (0, D - dv))
        qkv = torch.cat([q, k, v], dim=-1).reshape(T, H * 3 * D)
        if fc.kv is None:
            q, k, v = F.qk_norm_rope_train(qkv, fc.positions, self.rope, None, None, H, H, D, cfg.rms_eps, False, False, False)
            a = F.attention(q, k, v, fc.meta, self.scale)
        else:
            k_pool, v_pool = fc.kv[kv_idx]
            q = F.qk_norm_rope_fwd(qkv, fc.positions, fc.slots, self.rope, None, None, k_pool, v_pool, H, H, D, cfg.rms_eps,
                                   False, False, False)
            a, _ = F.attention_fwd(q, k_pool, v_pool, fc.meta, self.scale)
        a = a[..., :dv].reshape(T, H * dv) if dv < D else a.reshape(T, H * D)
        return tp_ops.row_parallel_linear(a, self.p(pfx + "o.weight"), ps, cfg)

    def _mlp_block(self, i: int, y: torch.Tensor, fc: ForwardCtx | None = None) -> torch.Tensor:
        cfg, pfx = self.cfg, f"layers.{i}."
        if cfg.has_moe:
            return moe_ops.moe_block(y, self, i)
        wgu = self.p(pfx + "mlp.gate_up.weight")
        sp_T = fc.sp_T if fc is not None else None
        if sp_T is not None:
            y = tp_ops.copy_to_tp(y, self.ps, sp_T)              # all rows for the column-parallel gate|up GEMM
        if y.is_cuda and y.dtype == torch.bfloat16 and not torch.is_grad_enabled() and (wgu.shape[0] // 2) % 32 == 0 and y.dim() == 2:
            # gate_up GEMM with the SwiGLU applied in its epilogue (one launch, no [T, 2F] intermediate). The epilogue
            # repeats the roundings of the separate kernels, so this and the differentiable path below agree bit for bit.
            _obs.note("mm", "tcgen05_batch_invariant")
            _obs.note("activation.swiglu", "fused_swiglu")
            a = moe_ops.grouped_gemm(y, wgu.unsqueeze(0), None, moe_ops.EPI_GLU)
        else:
            a = F.swiglu(F.linear(y if sp_T is not None else tp_ops.copy_to_tp(y, self.ps), wgu))
        return tp_ops.row_parallel_linear(a, self.p(pfx + "mlp.down.weight"), self.ps, cfg, sp=sp_T is not None)

    def layer(self, i: int, x: torch.Tensor, res: torch.Tensor | None, fc: ForwardCtx, kv_idx: int):
        cfg = self.cfg
        y, res = _norm(x, self.p(f"layers.{i}.ln1.weight"), cfg, res)
        if cfg.layer_type(i) == "attn":
            o = self._mla_block(i, y, fc, kv_idx) if cfg.is_mla else self._attn_block(i, y, fc, kv_idx)
        else:
            o = gdn_ops.gdn_block(y, self, i, fc, kv_idx)
        y, res = _norm(o, self.p(f"layers.{i}.ln2.weight"), cfg, res)
        return self._mlp_block(i, y, fc), res

    def forward(self, input_ids: torch.Tensor | None, fc: ForwardCtx, hidden_in: tuple | None = None,
                checkpoint_layers: bool | int = False):
        """Returns the final-norm hidden states [T, hidden] on the last pipeline stage, else the
        (x, residual) pair to send to the next stage."""
        if hidden_in is None:
            x, res = self.embed(input_ids, fc.mm), None
        else:
            x, res = hidden_in
        fc.sp_T = None
        if self._sequence_parallel(fc, hidden_in):
            # Megatron-style sequence parallelism (trainer sites): from here to the final norm every rank carries its
            # T / tp rows of the residual stream; the tensor-parallel regions gather rows on entry and keep this rank's
            # rows of the tree sum on exit. Same kernels on the same rows: the forward bits do not change.
            fc.sp_T = int(x.shape[0])
            x = tp_ops.sp_scatter(x, self.ps)
        # checkpoint_layers: True = recompute every layer in the backward; an int n = recompute only the first n
        # layers of this stage (the last layers' activations are consumed first, so keeping them costs the least time)
        n_ckpt = len(self.layer_ids) if checkpoint_layers is True else int(checkpoint_layers)
        for kv_idx, i in enumerate(self.layer_ids):
            if kv_idx < n_ckpt and torch.is_grad_enabled():
                x, res = _ckpt(self, i, x, res, fc, kv_idx)
            else:
                x, res = self.layer(i, x, res, fc, kv_idx)
            if _trace.active() is not None:   # region door: residual-stream contribution of layer i
                _trace.record(f"layer{i}.out", x)
        if not self.ps.is_last_pp:
            return x, res
        y, _ = _norm(x, self.p("final_norm.weight"), self.cfg, res)
        if fc.sp_T is not None:
            y = tp_ops.sp_gather(y, fc.sp_T, self.ps, summed=False)     # the LM head's input gradient is already summed over TP
        if _trace.active() is not None:
            _trace.record("final_norm", y)
        return y

    def _sequence_parallel(self, fc: ForwardCtx, hidden_in) -> bool:
        c, ps = self.cfg, self.ps
        return bool(getattr(c, "sequence_parallel", False) and ps.tp > 1 and ps.cp == 1 and ps.pp == 1 and hidden_in is None
                    and fc.kv is None and not (c.has_moe or c.has_gdn or c.is_mla))

    @torch.no_grad()
    def ep_idle_forward(self) -> None:
        """A step with zero tokens under expert parallelism: take part in every MoE layer's collectives (and run this
        rank's experts on the rows the other ranks send) without doing anything else."""
        if not self.cfg.has_moe:
            return
        y = torch.empty(0, self.cfg.hidden_size, dtype=self.cfg.torch_dtype, device=self.device_)
        for i in self.layer_ids:
            moe_ops.moe_block(y, self, i)

    def logits(self, hidden: torch.Tensor, out_f32: bool = False) -> torch.Tensor:
        """Vocabulary logits of the given rows ([rows, V/tp] on this rank)."""
        return F.linear(hidden, self.lm_head_weight(), out_f32)


def _norm(x, w, cfg: ModelConfig, res):
    y, new_res = F.rmsnorm(x, w, cfg.rms_eps, cfg.zero_centered_norm, residual=res)
    return y, (new_res if new_res is not None else x)


def _gate_attn(a, qkv, hq, hkv, d):
    if torch.is_grad_enabled() and (a.requires_grad or qkv.requires_grad):
        T, G = a.shape[0], hq // hkv
        gate = qkv.view(T, hkv, G * 2 * d + 2 * d)[..., : G * 2 * d].reshape(T, hq, 2 * d)[..., d:]
        return a * torch.sigmoid(gate.float()).to(a.dtype)
    return F.sigmoid_gate(a, qkv, hq, hkv, d)


def _ckpt(model: DecoderLM, i, x, res, fc, kv_idx):
    from torch.utils.checkpoint import checkpoint

    if res is None:
        def run0(x_):
            return model.layer(i, x_, None, fc, kv_idx)
        return checkpoint(run0, x, use_reentrant=False)

    def run(x_, r_):
        return model.layer(i, x_, r_, fc, kv_idx)
    return checkpoint(run, x, res, use_reentrant=False)
