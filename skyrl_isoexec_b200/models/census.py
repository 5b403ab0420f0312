"""Census of the dense GEMM sites of a model under a parallel layout (reference: ``gemm_census`` in
ISO/models/qwen3_5.py:137-155 and ``GemmSite`` in ISO/ops/mm/mm_shapes.py).

One ``GemmSite`` per distinct weight matrix shape that the batch-invariant GEMM serves: the contraction length K, the
output width N on one rank, the output dtype, how N or K is cut over tensor parallelism, and how many layers call it per
token. The census is derived from ``ModelConfig`` (never typed in by hand), so it covers every preset; it feeds tile
selection checks and the coverage report of a shape sweep. Routed experts are listed separately (``grouped=True``): they
run through the grouped GEMM, E/ep matrices per rank."""

from __future__ import annotations

from dataclasses import dataclass

from .config import ModelConfig


@dataclass(frozen=True)
class GemmSite:
    name: str
    k: int                    # contraction length on one rank
    n: int                    # output width on one rank
    out_dtype: str            # "bf16" | "fp32"
    sharding: str             # "column" (N cut over TP) | "row" (K cut over TP, followed by the TP sum) | "none"
    calls: int                # layers (passes per token) that use this shape
    grouped: bool = False     # expert matrices served by the grouped GEMM
    count: int = 1            # matrices per call on one rank (experts)

    def flops_per_token(self) -> int:
        """Multiply-adds x 2 of one token through this site; for expert sites, per expert the token is routed to."""
        return 2 * self.k * self.n * self.calls


def gemm_census(cfg: ModelConfig, tp: int = 1, ep: int = 1) -> list[GemmSite]:
    h = cfg.hidden_size
    act = "bf16" if cfg.dtype == "bfloat16" else "fp32"
    n_attn = sum(1 for i in range(cfg.num_layers) if cfg.layer_type(i) == "attn")
    n_gdn = cfg.num_layers - n_attn
    sites: list[GemmSite] = []

    def col(name, k, n_full, calls, dt=act):
        assert n_full % tp == 0, (name, n_full, tp)
        sites.append(GemmSite(name, k, n_full // tp, dt, "column", calls))

    def row(name, k_full, n, calls):
        assert k_full % tp == 0, (name, k_full, tp)
        sites.append(GemmSite(name, k_full // tp, n, act, "row", calls))

    def rep(name, k, n, calls, dt=act):
        sites.append(GemmSite(name, k, n, dt, "none", calls))

    if n_attn:
        H, D = cfg.num_q_heads, cfg.head_dim
        if cfg.is_mla:
            if cfg.q_lora_rank:
                rep("attn.q_a", h, cfg.q_lora_rank, n_attn)
                col("attn.q_b", cfg.q_lora_rank, H * D, n_attn)
            else:
                col("attn.q_b", h, H * D, n_attn)
            rep("attn.kv_a", h, cfg.kv_lora_rank + cfg.qk_rope_dim, n_attn)
            col("attn.kv_b", cfg.kv_lora_rank, H * (cfg.qk_nope_dim + cfg.v_head_dim), n_attn)
            row("attn.o", H * cfg.v_head_dim, h, n_attn)
        else:
            qkv = (H * (2 if cfg.attn_output_gate else 1) + 2 * cfg.num_kv_heads) * D
            if tp > cfg.num_kv_heads:       # KV heads replicated over tp / Hkv ranks
                rep_ = tp // cfg.num_kv_heads
                per = (H // cfg.num_kv_heads // rep_) * (2 if cfg.attn_output_gate else 1) * D + 2 * D
                sites.append(GemmSite("attn.qkv", h, per, act, "column", n_attn))
            else:
                col("attn.qkv", h, qkv, n_attn)
            row("attn.o", H * D, h, n_attn)
    if n_gdn:
        kd, vd = cfg.gdn_k_heads * cfg.gdn_head_dim, cfg.gdn_v_heads * cfg.gdn_head_dim
        col("gdn.in_proj", h, 2 * kd + 2 * vd + 2 * cfg.gdn_v_heads, n_gdn)
        row("gdn.out_proj", vd, h, n_gdn)
    L = cfg.num_layers
    if cfg.has_moe:
        rep("moe.router", h, cfg.num_experts, L, "fp32")
        assert cfg.num_experts % ep == 0
        sites.append(GemmSite("moe.experts.fc1", h, 2 * cfg.moe_ffn_size, act, "none", L, True, cfg.num_experts // ep))
        sites.append(GemmSite("moe.experts.fc2", cfg.moe_ffn_size, h, act, "none", L, True, cfg.num_experts // ep))
        if cfg.shared_expert_ffn:
            if cfg.shared_expert_gate:
                rep("moe.shared.gate", h, 1, L, "fp32")
            col("moe.shared.fc1", h, 2 * cfg.shared_expert_ffn, L)
            row("moe.shared.fc2", cfg.shared_expert_ffn, h, L)
    else:
        col("mlp.fc1", h, 2 * cfg.ffn_size, L)
        row("mlp.fc2", cfg.ffn_size, h, L)
    col("lm_head", h, cfg.vocab_size, 1)
    return sites


def census_table(cfg: ModelConfig, tp: int = 1, ep: int = 1) -> str:
    rows = ["site                 K       N  out   sharding  calls  matrices"]
    for s in gemm_census(cfg, tp, ep):
        rows.append(f"{s.name:18s} {s.k:6d} {s.n:7d}  {s.out_dtype:4s}  {s.sharding:8s} {s.calls:5d}  {s.count:8d}")
    return "\n".join(rows)
