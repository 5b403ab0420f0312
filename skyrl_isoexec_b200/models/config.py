"""Model configurations: one dataclass covers the four families the framework runs
(dense Qwen3, Qwen3-MoE, hybrid GatedDeltaNet, and tiny variants of each for tests)."""

from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace

import torch


@dataclass(frozen=True)
class ModelConfig:
    name: str
    architecture: str  # HF-style architecture string, keys the execution-contract profile
    vocab_size: int
    hidden_size: int
    num_layers: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    ffn_size: int
    rope_theta: float = 1e6
    rope_scaling: tuple = ()           # a Hugging Face rope_scaling mapping as sorted (key, value) pairs: linear | llama3 | yarn
    rms_eps: float = 1e-6
    tie_embeddings: bool = False
    qk_norm: bool = True
    max_position: int = 8192
    dtype: str = "bfloat16"
    # --- MoE (num_experts == 0 -> dense MLP)
    num_experts: int = 0
    top_k: int = 0
    moe_ffn_size: int = 0
    router: str = "softmax"  # "softmax" | "sigmoid_bias"
    norm_topk_prob: bool = True
    shared_expert_ffn: int = 0
    shared_expert_gate: bool = False   # the shared expert's output is scaled by sigmoid(x . w_gate), one scalar per token
    # --- hybrid GatedDeltaNet
    layer_types: tuple[str, ...] = ()  # per layer "attn" | "gdn"; empty = all attention
    gdn_k_heads: int = 0
    gdn_v_heads: int = 0
    gdn_head_dim: int = 0
    gdn_conv_kernel: int = 4
    gdn_chunk: int = 64
    gdn_snapshot: bool = False         # "cpr" scan: the fp32 state is rounded to the activation dtype at every chunk boundary
    attn_output_gate: bool = False
    zero_centered_norm: bool = False
    partial_rotary_factor: float = 1.0
    # --- multi-head latent attention (DeepSeek-V2/V3 style); on when kv_lora_rank > 0. Every query head has its own key
    # and value head (num_kv_heads == num_q_heads); head_dim = qk_rope_dim + the un-rotated part; v_head_dim <= head_dim
    kv_lora_rank: int = 0
    q_lora_rank: int = 0         # 0 = a plain query projection
    qk_rope_dim: int = 0
    v_head_dim: int = 0
    # --- vision tower (vision_depth == 0 -> text only); models/vision.py
    vision_depth: int = 0
    vision_hidden: int = 0
    vision_heads: int = 0
    vision_patch: int = 14
    vision_merge: int = 2          # merge x merge neighbouring patches become one placeholder token
    vision_max_grid: int = 64      # largest image side, in patches
    image_token_id: int = -1       # the placeholder token; its embedding rows are replaced by the tower's output
    # --- numerics pins that enter the execution contract
    logprob_leaves: int = 8
    pik_leaves: int = 8
    tp_invariant: bool = False  # row-parallel K reductions use the leaf tree so any TP | pik_leaves gives equal bits
    sequence_parallel: bool = False  # trainer forward: residual stream, norms and adds on T / tp rows per rank (dense attention models)

    def __post_init__(self):
        rs = self.rope_scaling
        if isinstance(rs, dict):
            object.__setattr__(self, "rope_scaling", tuple(sorted(rs.items())))
        elif rs is None:
            object.__setattr__(self, "rope_scaling", ())
        elif isinstance(rs, list):
            object.__setattr__(self, "rope_scaling", tuple(tuple(x) for x in rs))

    @property
    def rope_scaling_dict(self) -> dict | None:
        return dict(self.rope_scaling) if self.rope_scaling else None

    @property
    def torch_dtype(self) -> torch.dtype:
        return {"bfloat16": torch.bfloat16, "float32": torch.float32}[self.dtype]

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def qk_nope_dim(self) -> int:
        return self.head_dim - self.qk_rope_dim

    @property
    def rot_dim(self) -> int:
        if self.is_mla:
            return self.qk_rope_dim
        r = int(self.head_dim * self.partial_rotary_factor)
        return r - (r % 16) if r % 16 else r

    @property
    def has_vision(self) -> bool:
        return self.vision_depth > 0

    @property
    def has_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def has_gdn(self) -> bool:
        return any(t == "gdn" for t in self.layer_types)

    def layer_type(self, i: int) -> str:
        return self.layer_types[i] if self.layer_types else "attn"

    def to_dict(self) -> dict:
        d = asdict(self)
        d["layer_types"] = list(self.layer_types)
        d["rope_scaling"] = dict(self.rope_scaling)
        return d

    @staticmethod
    def from_dict(d: dict) -> "ModelConfig":
        d = dict(d)
        d["layer_types"] = tuple(d.get("layer_types", ()))
        return ModelConfig(**d)

    def with_(self, **kw) -> "ModelConfig":
        return replace(self, **kw)

    def param_count(self) -> int:
        h, L = self.hidden_size, self.num_layers
        attn = h * (self.num_q_heads * (2 if self.attn_output_gate else 1) + 2 * self.num_kv_heads) * self.head_dim \
            + self.num_q_heads * self.head_dim * h
        if self.is_mla:
            H, D = self.num_q_heads, self.head_dim
            q = (h * self.q_lora_rank + self.q_lora_rank * H * D) if self.q_lora_rank else h * H * D
            attn = q + h * (self.kv_lora_rank + self.qk_rope_dim) + self.kv_lora_rank * H * (self.qk_nope_dim + self.v_head_dim) \
                + H * self.v_head_dim * h
        if self.has_moe:
            mlp = self.num_experts * 3 * h * self.moe_ffn_size + h * self.num_experts + 3 * h * self.shared_expert_ffn
        else:
            mlp = 3 * h * self.ffn_size
        emb = self.vocab_size * h * (1 if self.tie_embeddings else 2)
        return L * (attn + mlp) + emb


def _hybrid_pattern(n: int) -> tuple[str, ...]:
    return tuple("attn" if (i % 4) == 3 else "gdn" for i in range(n))


PRESETS: dict[str, ModelConfig] = {
    # tiny Qwen3-style decoder for the CPU / gloo runs
    "tiny-qwen3": ModelConfig(
        name="tiny-qwen3", architecture="Qwen3ForCausalLM", vocab_size=2048, hidden_size=256, num_layers=2,
        num_q_heads=4, num_kv_heads=2, head_dim=64, ffn_size=768, tie_embeddings=True, dtype="float32",
        max_position=512),
    "qwen3-8b": ModelConfig(
        name="qwen3-8b", architecture="Qwen3ForCausalLM", vocab_size=151936, hidden_size=4096, num_layers=36,
        num_q_heads=32, num_kv_heads=8, head_dim=128, ffn_size=12288, max_position=40960),
    "qwen3-32b": ModelConfig(
        name="qwen3-32b", architecture="Qwen3ForCausalLM", vocab_size=151936, hidden_size=5120, num_layers=64,
        num_q_heads=64, num_kv_heads=8, head_dim=128, ffn_size=25600, max_position=40960),
    "qwen3-30b-a3b": ModelConfig(
        name="qwen3-30b-a3b", architecture="Qwen3MoeForCausalLM", vocab_size=151936, hidden_size=2048, num_layers=48,
        num_q_heads=32, num_kv_heads=4, head_dim=128, ffn_size=0, num_experts=128, top_k=8, moe_ffn_size=768,
        max_position=40960),
    # hybrid [GDN, GDN, GDN, gated attention] x 8 (the reference's Qwen3.5-style benchmark model)
    "qwen3.5-hybrid": ModelConfig(
        name="qwen3.5-hybrid", architecture="Qwen3NextForCausalLM", vocab_size=151936, hidden_size=2560,
        num_layers=32, num_q_heads=16, num_kv_heads=4, head_dim=128, ffn_size=9216,
        layer_types=_hybrid_pattern(32), gdn_k_heads=16, gdn_v_heads=32, gdn_head_dim=128, attn_output_gate=True,
        zero_centered_norm=True, max_position=40960),
    # the reference's own manifest model (ISO/models/qwen3_5.py:120-134): hybrid GDN + gated attention, 256 routed experts
    # plus a gated shared expert. Its 256-wide attention heads have no instance in the attention kernels yet (64 and 128
    # only), so on a GPU this preset builds and shards but does not run; the tiny variant below runs everywhere.
    "qwen3.5-35b-a3b": ModelConfig(
        name="qwen3.5-35b-a3b", architecture="Qwen3_5MoeForCausalLM", vocab_size=248320, hidden_size=2048, num_layers=40,
        num_q_heads=16, num_kv_heads=2, head_dim=256, ffn_size=0, layer_types=_hybrid_pattern(40), gdn_k_heads=16,
        gdn_v_heads=32, gdn_head_dim=128, attn_output_gate=True, zero_centered_norm=True, partial_rotary_factor=0.25,
        num_experts=256, top_k=8, moe_ffn_size=512, shared_expert_ffn=512, shared_expert_gate=True, max_position=40960),
    "tiny-hybrid-moe": ModelConfig(
        name="tiny-hybrid-moe", architecture="Qwen3_5MoeForCausalLM", vocab_size=2048, hidden_size=256, num_layers=4,
        num_q_heads=4, num_kv_heads=2, head_dim=64, ffn_size=0, layer_types=_hybrid_pattern(4), gdn_k_heads=2,
        gdn_v_heads=4, gdn_head_dim=64, attn_output_gate=True, zero_centered_norm=True, partial_rotary_factor=0.25,
        num_experts=8, top_k=2, moe_ffn_size=128, shared_expert_ffn=128, shared_expert_gate=True, dtype="float32",
        max_position=512),
    # Llama-3 style dense decoder (the reference's tx model zoo, R/tx/models/llama3.py): no QK-norm, untied head
    "llama3-8b": ModelConfig(
        name="llama3-8b", architecture="LlamaForCausalLM", vocab_size=128256, hidden_size=4096, num_layers=32,
        num_q_heads=32, num_kv_heads=8, head_dim=128, ffn_size=14336, qk_norm=False, rope_theta=5e5, rms_eps=1e-5,
        max_position=8192),
    "tiny-llama": ModelConfig(
        name="tiny-llama", architecture="LlamaForCausalLM", vocab_size=2048, hidden_size=256, num_layers=2,
        num_q_heads=4, num_kv_heads=2, head_dim=64, ffn_size=768, qk_norm=False, rope_theta=5e5, rms_eps=1e-5,
        tie_embeddings=False, dtype="float32", max_position=512),
    # DeepSeek-V3 style (the reference's tx model zoo, R/tx/models/deepseekv3.py): latent attention with low-rank query
    # and key/value projections, sigmoid router with a selection bias, one shared expert. Sized so that the query/key head
    # (rotated 64 + un-rotated 64) fits the 128-wide attention kernels
    "deepseek-mla-16b": ModelConfig(
        name="deepseek-mla-16b", architecture="DeepseekV3ForCausalLM", vocab_size=129280, hidden_size=2048, num_layers=27,
        num_q_heads=16, num_kv_heads=16, head_dim=128, ffn_size=0, qk_norm=False, rope_theta=1e4, kv_lora_rank=512,
        q_lora_rank=768, qk_rope_dim=64, v_head_dim=128, num_experts=64, top_k=6, moe_ffn_size=1408, router="sigmoid_bias",
        shared_expert_ffn=2816, max_position=16384),
    "tiny-mla": ModelConfig(
        name="tiny-mla", architecture="DeepseekV3ForCausalLM", vocab_size=2048, hidden_size=256, num_layers=2,
        num_q_heads=4, num_kv_heads=4, head_dim=64, ffn_size=768, qk_norm=False, rope_theta=1e4, kv_lora_rank=64,
        q_lora_rank=96, qk_rope_dim=32, v_head_dim=48, dtype="float32", max_position=512),
    "tiny-deepseek": ModelConfig(
        name="tiny-deepseek", architecture="DeepseekV3ForCausalLM", vocab_size=2048, hidden_size=256, num_layers=2,
        num_q_heads=4, num_kv_heads=4, head_dim=64, ffn_size=0, qk_norm=False, rope_theta=1e4, kv_lora_rank=64,
        q_lora_rank=0, qk_rope_dim=32, v_head_dim=64, num_experts=8, top_k=2, moe_ffn_size=128, router="sigmoid_bias",
        shared_expert_ffn=128, dtype="float32", max_position=512),
    # small variants used by tests and smoke runs
    "tiny-qwen3-bf16": ModelConfig(
        name="tiny-qwen3-bf16", architecture="Qwen3ForCausalLM", vocab_size=2048, hidden_size=256, num_layers=2,
        num_q_heads=4, num_kv_heads=2, head_dim=128, ffn_size=768, tie_embeddings=False, max_position=1024),
    "tiny-moe": ModelConfig(
        name="tiny-moe", architecture="Qwen3MoeForCausalLM", vocab_size=2048, hidden_size=256, num_layers=2,
        num_q_heads=4, num_kv_heads=2, head_dim=64, ffn_size=0, num_experts=8, top_k=2, moe_ffn_size=128,
        dtype="float32", max_position=512),
    # vision-language: the tiny Qwen3 decoder with a two-block vision tower; token 2047 is the image placeholder
    "tiny-vl": ModelConfig(
        name="tiny-vl", architecture="Qwen3ForCausalLM", vocab_size=2048, hidden_size=256, num_layers=2,
        num_q_heads=4, num_kv_heads=2, head_dim=64, ffn_size=768, tie_embeddings=True, dtype="float32",
        max_position=1024, vision_depth=2, vision_hidden=64, vision_heads=4, vision_patch=8, vision_merge=2,
        vision_max_grid=16, image_token_id=2047),
    "tiny-hybrid": ModelConfig(
        name="tiny-hybrid", architecture="Qwen3NextForCausalLM", vocab_size=2048, hidden_size=256, num_layers=4,
        num_q_heads=4, num_kv_heads=2, head_dim=64, ffn_size=512, layer_types=_hybrid_pattern(4), gdn_k_heads=2,
        gdn_v_heads=4, gdn_head_dim=64, attn_output_gate=True, zero_centered_norm=True, dtype="float32",
        max_position=512),
}


def config_from_hf(path: str) -> ModelConfig:
    """Resolve a model from a Hugging Face style directory (or its ``config.json``): ``architectures[0]`` selects the family,
    the size fields fill the rest (reference: the model-resolution step that reads ``config.json`` from a path or the HF
    cache before choosing a manifest, ISO/models/resolve.py). Families: Qwen3, Qwen3-MoE, Qwen3-Next / Qwen3.5 hybrids,
    Llama, DeepSeek-V3."""
    import json
    import os

    f = os.path.join(path, "config.json") if os.path.isdir(path) else path
    with open(f) as fh:
        c = json.load(fh)
    c = {**c.get("text_config", {}), **{k: v for k, v in c.items() if k != "text_config"}}
    arch = (c.get("architectures") or ["?"])[0]
    fam = {"Qwen3ForCausalLM": "dense", "Qwen2ForCausalLM": "dense", "LlamaForCausalLM": "dense", "MistralForCausalLM": "dense",
           "Qwen3MoeForCausalLM": "moe", "Qwen3NextForCausalLM": "hybrid", "Qwen3_5MoeForCausalLM": "hybrid",
           "Qwen3_5ForCausalLM": "hybrid", "DeepseekV3ForCausalLM": "mla", "DeepseekV2ForCausalLM": "mla"}.get(arch)
    if fam is None:
        raise KeyError(f"{f}: architecture {arch!r} has no decoder family here (known: Qwen3, Qwen3-MoE, Qwen3-Next/3.5, Llama, DeepSeek-V3)")
    h, L, Hq = c["hidden_size"], c["num_hidden_layers"], c["num_attention_heads"]
    kw = dict(name=os.path.basename(os.path.dirname(os.path.abspath(f))) or arch, architecture=arch, vocab_size=c["vocab_size"],
              hidden_size=h, num_layers=L, num_q_heads=Hq, num_kv_heads=c.get("num_key_value_heads", Hq),
              head_dim=c.get("head_dim") or h // Hq, ffn_size=c.get("intermediate_size", 0), rope_theta=float(c.get("rope_theta", 1e4)), rope_scaling=c.get("rope_scaling") or (),
              rms_eps=float(c.get("rms_norm_eps", 1e-6)), tie_embeddings=bool(c.get("tie_word_embeddings", False)),
              qk_norm=arch.startswith("Qwen3"), max_position=int(c.get("max_position_embeddings", 8192)),
              dtype={"float32": "float32"}.get(str(c.get("torch_dtype", "bfloat16")), "bfloat16"))
    if fam in ("moe", "hybrid", "mla") and (c.get("num_experts") or c.get("n_routed_experts")):
        kw.update(num_experts=c.get("num_experts") or c["n_routed_experts"], top_k=c["num_experts_per_tok"],
                  moe_ffn_size=c["moe_intermediate_size"], norm_topk_prob=bool(c.get("norm_topk_prob", True)), ffn_size=0)
        if c.get("shared_expert_intermediate_size"):
            kw.update(shared_expert_ffn=c["shared_expert_intermediate_size"], shared_expert_gate=True)
    if fam == "hybrid":
        types = c.get("layer_types")
        if types:
            types = tuple("gdn" if t in ("linear_attention", "gdn") else "attn" for t in types)
        else:
            every = int(c.get("full_attention_interval", 4))
            types = tuple("attn" if (i % every) == every - 1 else "gdn" for i in range(L))
        kw.update(layer_types=types, gdn_k_heads=c["linear_num_key_heads"], gdn_v_heads=c["linear_num_value_heads"],
                  gdn_head_dim=c.get("linear_key_head_dim", 128), gdn_conv_kernel=c.get("linear_conv_kernel_dim", 4),
                  attn_output_gate=True, zero_centered_norm=True, partial_rotary_factor=float(c.get("partial_rotary_factor", 1.0)))
    if fam == "mla":
        dr, dn = c["qk_rope_head_dim"], c["qk_nope_head_dim"]
        kw.update(kv_lora_rank=c["kv_lora_rank"], q_lora_rank=c.get("q_lora_rank") or 0, qk_rope_dim=dr, head_dim=dr + dn,
                  v_head_dim=c["v_head_dim"], num_kv_heads=Hq, qk_norm=False,
                  router="sigmoid_bias" if c.get("scoring_func") == "sigmoid" else "softmax")
        if c.get("n_shared_experts"):
            kw.update(shared_expert_ffn=c["moe_intermediate_size"] * c["n_shared_experts"])
    return ModelConfig(**kw)


def get_config(name: str, **overrides) -> ModelConfig:
    import os as _os

    if name not in PRESETS and (_os.path.isdir(name) or name.endswith("config.json")):
        cfg = config_from_hf(name)       # a checkpoint directory instead of a preset name
    elif name not in PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)} (or pass a directory holding a config.json)")
    else:
        cfg = PRESETS[name]
    # function flags of the environment select contract pins (core/flags.py); an explicit override wins over the flag
    import os

    env = {}
    k = os.environ.get("SKYRL_ISOEXEC_GDN_KERNEL", "")
    if k:
        if k not in ("recurrent", "cpr"):
            raise ValueError(f"SKYRL_ISOEXEC_GDN_KERNEL={k!r}: expected recurrent or cpr")
        env["gdn_snapshot"] = k == "cpr"
    for flag, field_ in (("SKYRL_ISOEXEC_PIK_LEAVES", "pik_leaves"), ("SKYRL_ISOEXEC_LOGPROB_LEAVES", "logprob_leaves")):
        v = os.environ.get(flag, "")
        if v:
            n = int(v)
            if n < 1 or n & (n - 1):
                raise ValueError(f"{flag}={v}: the number of leaves must be a power of two")
            env[field_] = n
    env.update(overrides)
    return cfg.with_(**env) if env else cfg
