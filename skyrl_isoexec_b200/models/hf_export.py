"""Export to / import from the Hugging Face checkpoint layout (``config.json`` + ``model.safetensors``), the
format ``trainer.export_path`` / ``hf_save_interval`` write (reference: B/workers/.../save_hf_model paths and the
Megatron<->HF bridges in B/workers/megatron/model_bridges.py).

Latent-attention (DeepSeek-style) models export ``q_a_proj / q_b_proj / kv_a_proj_with_mqa / kv_b_proj`` with the rotated
dims re-interleaved and moved behind the un-rotated ones, the order those checkpoints use.

Internally QKV and gate/up are fused and QKV rows are stored KV-group major; the export un-fuses them into
``q_proj / k_proj / v_proj`` and ``gate_proj / up_proj`` with the usual Qwen3 names, and the import does the reverse.
Tensor-parallel models are gathered on the way out (``sync.strategies.gather_full``); the import slices full tensors
to the local shard.
"""

from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from .config import ModelConfig
from .decoder import DecoderLM


def _split_qkv(w: torch.Tensor, cfg: ModelConfig):
    """[G-major fused rows, h] -> (q [Hq*D, h], k [Hkv*D, h], v [Hkv*D, h]) in head order."""
    Hq, Hkv, D = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
    G = Hq // Hkv
    qs = 2 * D if cfg.attn_output_gate else D
    grp = w.view(Hkv, G * qs + 2 * D, -1)
    q = grp[:, :G * qs].reshape(Hkv * G, qs, -1)
    k = grp[:, G * qs:G * qs + D].reshape(Hkv * D, -1)
    v = grp[:, G * qs + D:].reshape(Hkv * D, -1)
    return q.reshape(Hq * qs, -1), k, v


def _fuse_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: ModelConfig) -> torch.Tensor:
    Hq, Hkv, D = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
    G = Hq // Hkv
    qs = 2 * D if cfg.attn_output_gate else D
    h = q.shape[-1]
    return torch.cat([q.view(Hkv, G * qs, h), k.view(Hkv, D, h), v.view(Hkv, D, h)], 1).reshape(-1, h)


def _rope_perm(dr: int, to_hf: bool) -> torch.Tensor:
    """Row permutation between the rotate-half order of the rotated dims kept here ([first halves | second halves]) and the
    interleaved (pair-adjacent) order of DeepSeek checkpoints."""
    half = torch.arange(dr // 2)
    to = torch.stack([half, half + dr // 2], 1).reshape(-1)          # hf[2j] = ours[j], hf[2j + 1] = ours[dr/2 + j]
    return to if to_hf else torch.argsort(to)


def _mla_q_rows(w: torch.Tensor, cfg: ModelConfig, to_hf: bool) -> torch.Tensor:
    """Query up-projection rows per head: [rotated | un-rotated] here, [un-rotated | rotated, interleaved] in the checkpoint."""
    H, D, dr = cfg.num_q_heads, cfg.head_dim, cfg.qk_rope_dim
    g = w.view(H, D, -1)
    if to_hf:
        return torch.cat([g[:, dr:], g[:, :dr][:, _rope_perm(dr, True)]], 1).reshape(H * D, -1)
    dn = D - dr
    return torch.cat([g[:, dn:][:, _rope_perm(dr, False)], g[:, :dn]], 1).reshape(H * D, -1)


def _mla_kv_a_rows(w: torch.Tensor, cfg: ModelConfig, to_hf: bool) -> torch.Tensor:
    r = cfg.kv_lora_rank
    return torch.cat([w[:r], w[r:][_rope_perm(cfg.qk_rope_dim, to_hf)]], 0)


_MLA_NAMES = {"attn.q_a.weight": "self_attn.q_a_proj.weight", "attn.q_a_norm.weight": "self_attn.q_a_layernorm.weight",
              "attn.kv_a_norm.weight": "self_attn.kv_a_layernorm.weight", "attn.kv_b.weight": "self_attn.kv_b_proj.weight"}


def _shared_prefix(cfg: ModelConfig) -> str:
    return "mlp.shared_experts." if cfg.is_mla else "mlp.shared_expert."


def full_named_weights(model: DecoderLM):
    """(name, full-shape tensor) for every parameter. Under tensor / expert parallelism the sharded ones are all-gathered
    over the TP / EP group, so EVERY rank of those groups has to iterate (in lock step)."""
    from ..sync.strategies import gather_full

    ps = model.ps
    for name, t in model.named_weights():
        spec = model.store.specs[name]
        if ps.tp > 1 and spec.shard_dim is not None:
            t = gather_full(t.detach(), spec, ps)
        if ps.ep > 1 and spec.ep_sharded:                # experts of the other expert-parallel ranks, in rank order
            parts = [torch.empty_like(t) for _ in range(ps.ep)]
            dist.all_gather(parts, t.detach().contiguous(), group=ps.ep_group)
            t = torch.cat(parts, dim=0)
        yield name, t


def to_hf_state_dict(model: DecoderLM) -> dict[str, torch.Tensor]:
    """Un-fused, Hugging Face named tensors of the whole model. Tensor-parallel models are gathered (a collective over the
    TP and EP groups); pipeline-parallel models are not handled here."""
    cfg = model.cfg
    assert model.ps.pp == 1, "pipeline-parallel stages are not gathered by the exporter"
    out: dict[str, torch.Tensor] = {}
    for name, t in full_named_weights(model):
        t = t.detach().cpu().contiguous()
        if name == "embed.weight":
            out["model.embed_tokens.weight"] = t
        elif name == "lm_head.weight":
            out["lm_head.weight"] = t
        elif name == "final_norm.weight":
            out["model.norm.weight"] = t
        else:
            _, i, rest = name.split(".", 2)
            p = f"model.layers.{i}."
            if rest == "attn.qkv.weight":
                q, k, v = _split_qkv(t, cfg)
                out[p + "self_attn.q_proj.weight"], out[p + "self_attn.k_proj.weight"], out[p + "self_attn.v_proj.weight"] = \
                    q.contiguous(), k.contiguous(), v.contiguous()
            elif rest == "attn.q_b.weight":
                out[p + ("self_attn.q_b_proj.weight" if cfg.q_lora_rank else "self_attn.q_proj.weight")] = _mla_q_rows(t, cfg, True).contiguous()
            elif rest == "attn.kv_a.weight":
                out[p + "self_attn.kv_a_proj_with_mqa.weight"] = _mla_kv_a_rows(t, cfg, True).contiguous()
            elif rest == "mlp.gate_up.weight":
                f = t.shape[0] // 2
                out[p + "mlp.gate_proj.weight"], out[p + "mlp.up_proj.weight"] = t[:f].contiguous(), t[f:].contiguous()
            elif rest == "moe.shared.gate_up.weight":
                f = t.shape[0] // 2
                out[p + _shared_prefix(cfg) + "gate_proj.weight"], out[p + _shared_prefix(cfg) + "up_proj.weight"] = \
                    t[:f].contiguous(), t[f:].contiguous()
            elif rest == "moe.experts.gate_up":
                f = t.shape[1] // 2
                for e in range(t.shape[0]):
                    out[p + f"mlp.experts.{e}.gate_proj.weight"] = t[e, :f].contiguous()
                    out[p + f"mlp.experts.{e}.up_proj.weight"] = t[e, f:].contiguous()
            elif rest == "moe.experts.down":
                for e in range(t.shape[0]):
                    out[p + f"mlp.experts.{e}.down_proj.weight"] = t[e].contiguous()
            else:
                ren = {"ln1.weight": "input_layernorm.weight", "ln2.weight": "post_attention_layernorm.weight",
                       "attn.o.weight": "self_attn.o_proj.weight", "attn.q_norm.weight": "self_attn.q_norm.weight",
                       "attn.k_norm.weight": "self_attn.k_norm.weight", "mlp.down.weight": "mlp.down_proj.weight",
                       "moe.router.weight": "mlp.gate.weight", "moe.router.expert_bias": "mlp.gate.e_score_correction_bias",
                       "moe.shared.down.weight": _shared_prefix(cfg) + "down_proj.weight",
                       "moe.shared.gate.weight": "mlp.shared_expert_gate.weight", **_MLA_NAMES}
                out[p + ren.get(rest, rest)] = t
    return out


def hf_config(cfg: ModelConfig) -> dict:
    arch = "Qwen3MoeForCausalLM" if cfg.has_moe else ("Qwen3NextForCausalLM" if cfg.has_gdn else "Qwen3ForCausalLM")
    if not (cfg.has_moe or cfg.has_gdn or cfg.qk_norm):
        arch = "LlamaForCausalLM"       # dense, no QK-norm: the Llama checkpoint layout (same tensor names minus q_norm / k_norm)
    d = {"architectures": [arch], "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
         "num_attention_heads": cfg.num_q_heads, "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
         "intermediate_size": cfg.ffn_size, "vocab_size": cfg.vocab_size, "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_eps,
         "tie_word_embeddings": cfg.tie_embeddings, "max_position_embeddings": cfg.max_position, "torch_dtype": cfg.dtype,
         "hidden_act": "silu"}
    if cfg.is_mla:
        d["architectures"] = ["DeepseekV3ForCausalLM"]
        d.update({"kv_lora_rank": cfg.kv_lora_rank, "q_lora_rank": cfg.q_lora_rank or None, "qk_rope_head_dim": cfg.qk_rope_dim,
                  "qk_nope_head_dim": cfg.qk_nope_dim, "v_head_dim": cfg.v_head_dim})
        if cfg.has_moe:
            d.update({"n_routed_experts": cfg.num_experts, "n_shared_experts": 1 if cfg.shared_expert_ffn else 0,
                      "scoring_func": "sigmoid" if cfg.router == "sigmoid_bias" else "softmax"})
    if cfg.has_moe:
        d.update({"num_experts": cfg.num_experts, "num_experts_per_tok": cfg.top_k, "moe_intermediate_size": cfg.moe_ffn_size,
                  "norm_topk_prob": cfg.norm_topk_prob})
        if cfg.shared_expert_ffn and not cfg.is_mla:
            d["shared_expert_intermediate_size"] = cfg.shared_expert_ffn
    if cfg.has_gdn:
        d.update({"layer_types": ["linear_attention" if t == "gdn" else "full_attention" for t in cfg.layer_types],
                  "linear_num_key_heads": cfg.gdn_k_heads, "linear_num_value_heads": cfg.gdn_v_heads,
                  "linear_key_head_dim": cfg.gdn_head_dim, "linear_value_head_dim": cfg.gdn_head_dim,
                  "linear_conv_kernel_dim": cfg.gdn_conv_kernel, "partial_rotary_factor": cfg.partial_rotary_factor})
        if cfg.has_moe:
            d["architectures"] = ["Qwen3_5MoeForCausalLM"]
    if cfg.rope_scaling:
        d["rope_scaling"] = dict(cfg.rope_scaling)
    return d


def save_hf(model: DecoderLM, path: str, write: bool = True) -> None:
    """Every rank of a tensor-parallel group calls this (the gather is a collective); ``write=False`` on all but one."""
    from safetensors.torch import save_file

    sd = to_hf_state_dict(model)
    if getattr(model, "vision", None) is not None:
        sd.update({k: v.contiguous() for k, v in model.vision.state_dict().items()})     # the frozen tower, under its own ``visual.*`` names
    if not write:
        return
    from ..utils import io as uio

    with uio.local_work_dir(path) as d:                 # a remote ``path`` is written locally and uploaded on exit
        save_file(sd, os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(hf_config(model.cfg), f, indent=1)


class _LazyCheckpoint:
    """Tensors of a Hugging Face checkpoint directory, read one at a time: a single ``model.safetensors``, or the shards a
    released model comes in (``model.safetensors.index.json`` names the file of every tensor, or every ``*.safetensors`` file
    of the directory is looked through). Nothing but the tensor asked for is held, so a 64 GB checkpoint loads into a
    sharded model without a 64 GB host copy. Tied checkpoints without ``lm_head.weight`` answer it with the embedding."""

    def __init__(self, path: str):
        from safetensors import safe_open

        self._open = safe_open
        self.where: dict[str, str] = {}
        index = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as f:
                self.where = {k: os.path.join(path, v) for k, v in json.load(f)["weight_map"].items()}
        else:
            files = sorted(fn for fn in os.listdir(path) if fn.endswith(".safetensors"))
            if not files:
                raise FileNotFoundError(f"{path} holds no .safetensors file")
            for fn in files:
                with safe_open(os.path.join(path, fn), framework="pt", device="cpu") as f:
                    for k in f.keys():
                        self.where[k] = os.path.join(path, fn)
        self._handles: dict = {}

    def keys(self):
        return self.where.keys()

    def __iter__(self):
        return iter(self.where)

    def __contains__(self, k) -> bool:
        return k in self.where

    def __getitem__(self, k: str) -> torch.Tensor:
        if k not in self.where and k == "lm_head.weight" and "model.embed_tokens.weight" in self.where:
            k = "model.embed_tokens.weight"
        fn = self.where[k]
        h = self._handles.get(fn)
        if h is None:
            h = self._handles[fn] = self._open(fn, framework="pt", device="cpu").__enter__()
        return h.get_tensor(k)

    def close(self) -> None:
        for h in self._handles.values():
            h.__exit__(None, None, None)
        self._handles.clear()


def has_hf_weights(path: str) -> bool:
    return os.path.isdir(path) and any(fn.endswith(".safetensors") for fn in os.listdir(path))


def load_hf(model: DecoderLM, path: str) -> int:
    """Load a Hugging Face style checkpoint directory (one ``model.safetensors`` as ``save_hf`` writes it, or the sharded
    files of a released model) into ``model``: tensors are read one at a time and cut to this rank's shard."""
    sd = _LazyCheckpoint(path)
    try:
        return _load_from(model, sd)
    finally:
        sd.close()


def _load_from(model: DecoderLM, sd) -> int:
    if getattr(model, "vision", None) is not None and any(k.startswith("visual.") for k in sd):
        model.vision.load_state_dict({k: sd[k] for k in sd if k.startswith("visual.")})
    cfg = model.cfg
    n = 0
    with torch.no_grad():
        for name, t in model.named_weights():
            if name == "embed.weight":
                src = sd["model.embed_tokens.weight"]
            elif name == "lm_head.weight":
                src = sd["lm_head.weight"]
            elif name == "final_norm.weight":
                src = sd["model.norm.weight"]
            else:
                _, i, rest = name.split(".", 2)
                p = f"model.layers.{i}."
                if rest == "attn.qkv.weight":
                    src = _fuse_qkv(sd[p + "self_attn.q_proj.weight"], sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.v_proj.weight"], cfg)
                elif rest == "attn.q_b.weight":
                    src = _mla_q_rows(sd[p + ("self_attn.q_b_proj.weight" if cfg.q_lora_rank else "self_attn.q_proj.weight")], cfg, False)
                elif rest == "attn.kv_a.weight":
                    src = _mla_kv_a_rows(sd[p + "self_attn.kv_a_proj_with_mqa.weight"], cfg, False)
                elif rest == "mlp.gate_up.weight":
                    src = torch.cat([sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"]], 0)
                elif rest == "moe.shared.gate_up.weight":
                    src = torch.cat([sd[p + _shared_prefix(cfg) + "gate_proj.weight"], sd[p + _shared_prefix(cfg) + "up_proj.weight"]], 0)
                elif rest == "moe.experts.gate_up":
                    src = torch.stack([torch.cat([sd[p + f"mlp.experts.{e}.gate_proj.weight"], sd[p + f"mlp.experts.{e}.up_proj.weight"]], 0)
                                       for e in range(cfg.num_experts)])      # all experts; cut to this rank's below
                elif rest == "moe.experts.down":
                    src = torch.stack([sd[p + f"mlp.experts.{e}.down_proj.weight"] for e in range(cfg.num_experts)])
                else:
                    ren = {"ln1.weight": "input_layernorm.weight", "ln2.weight": "post_attention_layernorm.weight",
                           "attn.o.weight": "self_attn.o_proj.weight", "attn.q_norm.weight": "self_attn.q_norm.weight",
                           "attn.k_norm.weight": "self_attn.k_norm.weight", "mlp.down.weight": "mlp.down_proj.weight",
                           "moe.router.weight": "mlp.gate.weight", "moe.router.expert_bias": "mlp.gate.e_score_correction_bias",
                           "moe.shared.down.weight": _shared_prefix(cfg) + "down_proj.weight",
                       "moe.shared.gate.weight": "mlp.shared_expert_gate.weight", **_MLA_NAMES}
                    src = sd[p + ren.get(rest, rest)]
            spec = model.store.specs[name]
            if tuple(src.shape) != tuple(t.shape) and src.numel() != t.numel():
                from .decoder import shard_of     # a full tensor for a sharded parameter: cut this rank's part

                src = shard_of(src.view(spec.full_shape), spec, model.ps.tp_rank, model.ps.tp, model.ps.ep_rank, model.ps.ep)
            t.copy_(src.to(t.dtype).reshape(t.shape))
            n += 1
    return n
