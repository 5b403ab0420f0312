"""Multi-head latent attention (DeepSeek-V3 family): the materialised form on the shared attention path equals the direct
formulation, and rollout / training logprobs of a full RL step agree bit for bit."""

import json

import pytest
import torch

from skyrl_isoexec_b200.models import hf_export
from skyrl_isoexec_b200.models.config import get_config
from skyrl_isoexec_b200.models.decoder import DecoderLM, ForwardCtx
from skyrl_isoexec_b200.ops import functional as F
from skyrl_isoexec_b200.train.config import SkyRLTrainConfig


def _direct_mla(m: DecoderLM, i: int, y: torch.Tensor, lens, pos):
    """Textbook MLA in fp64: separate rotated / un-rotated parts, no padding, one softmax per sequence and head."""
    cfg, p = m.cfg, f"layers.{i}.attn."
    H, D, dn, dr, dv, r = cfg.num_q_heads, cfg.head_dim, cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.v_head_dim, cfg.kv_lora_rank
    w = {k: m.p(p + k).detach().double() for k in ("q_b.weight", "kv_a.weight", "kv_a_norm.weight", "kv_b.weight", "o.weight")}
    y = y.double()

    def rms(x, g):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * g

    if cfg.q_lora_rank:
        qa = rms(y @ m.p(p + "q_a.weight").detach().double().T, m.p(p + "q_a_norm.weight").detach().double())
    else:
        qa = y
    q = (qa @ w["q_b.weight"].T).view(-1, H, D)
    kva = y @ w["kv_a.weight"].T
    c, k_rot = rms(kva[:, :r], w["kv_a_norm.weight"]), kva[:, r:]
    kvb = (c @ w["kv_b.weight"].T).view(-1, H, dn + dv)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, dr, 2, dtype=torch.float64) / dr))
    ang = pos.double()[:, None] * inv[None, :]
    cos, sin = ang.cos(), ang.sin()

    def rope(x):      # x [..., dr]: rotate-half convention
        a, b = x[..., : dr // 2], x[..., dr // 2:]
        cs, sn = (cos, sin) if x.dim() == 2 else (cos[:, None], sin[:, None])
        return torch.cat([a * cs - b * sn, b * cs + a * sn], -1)

    q_rot, q_nope = rope(q[..., :dr]), q[..., dr:]
    k_rot = rope(k_rot)
    k_nope, v = kvb[..., :dn], kvb[..., dn:]
    out = torch.empty(y.shape[0], H, dv, dtype=torch.float64)
    t0 = 0
    for n in lens:
        sl = slice(t0, t0 + n)
        s = torch.einsum("thd,shd->hts", q_nope[sl], k_nope[sl]) + torch.einsum("thd,sd->hts", q_rot[sl], k_rot[sl])
        s = s / (D ** 0.5) + torch.full((n, n), float("-inf"), dtype=torch.float64).triu(1)
        out[sl] = torch.einsum("hts,shd->thd", s.softmax(-1), v[sl])
        t0 += n
    return out.reshape(-1, H * dv) @ w["o.weight"].T


@pytest.mark.parametrize("preset", ["tiny-mla", "tiny-deepseek"])
def test_materialised_latent_attention_equals_the_direct_form(preset):
    cfg = get_config(preset)
    m = DecoderLM(cfg, seed=5)
    lens = [7, 12]
    T = sum(lens)
    pos = torch.cat([torch.arange(n) for n in lens]).int()
    y = torch.randn(T, cfg.hidden_size)
    fc = ForwardCtx(positions=pos, meta=F.AttnMeta.packed(lens, m.hq, m.hkv, "cpu"))
    with torch.no_grad():
        got = m._mla_block(0, y, fc, 0)
    ref = _direct_mla(m, 0, y, lens, pos)
    assert torch.allclose(got.double(), ref, atol=2e-5, rtol=1e-4), (got.double() - ref).abs().max()
    # gradients reach every latent-attention parameter
    m.zero_grad()
    m._mla_block(0, y, fc, 0).square().sum().backward()
    names = [n for n in m.store.order if n.startswith("layers.0.attn.")]
    assert len(names) == (7 if cfg.q_lora_rank else 5)
    assert all(m.p(n).grad is not None and m.p(n).grad.abs().sum() > 0 for n in names)


@pytest.mark.parametrize("preset", ["tiny-mla", "tiny-deepseek"])
def test_latent_attention_model_runs_a_full_rl_step_with_bitwise_rollout_logprobs(tmp_path, preset):
    from skyrl_isoexec_b200.train.entrypoints import main_base

    ov = [f"trainer.policy.model={preset}", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
          "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8",
          "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=8",
          "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.num_steps=1",
          f"trainer.ckpt_path={tmp_path}", "trainer.ckpt_interval=0", "trainer.logger=jsonl"]
    tr = main_base.BasePPOExp(SkyRLTrainConfig.from_cli_overrides(ov)).get_trainer()
    tr.build_models()
    tr.sync_weights()
    met = tr.train_step(next(iter(tr.loader)))
    assert met["policy/rollout_train_logprob_bit_mismatches"] == 0 and met["policy/grad_norm"] > 0


@pytest.mark.parametrize("preset", ["tiny-mla", "tiny-deepseek"])
def test_latent_attention_checkpoint_layout_round_trips(tmp_path, preset):
    from safetensors.torch import load_file

    cfg = get_config(preset)
    m = DecoderLM(cfg, seed=3)
    with torch.no_grad():
        for n in m.store.order:
            if n.endswith("expert_bias"):
                m.p(n).normal_()
    d = str(tmp_path / preset)
    hf_export.save_hf(m, d)
    sd = load_file(d + "/model.safetensors")
    H, D, dn, dr, dv, r = cfg.num_q_heads, cfg.head_dim, cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.v_head_dim, cfg.kv_lora_rank
    qname = "model.layers.0.self_attn." + ("q_b_proj" if cfg.q_lora_rank else "q_proj") + ".weight"
    assert sd[qname].shape[0] == H * D and sd["model.layers.0.self_attn.kv_a_proj_with_mqa.weight"].shape == (r + dr, cfg.hidden_size)
    assert sd["model.layers.0.self_attn.kv_b_proj.weight"].shape == (H * (dn + dv), r)
    assert sd["model.layers.0.self_attn.o_proj.weight"].shape == (cfg.hidden_size, H * dv)
    # head 1 of the export: un-rotated rows first, then the rotated rows as adjacent pairs (j, j + dr/2 of the storage here)
    ours = m.p("layers.0.attn.q_b.weight").detach().view(H, D, -1)[1]
    exp = sd[qname].view(H, D, -1)[1]
    assert torch.equal(exp[:dn], ours[dr:]) and torch.equal(exp[dn], ours[0]) and torch.equal(exp[dn + 1], ours[dr // 2])
    assert torch.equal(exp[dn + 2], ours[1])
    if cfg.has_moe:
        assert "model.layers.0.mlp.gate.e_score_correction_bias" in sd and "model.layers.0.mlp.shared_experts.down_proj.weight" in sd
    m2 = DecoderLM(cfg, seed=99)
    assert hf_export.load_hf(m2, d) == len(m.store.order) and torch.equal(m2.store.flat, m.store.flat)
    c = json.load(open(d + "/config.json"))
    assert c["architectures"] == ["DeepseekV3ForCausalLM"] and c["kv_lora_rank"] == r and c["qk_rope_head_dim"] == dr


def test_gemm_census_matches_the_manifest_model_and_the_parameter_inventory():
    """The census of the 35B-A3B hybrid reproduces the reference manifest's widths (ISO/models/qwen3_5.py:120-155), and
    for every preset each column / row / replicated site agrees with the shape of the parameter that serves it."""
    from skyrl_isoexec_b200.models.census import census_table, gemm_census
    from skyrl_isoexec_b200.models.config import PRESETS
    from skyrl_isoexec_b200.models.decoder import build_param_specs
    from skyrl_isoexec_b200.parallel.state import ParallelState

    cfg = get_config("qwen3.5-35b-a3b")
    by = {s.name: s for s in gemm_census(cfg, tp=1)}
    assert (by["gdn.in_proj"].k, by["gdn.in_proj"].n, by["gdn.in_proj"].calls) == (2048, 12352, 30)
    assert (by["attn.qkv"].n, by["attn.qkv"].calls) == (9216, 10)
    assert (by["moe.router"].n, by["moe.router"].out_dtype, by["moe.router"].calls) == (256, "fp32", 40)
    assert by["moe.shared.gate"].n == 1 and by["moe.shared.fc1"].n == 1024 and by["lm_head"].n == 248320
    by2 = {s.name: s for s in gemm_census(cfg, tp=2, ep=8)}
    assert by2["gdn.in_proj"].n == 6176 and by2["attn.qkv"].n == 4608 and by2["lm_head"].n == 124160
    assert by2["moe.router"].n == 256 and by2["moe.experts.fc1"].count == 32 and by2["attn.o"].k == 16 * 256 // 2
    assert "moe.experts.fc2" in census_table(cfg, 2, 8)
    names = {"attn.qkv": "attn.qkv.weight", "attn.o": "attn.o.weight", "gdn.in_proj": "gdn.in_proj.weight",
             "gdn.out_proj": "gdn.out_proj.weight", "moe.router": "moe.router.weight", "moe.shared.gate": "moe.shared.gate.weight",
             "moe.shared.fc1": "moe.shared.gate_up.weight", "moe.shared.fc2": "moe.shared.down.weight", "mlp.fc1": "mlp.gate_up.weight",
             "mlp.fc2": "mlp.down.weight", "attn.q_a": "attn.q_a.weight", "attn.q_b": "attn.q_b.weight", "attn.kv_a": "attn.kv_a.weight",
             "attn.kv_b": "attn.kv_b.weight"}
    for preset, c in PRESETS.items():
        if c.vocab_size > 4096:
            continue                                   # the tiny presets cover every family; skip building big inventories
        specs = {s.name: s for s in build_param_specs(c, ParallelState.single())}
        for site in gemm_census(c):
            if site.grouped or site.name == "lm_head":
                continue
            layer = next(i for i in range(c.num_layers) if f"layers.{i}.{names[site.name]}" in specs)
            assert specs[f"layers.{layer}.{names[site.name]}"].shape == (site.n, site.k), (preset, site)


def test_gated_shared_expert_hybrid_moe_runs_a_full_rl_step_with_bitwise_rollout_logprobs(tmp_path):
    from skyrl_isoexec_b200.train.entrypoints import main_base

    cfg = get_config("tiny-hybrid-moe")
    m = DecoderLM(cfg, seed=1)
    assert m.p("layers.0.moe.shared.gate.weight").shape == (1, cfg.hidden_size)
    ov = ["trainer.policy.model=tiny-hybrid-moe", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
          "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8",
          "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=8",
          "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.num_steps=1",
          f"trainer.ckpt_path={tmp_path}", "trainer.ckpt_interval=0", "trainer.logger=jsonl"]
    tr = main_base.BasePPOExp(SkyRLTrainConfig.from_cli_overrides(ov)).get_trainer()
    tr.build_models()
    tr.sync_weights()
    met = tr.train_step(next(iter(tr.loader)))
    assert met["policy/rollout_train_logprob_bit_mismatches"] == 0 and met["policy/grad_norm"] > 0
    g = tr.policy.model.p("layers.0.moe.shared.gate.weight")
    d = str(tmp_path / "hf")
    hf_export.save_hf(tr.policy.model, d)
    from safetensors.torch import load_file

    assert torch.equal(load_file(d + "/model.safetensors")["model.layers.0.mlp.shared_expert_gate.weight"], g.detach())
    m2 = DecoderLM(cfg, seed=9)
    hf_export.load_hf(m2, d)
    assert torch.equal(m2.store.flat, tr.policy.model.store.flat)
