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
