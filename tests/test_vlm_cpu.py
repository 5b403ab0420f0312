"""Vision-language policies on CPU: the vision tower, image splicing in the engine and in the trainer (same bits), the
renderer, the batch container's per-sample tensor lists, the multi-turn generator over an environment with image
observations, and a full RL step."""
import asyncio
import base64
import io
import pickle

import pytest
import torch

from skyrl_isoexec_b200.engine.interface import NativeInferenceEngine
from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
from skyrl_isoexec_b200.engine.renderer import decode_features, encode_features, render_conversation
from skyrl_isoexec_b200.engine.sampler import SamplingParams
from skyrl_isoexec_b200.models.config import get_config
from skyrl_isoexec_b200.models.decoder import DecoderLM
from skyrl_isoexec_b200.models.vision import patchify
from skyrl_isoexec_b200.train.batch import TensorList, TrainingInputBatch, build_sequences, pad_training_input_batch
from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

CFG = get_config("tiny-vl")


class CharTokenizer:
    """One character per token id, both ways, over the whole vocabulary of the tiny model: ids below 256 are the Latin-1
    characters, the others sit in a block of their own. What the model generates therefore decodes and encodes back to
    itself, which a prefix-stable multi-turn render needs."""

    BASE = 0x4E00
    IM_START, IM_END, EOS = 2000, 2001, 2002
    eos_token_id = EOS

    def encode(self, text, add_special_tokens=False):
        return [ord(c) if ord(c) < 256 else ord(c) - self.BASE for c in text]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(i) if i < 256 else chr(self.BASE + i) for i in ids)

    def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=True):
        ids = []
        for m in messages:
            ids += [self.IM_START] + self.encode(f"{m['role']}\n{m['content']}") + [self.IM_END] + self.encode("\n")
        if add_generation_prompt:
            ids += [self.IM_START] + self.encode("assistant\n")
        return ids if tokenize else self.decode(ids)


def test_patch_order_matches_the_towers_position_table_and_features_do_not_depend_on_company():
    m = DecoderLM(CFG, seed=0)
    p, mg = CFG.vision_patch, CFG.vision_merge
    h, w = 4, 6
    # every patch is filled with a code of its (row, column): the patch list must come out in the order the tower assumes
    img = torch.zeros(3, h * p, w * p)
    for r in range(h):
        for c in range(w):
            img[:, r * p:(r + 1) * p, c * p:(c + 1) * p] = (r * 10 + c) / 100.0
    pv, grid = patchify(img, p, mg, mean=(0, 0, 0), std=(1, 1, 1))
    assert grid.tolist() == [[1, h, w]] and pv.shape == (h * w, 3 * p * p)
    rr, cc = m.vision._positions(h, w)
    assert torch.allclose(pv[:, 0] * 100.0, (rr * 10 + cc).float(), atol=1e-4)
    # four consecutive patches form one 2 x 2 neighbourhood
    assert {(int(r), int(c)) for r, c in zip(rr[:4], cc[:4])} == {(0, 0), (0, 1), (1, 0), (1, 1)}
    a = torch.rand(3, 32, 48, generator=torch.Generator().manual_seed(1))
    b = torch.rand(3, 48, 32, generator=torch.Generator().manual_seed(2))
    (pa, ga), (pb, gb) = patchify(a, p, mg), patchify(b, p, mg)
    fa = m.vision.encode(pa, ga)
    both = m.vision.encode(torch.cat([pb, pa]), torch.cat([gb, ga]))
    assert fa.shape == (m.vision.num_image_tokens(ga[0]), CFG.hidden_size) and torch.equal(both[-fa.shape[0]:], fa)
    assert torch.equal(DecoderLM(CFG, seed=0).vision.encode(pa, ga), fa)            # weights come from the seed alone
    with pytest.raises(ValueError, match="do not match"):
        m.vision.encode(pa[:-1], ga)
    sd = m.vision.state_dict()
    other = DecoderLM(CFG, seed=5)
    assert not torch.equal(other.vision.encode(pa, ga), fa)
    other.vision.load_state_dict(sd)
    assert torch.equal(other.vision.encode(pa, ga), fa)
    # uint8 pixels and cropping to whole neighbourhoods
    pu, gu = patchify((a * 255).to(torch.uint8)[:, :37, :50], p, mg)
    assert gu.tolist() == [[1, 4, 6]] and pu.dtype == torch.float32


def test_tensor_lists_travel_through_the_batch_container():
    tl = TensorList([torch.rand(i, 5) for i in range(4)])
    b = TrainingInputBatch({"sequences": torch.arange(12).view(4, 3), "loss_mask": torch.ones(4, 2), "pixel_values": tl})
    assert b.batch_size == 4 and [tuple(t.shape) for t in b.slice(1, 3)["pixel_values"]] == [(1, 5), (2, 5)]
    assert [tuple(t.shape) for t in b.select([3, 0])["pixel_values"]] == [(3, 5), (0, 5)]
    assert TrainingInputBatch.cat(b.chunk(2))["pixel_values"] == tl
    assert pickle.loads(pickle.dumps(b))["pixel_values"] == tl and b.to("cpu")["pixel_values"] == tl
    padded = pad_training_input_batch(b, 3)
    assert len(padded["pixel_values"]) == 6 and padded["pixel_values"][5].shape == (0, 5) and float(padded["loss_mask"][4:].sum()) == 0
    with pytest.raises(ValueError):
        TrainingInputBatch({"sequences": torch.zeros(3, 2), "pixel_values": tl})


def _image_request(model, g, h, w, n_before=20, n_after=15):
    pv, grid = patchify(torch.rand(3, h, w, generator=g), CFG.vision_patch, CFG.vision_merge)
    n = model.vision.num_image_tokens(grid[0])
    ids = torch.randint(5, 500, (n_before,), generator=g).tolist() + [CFG.image_token_id] * n + torch.randint(5, 500, (n_after,), generator=g).tolist()
    return ids, {"pixel_values": pv, "image_grid_thw": grid}


def test_rollout_logprobs_with_images_are_the_trainers_bits_and_the_images_matter():
    m = DecoderLM(CFG, seed=0)
    eng = LLMEngine(m, EngineConfig(max_num_seqs=4, num_kv_pages=16, seed=1, max_num_batched_tokens=50))   # images span prefill chunks
    g = torch.Generator().manual_seed(0)
    reqs = [_image_request(m, g, 32, 64), _image_request(m, g, 48, 48), (torch.randint(5, 500, (30,), generator=g).tolist(), None)]
    sp = SamplingParams(max_generate_length=10, ignore_eos=True)
    outs = eng.generate([r[0] for r in reqs], sp, mm=[r[1] for r in reqs])
    w = PolicyWorker(m, WorkerConfig(max_tokens_per_microbatch=100))
    seq, att, rmask = build_sequences([o.prompt_ids for o in outs], [o.response_ids for o in outs])
    dim = 3 * CFG.vision_patch ** 2
    fields = {"sequences": seq, "attention_mask": att, "response_mask": rmask,
              "pixel_values": TensorList([r[1]["pixel_values"] if r[1] else torch.zeros(0, dim) for r in reqs]),
              "image_grid_thw": TensorList([r[1]["image_grid_thw"] if r[1] else torch.zeros(0, 3, dtype=torch.int64) for r in reqs])}
    ro = torch.tensor([o.response_logprobs for o in outs])
    lp = w.forward(TrainingInputBatch(fields))
    assert torch.equal(lp.view(torch.int32), ro.view(torch.int32))
    # explicit positions give the same rows
    pos = [torch.tensor([i for i, t in enumerate(r[0]) if t == CFG.image_token_id], dtype=torch.int64) for r in reqs]
    lp_pos = w.forward(TrainingInputBatch(dict(fields, mm_positions=TensorList(pos))))
    assert torch.equal(lp_pos, lp)
    # without the images the image prompts score differently, the text prompt the same
    lp_text = w.forward(TrainingInputBatch({k: v for k, v in fields.items() if k in ("sequences", "attention_mask", "response_mask")}))
    assert not torch.equal(lp_text[0], lp[0]) and not torch.equal(lp_text[1], lp[1]) and torch.equal(lp_text[2], lp[2])
    # another image, other logprobs for the same tokens
    other = dict(fields, pixel_values=TensorList([fields["pixel_values"][0] * 0.5, fields["pixel_values"][1], fields["pixel_values"][2]]))
    lp_other = w.forward(TrainingInputBatch(other))
    assert not torch.equal(lp_other[0], lp[0]) and torch.equal(lp_other[1], lp[1])
    # a batch whose image rows do not fit its placeholder tokens is refused
    bad = dict(fields, pixel_values=TensorList([fields["pixel_values"][1], fields["pixel_values"][1], fields["pixel_values"][2]]),
               image_grid_thw=TensorList([fields["image_grid_thw"][1], fields["image_grid_thw"][1], fields["image_grid_thw"][2]]))
    with pytest.raises(ValueError, match="placeholder"):
        w.forward(TrainingInputBatch(bad))
    # gradients flow to the text embeddings and the decoder, not into the frozen tower
    b = TrainingInputBatch(dict(fields, loss_mask=rmask.clone(), advantages=torch.ones_like(rmask), action_log_probs=ro.clone(),
                                rollout_logprobs=ro.clone()))
    w.forward_backward(b)
    assert float(w.opt.grad_sq_norm(m.ps)) > 0
    # samples of one prompt share pages only when the images are the same
    eng2 = LLMEngine(m, EngineConfig(max_num_seqs=8, num_kv_pages=32, seed=1))
    ids, mm = _image_request(m, torch.Generator().manual_seed(3), 64, 64, n_before=120, n_after=40)       # two full pages of prompt
    mm2 = {"pixel_values": mm["pixel_values"] * 0.9, "image_grid_thw": mm["image_grid_thw"]}
    eng2.generate([ids, ids, ids], sp, mm=[mm, mm, mm2])
    assert eng2.scheduler.shared_prompt_tokens == 128
    with pytest.raises(ValueError, match="feature rows"):
        eng2.generate([ids[:-50]], sp, mm=[mm])
    with pytest.raises(ValueError, match="no vision tower"):
        LLMEngine(DecoderLM(get_config("tiny-qwen3"), seed=0), EngineConfig(num_kv_pages=8)).generate([ids], sp, mm=[mm])


def test_renderer_places_placeholders_and_round_trips_features():
    tok = CharTokenizer()
    img = (torch.rand(3, 32, 48, generator=torch.Generator().manual_seed(0)) * 255).to(torch.uint8)
    msgs = [{"role": "system", "content": "be brief"},
            {"role": "user", "content": [{"type": "text", "text": "look: "}, {"type": "image", "image": img}, {"type": "text", "text": " what?"}]}]
    r = render_conversation(msgs, tok, CFG)
    f = r["features"]
    assert f["mm_placeholders"]["image"] == [{"offset": r["token_ids"].index(CFG.image_token_id), "length": 6}]
    assert f["positions"] == [i for i, t in enumerate(r["token_ids"]) if t == CFG.image_token_id] and len(f["positions"]) == 6
    assert f["pixel_values"].shape == (24, 192) and f["image_grid_thw"].tolist() == [[1, 4, 6]]
    plain = tok.apply_chat_template([msgs[0], {"role": "user", "content": "look:  what?"}])
    assert [t for t in r["token_ids"] if t != CFG.image_token_id] == plain
    # text-only conversations come back without features; a model without a tower refuses images
    assert render_conversation([{"role": "user", "content": "hi"}], tok, CFG) == {"token_ids": tok.apply_chat_template([{"role": "user", "content": "hi"}]), "features": None}
    with pytest.raises(ValueError, match="no vision tower"):
        render_conversation(msgs, tok, get_config("tiny-qwen3"))
    # the same picture as PNG bytes in a data URL, as numpy and as PIL
    from PIL import Image

    pil = Image.fromarray(img.permute(1, 2, 0).numpy())
    buf = io.BytesIO()
    pil.save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    for part in ({"type": "image_url", "image_url": {"url": url}}, {"type": "image", "image": pil},
                 {"type": "image", "image": img.permute(1, 2, 0).numpy()}, {"type": "image", "image": buf.getvalue()}):
        r2 = render_conversation([msgs[0], {"role": "user", "content": [{"type": "text", "text": "look: "}, part, {"type": "text", "text": " what?"}]}], tok, CFG)
        assert r2["token_ids"] == r["token_ids"] and torch.equal(r2["features"]["pixel_values"], f["pixel_values"])
    with pytest.raises(ValueError, match="data: URLs"):
        render_conversation([{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "http://x/y.png"}}]}], tok, CFG)
    # the JSON-safe form
    back = decode_features(encode_features(f))
    assert torch.equal(back["pixel_values"], f["pixel_values"]) and torch.equal(back["image_grid_thw"], f["image_grid_thw"])
    assert back["positions"] == f["positions"] and decode_features(f) is f and encode_features(None) is None
    # an added turn extends the earlier render
    later = render_conversation(msgs + [{"role": "assistant", "content": "a cat"}, {"role": "user", "content": [{"type": "image", "image": img}]}], tok, CFG)
    assert later["token_ids"][:len(r["token_ids"])] == r["token_ids"] and len(later["features"]["positions"]) == 12


def _generator(max_turns=3, seed=0):
    from skyrl_isoexec_b200.train.vlm_generator import SkyRLVLMGymGenerator

    m = DecoderLM(CFG, seed=seed)
    eng = LLMEngine(m, EngineConfig(max_num_seqs=8, num_kv_pages=48, seed=2))
    tok = CharTokenizer()
    return m, SkyRLVLMGymGenerator(NativeInferenceEngine(eng, tok), tok, max_turns=max_turns)


def test_vlm_generator_runs_image_turns_and_the_trainer_scores_them_bit_for_bit():
    m, gen = _generator()
    inp = {"prompts": [[{"role": "user", "content": "count"}], [{"role": "user", "content": "count"}], [{"role": "user", "content": "just say hi"}]],
           "env_classes": ["visual_count", "visual_count", "multiply"],
           "env_extras": [{"count": 3, "seed": 1}, {"count": 5, "seed": 2}, {"reward_spec": {"ground_truth": "6"}}],
           "sampling_params": {"max_generate_length": 8, "ignore_eos": True}, "trajectory_ids": ["a", "b", "c"]}
    go = asyncio.run(gen.generate(inp))
    n_img_tok = m.vision.num_image_tokens((1, 8, 8))
    for i in range(2):                                   # three turns, three images (the random policy never answers right)
        assert len(go["mm_positions"][i]) == 3 * n_img_tok and go["image_grid_thw"][i].tolist() == [[1, 8, 8]] * 3
        assert go["pixel_values"][i].shape == (3 * 64, 192)
        full = go["prompt_token_ids"][i] + go["response_ids"][i]
        assert all(full[p] == CFG.image_token_id for p in go["mm_positions"][i].tolist())
        assert sum(go["loss_masks"][i]) == 24 and len(go["rewards"][i]) == len(go["response_ids"][i])
        zeros = [lp for lp, mk in zip(go["rollout_logprobs"][i], go["loss_masks"][i]) if not mk]
        assert zeros and all(z == 0.0 for z in zeros)
    assert go["pixel_values"][2].shape == (0, 192) and go["mm_positions"][2].numel() == 0       # a text-only trajectory beside them
    assert go["rollout_metrics"] is not None and go["env_metrics"][0]["turns"] == 3
    # through the trainer's conversion and the scoring forward: generated tokens score to the engine's bits
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    tr = RayPPOTrainer.__new__(RayPPOTrainer)
    batch = RayPPOTrainer.convert_to_training_input(tr, go, ["a", "b", "c"])
    assert isinstance(batch["pixel_values"], TensorList) and isinstance(batch["mm_positions"], TensorList)
    lp = PolicyWorker(m, WorkerConfig(max_tokens_per_microbatch=512)).forward(batch)
    sel = batch["loss_mask"] > 0
    assert torch.equal(lp[sel].view(torch.int32), batch["rollout_logprobs"][sel].view(torch.int32))
    assert SkyRLTrainConfig is not None


def test_vlm_generator_refuses_batched_and_step_wise_and_a_template_that_rewrites_history():
    from skyrl_isoexec_b200.train.vlm_generator import SkyRLVLMGymGenerator

    with pytest.raises(ValueError, match="batched"):
        SkyRLVLMGymGenerator(None, None, batched=True)
    with pytest.raises(ValueError, match="step-wise"):
        SkyRLVLMGymGenerator(None, None, step_wise=True)
    m, gen = _generator()

    class Forgetful(CharTokenizer):                      # drops the first half of earlier assistant turns, like a template that strips reasoning
        def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=True):
            msgs = [dict(x, content=x["content"][len(x["content"]) // 2:]) if x["role"] == "assistant" else x for x in messages]
            return super().apply_chat_template(msgs, add_generation_prompt, tokenize)

    gen.engine.tokenizer = gen.tokenizer = Forgetful()
    inp = {"prompts": [[{"role": "user", "content": "count"}]], "env_classes": ["visual_count"], "env_extras": [{"count": 2, "seed": 0}],
           "sampling_params": {"max_generate_length": 6, "ignore_eos": True}}
    with pytest.raises(RuntimeError, match="prefix-stable"):
        asyncio.run(gen.generate(inp))


def test_validate_cfg_for_multimodal_runs():
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig, validate_cfg

    base = ["trainer.policy.model=tiny-vl", "generator.multimodal=true", "generator.max_turns=2"]
    with pytest.raises(ValueError, match="batched=false"):
        validate_cfg(SkyRLTrainConfig.from_cli_overrides(base))
    validate_cfg(SkyRLTrainConfig.from_cli_overrides(base + ["generator.batched=false"]))


class _Rows:
    def __init__(self, n):
        self.rows = [{"prompt": [{"role": "user", "content": "count"}], "env_class": "visual_count",
                      "env_extras": {"count": 1 + i % 4, "seed": 10 + i}, "uid": f"v{i}"} for i in range(n)]

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]


def test_full_rl_steps_on_image_conversations_under_the_contract(tmp_path):
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-vl", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=6",
        "generator.sampling_params.ignore_eos=true", "generator.multimodal=true", "generator.batched=false", "generator.max_turns=2",
        "trainer.max_prompt_length=256", "generator.inference_engine.num_kv_pages=48", "trainer.num_steps=2",
        "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}", "trainer.resume_mode=none",
        "trainer.policy.optimizer_config.lr=1e-3"])
    tr = RayPPOTrainer(cfg, device="cpu", dataset=_Rows(8), tokenizer=CharTokenizer())
    tr.train()
    assert tr.global_step == 2
    assert tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0
    assert "policy/grad_norm" in tr.all_metrics          # (a random policy never counts right: rewards, hence advantages, are zero)
    assert tr.adapter_engine.ledger.verdict()["ok"] and tr.adapter_trainer.ledger.verdict()["ok"]


def test_http_server_renders_and_generates_with_images_like_the_in_process_engine():
    from PIL import Image

    from skyrl_isoexec_b200.engine.server import InferenceServer, RemoteInferenceClient

    tok = CharTokenizer()
    img = (torch.rand(3, 32, 32, generator=torch.Generator().manual_seed(4)) * 255).to(torch.uint8)
    buf = io.BytesIO()
    Image.fromarray(img.permute(1, 2, 0).numpy()).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    msgs = [{"role": "user", "content": [{"type": "text", "text": "what is this? "}, {"type": "image_url", "image_url": {"url": url}}]}]
    sp = {"max_generate_length": 6, "ignore_eos": True, "temperature": 0.0}
    local = NativeInferenceEngine(LLMEngine(DecoderLM(CFG, seed=0), EngineConfig(num_kv_pages=16, seed=2)), tok)
    r0 = asyncio.run(local.render_chat_completion({"json": {"messages": msgs}}))
    o0 = asyncio.run(local.generate({"prompt_token_ids": [r0["token_ids"]], "sampling_params": sp, "mm_features": [r0["features"]]}))
    srv = InferenceServer(LLMEngine(DecoderLM(CFG, seed=0), EngineConfig(num_kv_pages=16, seed=2)), tok).start()
    try:
        client = RemoteInferenceClient([srv.url])
        r1 = asyncio.run(client.render_chat_completion({"json": {"messages": msgs}}))
        assert r1["token_ids"] == r0["token_ids"] and torch.equal(r1["features"]["pixel_values"], r0["features"]["pixel_values"])
        o1 = asyncio.run(client.generate({"prompt_token_ids": [r1["token_ids"]], "sampling_params": sp, "mm_features": [r1["features"]]}))
        assert o1["response_ids"] == o0["response_ids"] and o1["response_logprobs"] == o0["response_logprobs"]
        # without the image features the same ids answer differently
        o2 = asyncio.run(client.generate({"prompt_token_ids": [r1["token_ids"]], "sampling_params": sp}))
        assert o2["response_logprobs"] != o1["response_logprobs"]
    finally:
        srv.shutdown()


def test_tinker_backend_takes_image_chunks_for_sampling_and_training():
    from PIL import Image

    from skyrl_isoexec_b200.tinker.backend import SkyRLTrainBackend

    img = (torch.rand(3, 32, 48, generator=torch.Generator().manual_seed(7)) * 255).to(torch.uint8)
    buf = io.BytesIO()
    Image.fromarray(img.permute(1, 2, 0).numpy()).save(buf, format="PNG")
    chunks = [{"type": "encoded_text", "tokens": list(range(10, 30))},
              {"type": "image", "data": base64.b64encode(buf.getvalue()).decode(), "format": "png", "expected_tokens": 6},
              {"type": "encoded_text", "tokens": list(range(40, 50))}]
    be = SkyRLTrainBackend("tiny-vl", device="cpu")
    s = be.handle({"type": "sample", "chunks": chunks, "num_samples": 2, "sampling_params": {"max_generate_length": 5, "ignore_eos": True}})
    assert len(s["sequences"]) == 2
    data = [{"chunks": chunks, "response_ids": q["tokens"], "logprobs": q["logprobs"]} for q in s["sequences"]]
    lp = be.handle({"type": "forward", "data": data})["logprobs"]
    for got, q in zip(lp, s["sequences"]):               # the trainer's forward sees the same image rows as the sampler did
        assert torch.equal(torch.tensor(got).view(torch.int32), torch.tensor(q["logprobs"]).view(torch.int32))
    out = be.handle({"type": "forward_backward", "data": [dict(d, advantages=1.0) for d in data], "loss_fn": "importance_sampling"})
    assert out["num_tokens"] == 10
    with pytest.raises(ValueError, match="expected_tokens"):
        be.handle({"type": "sample", "chunks": [dict(chunks[1], expected_tokens=7)], "num_samples": 1})
    with pytest.raises(ValueError, match="no vision tower"):
        SkyRLTrainBackend("tiny-qwen3", device="cpu").handle({"type": "sample", "chunks": chunks, "num_samples": 1})


def test_hf_export_carries_the_vision_tower(tmp_path):
    from skyrl_isoexec_b200.models import hf_export

    a, b = DecoderLM(CFG, seed=0), DecoderLM(CFG, seed=7)
    pv, grid = patchify(torch.rand(3, 32, 32, generator=torch.Generator().manual_seed(0)), CFG.vision_patch, CFG.vision_merge)
    assert not torch.equal(a.vision.encode(pv, grid), b.vision.encode(pv, grid))
    hf_export.save_hf(a, str(tmp_path / "m"))
    hf_export.load_hf(b, str(tmp_path / "m"))
    assert torch.equal(a.vision.encode(pv, grid), b.vision.encode(pv, grid)) and torch.equal(a.store.flat, b.store.flat)
