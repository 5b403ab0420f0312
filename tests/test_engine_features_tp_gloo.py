"""Engine features on a tensor-parallel engine (two gloo ranks, CPU kernels): prefix reuse across requests, image inputs and
prompt logprobs give, on BOTH ranks, the bits a single-rank engine gives."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(ps, kind):
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import SamplingParams
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.models.vision import patchify
    from skyrl_isoexec_b200.ops.functional import PAGE

    g = torch.Generator().manual_seed(5)
    toks = lambda n: torch.randint(5, 500, (n,), generator=g).tolist()
    sp = SamplingParams(max_generate_length=10, temperature=0.0, ignore_eos=True)
    if kind in ("prefix", "prefix-hybrid"):
        cfg = get_config("tiny-hybrid" if kind == "prefix-hybrid" else "tiny-qwen3", tp_invariant=True)
        eng = LLMEngine(DecoderLM(cfg, ps, seed=3), EngineConfig(num_kv_pages=24, seed=1, enable_prefix_caching=True, max_num_batched_tokens=200))
        p1 = toks(2 * PAGE + 11)
        a = eng.generate([p1], sp)[0]
        b = eng.generate([p1 + a.response_ids + toks(20), p1], sp)
        return [a.response_ids, a.response_logprobs] + [x for o in b for x in (o.response_ids, o.response_logprobs)] + [eng.prefix_cache.hit_tokens]
    if kind == "images":
        cfg = get_config("tiny-vl", tp_invariant=True)
        m = DecoderLM(cfg, ps, seed=3)
        eng = LLMEngine(m, EngineConfig(num_kv_pages=16, seed=1, max_num_batched_tokens=50))
        pv, grid = patchify(torch.rand(3, 32, 64, generator=g), cfg.vision_patch, cfg.vision_merge)
        ids = toks(20) + [cfg.image_token_id] * m.vision.num_image_tokens(grid[0]) + toks(12)
        o = eng.generate([ids, toks(30)], sp, mm=[{"pixel_values": pv, "image_grid_thw": grid}, None])
        return [x for r in o for x in (r.response_ids, r.response_logprobs)]
    cfg = get_config("tiny-qwen3", tp_invariant=True)
    eng = LLMEngine(DecoderLM(cfg, ps, seed=3), EngineConfig(num_kv_pages=16, seed=1, max_num_batched_tokens=48))
    o = eng.generate([toks(100), toks(33)], SamplingParams(max_generate_length=4, temperature=0.0, ignore_eos=True, prompt_logprobs=1))
    return [x for r in o for x in (r.response_ids, r.response_logprobs, r.prompt_logprobs[1:])]


def _worker(rank, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="2")
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=2)
    try:
        from skyrl_isoexec_b200.parallel.state import ParallelState

        ps2 = ParallelState.build(tp=2)
        out = {}
        for kind in ("prefix", "prefix-hybrid", "images", "prompt_logprobs"):
            got = _run(ps2, kind)
            ref = _run(ParallelState.single(), kind) if rank == 0 else None
            out[kind] = (got, ref)
        q.put((rank, out))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


def _bits(x):
    return torch.tensor(x, dtype=torch.float32).view(torch.int32).tolist() if x and isinstance(x[0], float) else x


@pytest.mark.timeout(900)
def test_prefix_cache_images_and_prompt_logprobs_on_a_tp2_engine_match_tp1_bitwise():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for kind in res[0]:
        got0, ref = res[0][kind]
        got1, _ = res[1][kind]
        assert [_bits(x) if isinstance(x, list) else x for x in got0] == [_bits(x) if isinstance(x, list) else x for x in got1], f"{kind}: the two ranks differ"
        assert [_bits(x) if isinstance(x, list) else x for x in got0] == [_bits(x) if isinstance(x, list) else x for x in ref], f"{kind}: TP=2 differs from TP=1"
    assert res[0]["prefix"][0][-1] > 0 and res[0]["prefix-hybrid"][0][-1] > 0           # the later requests did hit the cache
