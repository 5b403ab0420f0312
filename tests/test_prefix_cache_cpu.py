"""Prefix reuse across requests: the bits of a request do not depend on whether its leading pages came out of the cache;
pages are reference-counted, evicted under pressure and dropped at a weight sync; models with recurrent layers resume
from a boundary state kept beside the pages."""
import pytest
import torch

from skyrl_isoexec_b200.engine.kv_cache import PageAllocator
from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
from skyrl_isoexec_b200.engine.prefix_cache import BoundaryStates, PrefixCache, chain_keys
from skyrl_isoexec_b200.engine.sampler import SamplingParams
from skyrl_isoexec_b200.models.config import get_config
from skyrl_isoexec_b200.models.decoder import DecoderLM
from skyrl_isoexec_b200.ops.functional import PAGE


def _toks(n, seed):
    return torch.randint(5, 500, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_table_matches_chains_counts_references_and_evicts_leaves_first():
    al = PageAllocator(8)
    pc = PrefixCache(al)
    a = _toks(3 * PAGE + 5, 0)
    pages = al.alloc(4)
    assert pc.insert(a, pages, 3 * PAGE + 5) == 3 and al.refs[pages[0]] == 2 and al.refs[pages[3]] == 1
    assert pc.insert(a, pages, 3 * PAGE + 5) == 0                                    # listed already
    al.release(pages)                                                                # the request ends: 3 pages stay, 1 is free
    assert al.num_free == 5 and pc.evictable() == 3
    got, key = pc.match(a[:2 * PAGE + 1])                                            # two full pages, one token left to compute
    assert got == pages[:2] and key == chain_keys(a, 2)[-1] and al.refs[pages[0]] == 2
    assert pc.match(a[:2 * PAGE])[0] == pages[:1]                                    # exactly two pages of tokens: the last is computed
    al.release(pages[:1])
    b = a[:PAGE] + _toks(PAGE + 1, 1)                                                # same first page, then different
    assert pc.match(b)[0] == pages[:1]
    al.release(pages[:1])
    assert pc.match(_toks(2 * PAGE, 2)) == ([], None)
    # a key that collides is refused by the token comparison
    forged = dict(pc.table)
    k0 = chain_keys(a, 1)[0]
    pc.table[k0] = (forged[k0][0], forged[k0][1], tuple(_toks(PAGE, 9)))
    assert pc.match(a)[0] == []
    pc.table[k0] = forged[k0]
    # eviction: only pages nobody reads, the deepest page of a chain first
    assert pc.evict(1) == 1 and chain_keys(a, 3)[2] not in pc.table and chain_keys(a, 3)[0] in pc.table
    al.release(got)
    assert pc.evict(10) == 2 and len(pc) == 0 and al.num_free == 8
    # clear gives every reference back
    pages = al.alloc(2)
    pc.insert(a, pages, 2 * PAGE)
    al.release(pages)
    pc.clear()
    assert al.num_free == 8 and all(r == 0 for r in al.refs)


def test_boundary_store_is_lru_within_a_byte_budget(capsys):
    st = lambda v: {0: (torch.full((4, 3), float(v)), torch.full((2, 8, 8), float(v)))}
    one = 4 * 3 * 4 + 2 * 8 * 8 * 4
    bs = BoundaryStates(2 * one)
    assert bs.put(b"a", st(1)) and bs.put(b"b", st(2)) and not bs.put(b"a", st(1))    # the second put of a key only touches it
    assert bs.put(b"c", st(3)) and b"b" not in bs and b"a" in bs and bs.evictions == 1
    assert float(bs.get(b"c")[0][1][0, 0, 0]) == 3.0 and bs.bytes == 2 * one
    bs.drop(b"a")
    assert bs.bytes == one
    small = BoundaryStates(one - 1)
    assert not small.put(b"x", st(1)) and not small.put(b"y", st(1)) and small.oversize == 2
    assert capsys.readouterr().out.count("no state can be stored") == 1


def _engine(preset, cached, pages=24, **kw):
    m = DecoderLM(get_config(preset), seed=0)
    return LLMEngine(m, EngineConfig(max_num_seqs=8, num_kv_pages=pages, seed=3, enable_prefix_caching=cached, max_num_batched_tokens=200, **kw))


def _same(a, b):
    return all(x.response_ids == y.response_ids and
               torch.equal(torch.tensor(x.response_logprobs).view(torch.int32), torch.tensor(y.response_logprobs).view(torch.int32))
               for x, y in zip(a, b))


@pytest.mark.parametrize("preset", ["tiny-qwen3", "tiny-hybrid"])
def test_a_later_turn_reuses_the_earlier_turns_pages_with_the_same_bits(preset):
    sp = SamplingParams(max_generate_length=40, temperature=0.0, ignore_eos=True)
    plain, cached = _engine(preset, False), _engine(preset, True)
    p1 = [_toks(2 * PAGE + 17, 0), _toks(PAGE + 60, 1)]
    r_plain, r_cached = plain.generate(p1, sp), cached.generate(p1, sp)
    assert _same(r_plain, r_cached) and cached.prefix_cache.hits == 0 and len(cached.prefix_cache) >= 3
    # second turn: the conversation so far (prompt + answer) plus an observation; and the first prompt once more
    p2 = [p1[0] + r_plain[0].response_ids + _toks(30, 5), p1[1] + r_plain[1].response_ids + _toks(9, 6), p1[0]]
    before = cached.stats["prefill_tokens"], plain.stats["prefill_tokens"]
    r_plain, r_cached = plain.generate(p2, sp), cached.generate(p2, sp)
    assert _same(r_plain, r_cached)
    pc = cached.prefix_cache
    assert pc.hits == 3 and pc.hit_tokens >= 2 * PAGE + PAGE + 2 * PAGE
    saved = (plain.stats["prefill_tokens"] - before[1]) - (cached.stats["prefill_tokens"] - before[0])
    assert saved == pc.hit_tokens
    if preset == "tiny-hybrid":
        assert pc.boundary.stores >= 3 and all(k in pc.table for k in pc.boundary.d)
    # nothing leaks: every page is free or listed by the cache, and a weight sync drops the lot and finds the cache clean
    al = cached.cache.allocator
    assert al.num_free + len(pc) == al.num_pages and pc.evictable() == len(pc)
    n0 = cached.cache.invalidations["weight_sync"]
    cached.reset_prefix_cache()
    assert len(pc) == 0 and al.num_free == al.num_pages and cached.cache.invalidations["weight_sync"] == n0 + 1
    assert pc.boundary is None or len(pc.boundary.d) == 0
    # after the drop nothing matches, and the bits are still the same
    assert _same(plain.generate(p2[:1], sp), cached.generate(p2[:1], sp)) and pc.hits == 3
    # sleep starts a fresh allocator: the cache follows it
    cached.sleep()
    cached.wake_up()
    assert pc.alloc is cached.cache.allocator and len(pc) == 0
    assert _same(plain.generate(p2[:1], sp), cached.generate(p2[:1], sp))


def test_cached_pages_go_before_a_running_sequence_is_preempted():
    sp = SamplingParams(max_generate_length=20, temperature=0.0, ignore_eos=True)
    plain, cached = _engine("tiny-qwen3", False, pages=6), _engine("tiny-qwen3", True, pages=6)
    for seed in range(4):                                   # 4 x 2 full pages would fill the pool: older prefixes are evicted
        p = [_toks(2 * PAGE + 30, 10 + seed)]
        assert _same(plain.generate(p, sp), cached.generate(p, sp))
    pc, al = cached.prefix_cache, cached.cache.allocator
    assert pc.evicted >= 2 and cached.scheduler.preemptions == 0 and al.num_free + len(pc) == al.num_pages
    # the most recent prompt is still there
    assert _same(plain.generate(p, sp), cached.generate(p, sp)) and pc.hits == 1


def test_samples_of_a_prompt_seen_before_on_a_hybrid_model_start_from_the_cached_boundary():
    sp = SamplingParams(max_generate_length=12, temperature=0.0, ignore_eos=True)
    plain = _engine("tiny-hybrid", False)
    cached = _engine("tiny-hybrid", True, share_recurrent_state=True)
    p = _toks(2 * PAGE + 9, 21)
    assert _same(plain.generate([p], sp), cached.generate([p], sp))
    # now three samples of the same prompt: the leader matches the cache up to the very boundary its siblings wait for
    r_plain, r_cached = plain.generate([p, p, p], sp), cached.generate([p, p, p], sp)
    assert _same(r_plain, r_cached) and cached.prefix_cache.hits == 1 and cached.scheduler.shared_prompt_tokens == 2 * 2 * PAGE


def test_validate_cfg_lets_prefix_caching_through_under_the_contract():
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig, validate_cfg

    cfg = SkyRLTrainConfig.from_cli_overrides(["trainer.policy.model=tiny-qwen3", "generator.inference_engine.enable_prefix_caching=true"])
    assert cfg.trainer.isoexec.enabled
    validate_cfg(cfg)


def test_server_turns_of_a_conversation_hit_the_cache_and_a_weight_update_drops_it():
    import json
    import urllib.request

    from skyrl_isoexec_b200.train.entrypoints import serve

    def call(url, path, body=None):
        req = urllib.request.Request(url + path, data=None if body is None else json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"}, method="GET" if body is None else "POST")
        with urllib.request.urlopen(req, timeout=60) as r:
            raw = r.read()
            return json.loads(raw) if r.headers.get("Content-Type", "").startswith("application/json") else raw.decode()

    srv = serve.build(["--model", "tiny-qwen3", "--num-kv-pages", "16", "--device", "cpu", "--enable-prefix-caching"]).start()
    try:
        sp = {"max_generate_length": 6, "ignore_eos": True, "temperature": 0.0}
        turn1 = _toks(PAGE + 40, 3)
        out = call(srv.url, "/generate", {"prompt_token_ids": [turn1], "sampling_params": sp})
        turn2 = turn1 + out["response_ids"][0] + _toks(20, 4)
        call(srv.url, "/generate", {"prompt_token_ids": [turn2], "sampling_params": sp})
        text = call(srv.url, "/metrics")
        vals = {ln.split("{")[0]: float(ln.rsplit(" ", 1)[1]) for ln in text.splitlines() if ln and not ln.startswith("#")}
        assert vals["isoexec_prefix_cache_hits_total"] == 1 and vals["isoexec_prefix_cache_hit_tokens_total"] == PAGE
        assert vals["isoexec_prefix_cache_pages"] >= 1
        call(srv.url, "/reset_prefix_cache", {})
        text = call(srv.url, "/metrics")
        assert 'isoexec_prefix_cache_pages{model="tiny-qwen3"} 0' in text
    finally:
        srv.shutdown()


def test_rl_steps_with_prefix_caching_stay_bitwise_and_the_sync_is_seen_to_empty_the_cache(tmp_path):
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=6",
        "generator.sampling_params.ignore_eos=true", f"data.synthetic_prompt_len={PAGE + 12}", "data.synthetic_prompts=8",
        f"trainer.max_prompt_length={PAGE + 12}", "generator.inference_engine.num_kv_pages=16",
        "generator.inference_engine.enable_prefix_caching=true", "trainer.num_steps=2", "trainer.logger=jsonl",
        f"trainer.ckpt_path={tmp_path}", "trainer.resume_mode=none"])
    tr = RayPPOTrainer(cfg, device="cpu")
    tr.train()
    assert tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0
    pc = tr.engine.prefix_cache
    assert pc is not None and pc.stored >= 4 and tr.engine.stats["prefix_cache_drops"] >= 2
    verdict = tr.adapter_engine.ledger.verdict()
    assert verdict["ok"], verdict


def test_random_request_streams_keep_the_page_accounting_exact():
    """Property test: whatever the order of inserts, matches, releases and evictions, every page is either free or
    referenced, reference counts equal the number of holders, and a match only ever returns pages whose tokens are the
    request's own prefix."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    @settings(max_examples=60, deadline=None)
    @given(st.lists(st.tuples(st.integers(0, 5), st.integers(1, 3), st.integers(0, PAGE - 1), st.sampled_from(["finish", "evict", "hold"])), min_size=1, max_size=25))
    def run(ops):
        al = PageAllocator(12)
        pc = PrefixCache(al)
        held: list[tuple[list[int], list[int]]] = []                       # (tokens, pages) of requests still running
        content: dict[int, tuple] = {}                                      # page -> the tokens written into it
        for family, n_pages, extra, what in ops:
            # prompts of one family share their first pages: family f, page k holds tokens f * 1000 + k
            tokens = [family * 1000 + k for k in range(n_pages) for _ in range(PAGE)] + [7] * extra + [9]
            got, _key = pc.match(tokens)
            for k, p in enumerate(got):
                assert content[p] == tuple(tokens[k * PAGE:(k + 1) * PAGE])
            need = (len(tokens) + PAGE - 1) // PAGE - len(got)
            if not al.can_alloc(need):
                pc.evict(need - al.num_free)
            if not al.can_alloc(need):
                al.release(got)
                continue
            pages = got + al.alloc(need)
            for k in range(len(got), len(pages)):
                content[pages[k]] = tuple(tokens[k * PAGE:(k + 1) * PAGE])
            if what == "hold":
                held.append((tokens, pages))
            else:
                pc.insert(tokens, pages, len(tokens))
                al.release(pages)
                if what == "evict":
                    pc.evict(2)
            # invariants
            holders = [0] * al.num_pages
            for _t, ps_ in held:
                for p in ps_:
                    holders[p] += 1
            for page, _par, _tok in pc.table.values():
                holders[page] += 1
            assert holders == al.refs
            assert sorted(al.free) == [p for p in range(al.num_pages) if al.refs[p] == 0] and len(set(al.free)) == len(al.free)
        for tokens, pages in held:
            pc.insert(tokens, pages, len(tokens))
            al.release(pages)
        pc.clear()
        assert al.num_free == al.num_pages and all(r == 0 for r in al.refs)

    run()


@pytest.mark.parametrize("preset", ["tiny-qwen3", "tiny-hybrid"])
def test_prefix_cache_under_page_pressure_and_preemption_still_gives_the_plain_engines_bits(preset):
    """A pool too small for the running batch: sequences are preempted and recomputed, cached pages are evicted and found
    again, and every answer is still the answer of an engine without a cache and with room to spare."""
    sp = SamplingParams(max_generate_length=140, temperature=0.0, ignore_eos=True)
    roomy = _engine(preset, False, pages=64)
    tight = _engine(preset, True, pages=7)
    fam = [_toks(PAGE + 5, 100 + f) for f in range(3)]
    g = torch.Generator().manual_seed(0)
    for rnd in range(4):
        prompts = []
        for _ in range(4):
            f = int(torch.randint(0, 3, (1,), generator=g))
            prompts.append(fam[f] + _toks(int(torch.randint(3, 60, (1,), generator=g)), 1000 + rnd * 10 + len(prompts)))
        assert _same(roomy.generate(prompts, sp), tight.generate(prompts, sp)), rnd
    pc, al = tight.prefix_cache, tight.cache.allocator
    assert tight.scheduler.preemptions > 0 and pc.hits > 0 and pc.evicted > 0
    assert al.num_free + len(pc) == al.num_pages and pc.evictable() == len(pc)
