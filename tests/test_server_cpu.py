"""HTTP inference server + remote client on CPU (127.0.0.1, ephemeral ports)."""
import asyncio
import threading
import time

import pytest
import torch

from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
from skyrl_isoexec_b200.engine.server import InferenceServer, RemoteInferenceClient, ServerGroup
from skyrl_isoexec_b200.models.config import get_config
from skyrl_isoexec_b200.models.decoder import DecoderLM


def _engine(seed=0, max_position=512, pages=32):
    cfg = get_config("tiny-qwen3", max_position=max_position)
    return LLMEngine(DecoderLM(cfg, seed=seed), EngineConfig(max_num_seqs=16, num_kv_pages=pages, seed=3))


def test_server_data_and_control_plane(tmp_path):
    e1, e2 = _engine(), _engine()
    group = ServerGroup([e1, e2])
    urls = group.start()
    try:
        cl = RemoteInferenceClient(urls, max_retries=1, backoff_s=0.01, timeout_s=60)
        infos = cl.server_info()
        assert len(infos) == 2 and infos[0]["tp_size"] == 1 and cl.dp_size() == 2
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, 2048, (9,), generator=g).tolist() for _ in range(5)]
        sp = {"max_generate_length": 7, "ignore_eos": True}
        out = asyncio.run(cl.generate({"prompt_token_ids": prompts, "sampling_params": sp, "session_ids": list("abcde")}))
        assert all(len(r) == 7 for r in out["response_ids"]) and all(len(l) == 7 for l in out["response_logprobs"])
        assert sum(i["requests_served"] for i in cl.server_info()) == 5
        # Prometheus-style counters, summed over the servers
        m = cl.scrape_metrics()
        assert m["engine/isoexec_requests_served_total"] == 5 and m["engine/isoexec_decode_tokens_total"] >= 5 * 6
        assert m["engine/isoexec_prefill_tokens_total"] == 5 * 9 and m["engine/isoexec_requests_running"] == 0
        # the logprobs the server reports are the model's: a clean scoring pass reproduces them bit for bit
        from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
        from skyrl_isoexec_b200.train.policy_worker import PolicyWorker

        seq, att, rmask = build_sequences(prompts, out["response_ids"])
        lp = PolicyWorker(e1.model).forward(TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask}))
        assert torch.equal(lp, torch.tensor(out["response_logprobs"]))
        # OpenAI-style completion with token-id prompts
        r = asyncio.run(cl.completion({"prompt": prompts[0], "max_tokens": 4, "n": 2, "logprobs": 1, "ignore_eos": True}))
        assert len(r["choices"]) == 2 and r["usage"]["completion_tokens"] == 8 and len(r["choices"][0]["logprobs"]["token_logprobs"]) == 4
        # weights from a file: after the update server 0 computes with the new weights
        new = DecoderLM(get_config("tiny-qwen3"), seed=9)
        path = str(tmp_path / "w.pt")
        torch.save({"model": dict(new.named_weights())}, path)
        asyncio.run(cl.pause_generation("finish"))
        asyncio.run(cl.update_named_weights({"path": path}))
        asyncio.run(cl.resume_generation())
        assert torch.equal(e1.model.store.flat, new.store.flat)
        # a dead URL: transient errors are retried, then reported
        dead = RemoteInferenceClient(["http://127.0.0.1:9"], max_retries=2, backoff_s=0.001, timeout_s=1)
        with pytest.raises(ConnectionError):
            dead.server_info()
        assert dead.retries == 3
    finally:
        group.shutdown()


def test_pause_abort_ends_running_requests_and_keep_resumes():
    # a context long enough that the request cannot run into the length limit before the test aborts it
    srv = InferenceServer(_engine(max_position=16384, pages=160)).start()
    try:
        cl = RemoteInferenceClient([srv.url], timeout_s=60)
        res = {}

        def long_call():
            res["out"] = asyncio.run(cl.generate({"prompt_token_ids": [[1, 2, 3]], "sampling_params": {"max_generate_length": 100000, "ignore_eos": True}}))

        t = threading.Thread(target=long_call)
        t.start()
        t0 = time.time()
        while time.time() - t0 < 20 and not (srv._pending and srv._pending[0].seqs and len(srv._pending[0].seqs[0].output_ids) > 2):
            time.sleep(0.02)                      # wait until the request is really decoding, however slow the machine
        asyncio.run(cl.pause_generation("keep"))
        n1 = len(srv._pending[0].seqs[0].output_ids)
        time.sleep(0.1)
        assert len(srv._pending[0].seqs[0].output_ids) == n1 and n1 > 0      # parked, not lost
        asyncio.run(cl.resume_generation())
        time.sleep(0.1)
        r = asyncio.run(cl.pause_generation("abort"))
        t.join(timeout=20)
        assert r[0]["aborted"] == 1 and res["out"]["stop_reasons"][0] == "abort"
        assert len(res["out"]["response_ids"][0]) > n1
        with pytest.raises(RuntimeError, match="paused"):
            asyncio.run(cl.generate({"prompt_token_ids": [[1, 2, 3]], "sampling_params": {"max_generate_length": 2}}))
        asyncio.run(cl.resume_generation())
        out = asyncio.run(cl.generate({"prompt_token_ids": [[1, 2, 3]], "sampling_params": {"max_generate_length": 2, "ignore_eos": True}}))
        assert len(out["response_ids"][0]) == 2
    finally:
        srv.shutdown()


def test_tinker_backend_samples_through_an_external_server_and_trains_on_the_result():
    """The training backend forwards ``sample`` to an OpenAI-compatible server (here: this framework's own, holding the
    same weights) and gets back ids and logprobs that its own forward reproduces bit for bit."""
    from skyrl_isoexec_b200.tinker.backend import SkyRLTrainBackend

    srv = InferenceServer(_engine(seed=0)).start()
    try:
        be = SkyRLTrainBackend("tiny-qwen3", device="cpu", seed=0, external_inference_url=srv.url + "/", lr=1e-3)
        assert torch.equal(be.model.store.flat, srv.llm.model.store.flat), "same preset and seed: same weights on both sides"
        prompt = list(range(5, 17))
        out = be.handle({"type": "sample", "prompt_ids": prompt, "num_samples": 3,
                         "sampling_params": {"max_generate_length": 6, "ignore_eos": True, "temperature": 1.0}})
        seqs = out["sequences"]
        assert len(seqs) == 3 and all(len(s["tokens"]) == 6 == len(s["logprobs"]) and s["stop_reason"] == "length" for s in seqs)
        data = [{"prompt_ids": prompt, "response_ids": s["tokens"], "advantages": [1.0] * 6, "logprobs": s["logprobs"]} for s in seqs]
        fwd = be.handle({"type": "forward", "data": data, "loss_fn": "importance_sampling"})
        for got, s in zip(fwd["logprobs"], seqs):
            assert got == s["logprobs"], "the external engine's logprobs are the trainer's, bit for bit"
    finally:
        srv.shutdown()


def test_router_routes_pins_sessions_fans_out_control_and_survives_a_dead_backend(tmp_path):
    """One address in front of two engine servers: conversations stick to a backend, a batch is split and joined in
    order, control calls reach every backend, a layer-wise reload changes the weights of both, and a backend that went
    away is skipped (and the call that found it dead is retried elsewhere)."""
    import json
    import urllib.request

    from safetensors.torch import save_file

    from skyrl_isoexec_b200.engine.router import Router

    def call(url, path, body=None, headers=None):
        req = urllib.request.Request(url + path, data=None if body is None else json.dumps(body).encode(),
                                     method="GET" if body is None else "POST", headers={"Content-Type": "application/json", **(headers or {})})
        try:
            with urllib.request.urlopen(req, timeout=60) as r:
                raw = r.read()
                return r.status, (json.loads(raw) if r.headers.get("Content-Type", "").startswith("application/json") else raw.decode())
        except urllib.error.HTTPError as e:
            return e.code, json.loads(e.read())

    e1, e2 = _engine(seed=0), _engine(seed=0)
    group = ServerGroup([e1, e2])
    urls = group.start()
    router = Router(urls, probe_s=0.2, timeout_s=60).start()
    try:
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, 2048, (8,), generator=g).tolist() for _ in range(6)]
        sp = {"max_generate_length": 5, "ignore_eos": True, "temperature": 0.0}
        code, out = call(router.url, "/generate", {"prompt_token_ids": prompts, "sampling_params": sp})
        assert code == 200 and len(out["response_ids"]) == 6
        code, one = call(router.url, "/generate", {"prompt_token_ids": [prompts[4]], "sampling_params": sp})
        assert one["response_ids"][0] == out["response_ids"][4]                     # split and joined in order
        assert sorted(router.served.values()) == [2, 2] or sum(router.served.values()) == 3
        # a conversation stays on one backend
        before = dict(router.served)
        for _ in range(3):
            assert call(router.url, "/generate", {"prompt_token_ids": [prompts[0]], "sampling_params": sp, "session_id": "conv-7"})[0] == 200
        assert call(router.url, "/generate", {"prompt_token_ids": [prompts[1]], "sampling_params": sp}, {"X-Session-Id": "conv-7"})[0] == 200
        grown = [router.served[b] - before[b] for b in router.backends]
        assert sorted(grown) == [0, 4]
        # control plane: every backend, and a failure of one is a failure of the call
        code, res = call(router.url, "/pause", {"mode": "keep"})
        assert code == 200 and res["ok"] and len(res["backends"]) == 2
        donor = DecoderLM(get_config("tiny-qwen3", max_position=512), seed=42)
        wfile = str(tmp_path / "w.safetensors")
        save_file({n: t.detach().clone().contiguous() for n, t in donor.named_weights()}, wfile)
        code, res = call(router.url, "/update_weights_layerwise", {"path": wfile, "layers_per_step": 1})
        assert code == 200 and all(r["reply"]["steps"] >= 3 and r["reply"]["tensors"] == len(list(donor.named_weights()))
                                   for r in res["backends"].values())
        total = sum(t.numel() * t.element_size() for _, t in donor.named_weights())
        assert all(r["reply"]["peak_host_bytes"] < total for r in res["backends"].values())      # never the whole model at once
        assert call(router.url, "/resume", {})[0] == 200
        for e in (e1, e2):
            assert all(torch.equal(a, b) for (_, a), (_, b) in zip(e.model.named_weights(), donor.named_weights()))
        code, res = call(router.url, "/update_weights", {"path": str(tmp_path / "missing.pt")})
        assert code == 502 and not res["ok"]
        code, text = call(router.url, "/metrics")
        assert code == 200 and "router_requests_served" in text and "isoexec_requests_served_total" in text
        assert call(router.url, "/get_server_info")[1]["router"]["sessions"] == 1
        # one backend goes away: the data plane keeps answering from the other
        group.servers[0].shutdown()
        dead = group.servers[0].url if hasattr(group.servers[0], "url") else urls[0]
        for _ in range(4):
            assert call(router.url, "/generate", {"prompt_token_ids": [prompts[2]], "sampling_params": sp})[0] == 200
        assert router.healthy[dead.rstrip("/")] is False and call(router.url, "/health")[1]["healthy_backends"] == 1
    finally:
        router.shutdown()
        group.shutdown()


def test_server_samples_of_one_prompt_share_pages():
    """``n`` completions of one prompt through the HTTP server prefill the prompt once."""
    e = _engine(pages=40)
    srv = InferenceServer(e).start()
    try:
        import json
        import urllib.request

        prompt = torch.randint(0, 2048, (300,), generator=torch.Generator().manual_seed(3)).tolist()
        req = urllib.request.Request(srv.url + "/v1/completions", data=json.dumps({"prompt": prompt, "n": 4, "max_tokens": 5, "temperature": 0.0}).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            out = json.loads(r.read())
        assert len(out["choices"]) == 4 and len({tuple(c["token_ids"]) for c in out["choices"]}) == 1      # greedy: identical
        assert e.scheduler.shared_prompt_tokens == 3 * 256 and e.stats["prefill_tokens"] == 300 + 3 * 44
    finally:
        srv.shutdown()
