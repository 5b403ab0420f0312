"""Concurrency load test of the HTTP inference server (reference: R/benchmarks/ concurrency load test).

    python -m skyrl_isoexec_b200.benchmarks.load_test --url http://127.0.0.1:8000 --concurrency 64 --requests 512 \
        --prompt-len 512 --max-tokens 256
    python -m skyrl_isoexec_b200.benchmarks.load_test --self-host tiny-qwen3 ...      # starts a server in this process

Reports requests/s, generated tokens/s and latency percentiles. Uses only the standard library on the client side.
"""

from __future__ import annotations

import argparse
import json
import random
import threading
import time
import urllib.request


def _post(url, body, timeout):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def run(url: str, concurrency: int, requests: int, prompt_len: int, max_tokens: int, vocab: int, timeout: float = 600.0) -> dict:
    lat, toks, errs = [], [], []
    lock = threading.Lock()
    todo = list(range(requests))

    def worker(seed):
        rng = random.Random(seed)
        while True:
            with lock:
                if not todo:
                    return
                todo.pop()
            body = {"prompt_token_ids": [rng.randrange(vocab) for _ in range(prompt_len)],
                    "sampling_params": {"max_generate_length": max_tokens, "ignore_eos": True}}
            t0 = time.perf_counter()
            try:
                out = _post(url + "/generate", body, timeout)
                with lock:
                    lat.append(time.perf_counter() - t0)
                    toks.append(len(out["response_ids"][0]))
            except Exception as e:  # noqa: BLE001
                with lock:
                    errs.append(str(e))

    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker, args=(i,)) for i in range(concurrency)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    lat.sort()
    pct = lambda p: lat[min(len(lat) - 1, int(p * len(lat)))] if lat else float("nan")  # noqa: E731
    return {"requests": len(lat), "errors": len(errs), "wall_s": wall, "req_per_s": len(lat) / wall, "tok_per_s": sum(toks) / wall,
            "p50_s": pct(0.5), "p90_s": pct(0.9), "p99_s": pct(0.99)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="")
    ap.add_argument("--self-host", default="", help="model preset to serve from this process")
    ap.add_argument("--concurrency", type=int, default=16)
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=64)
    ap.add_argument("--max-tokens", type=int, default=32)
    args = ap.parse_args(argv)
    srv, vocab = None, 32000
    if args.self_host:
        import torch

        from ..engine.llm_engine import EngineConfig, LLMEngine
        from ..engine.server import InferenceServer
        from ..models.config import get_config
        from ..models.decoder import DecoderLM

        cfg = get_config(args.self_host)
        vocab = cfg.vocab_size
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        eng = LLMEngine(DecoderLM(cfg, device=dev), EngineConfig(max_num_seqs=max(16, args.concurrency),
                                                                 num_kv_pages=max(64, args.concurrency * ((args.prompt_len + args.max_tokens) // 128 + 2))))
        srv = InferenceServer(eng).start()
        args.url = srv.url
    try:
        print(json.dumps(run(args.url, args.concurrency, args.requests, args.prompt_len, args.max_tokens, vocab)))
    finally:
        if srv is not None:
            srv.shutdown()


if __name__ == "__main__":
    main()
