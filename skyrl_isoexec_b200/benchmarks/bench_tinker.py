"""Throughput of the Tinker-style service: requests per second through the futures queue for the three verbs that
matter (sample, forward_backward, optim_step), over HTTP on 127.0.0.1 (reference: R/benchmarks/ Tinker engine bench).

    python -m skyrl_isoexec_b200.benchmarks.bench_tinker [--model tiny-qwen3] [--requests 16] [--device cpu]
"""

from __future__ import annotations

import argparse
import json
import time

import torch

from ..tinker.api import TinkerClient, TinkerServer


def run(model: str = "tiny-qwen3", requests: int = 16, device: str | None = None, prompt_len: int = 16, response_len: int = 16) -> dict:
    srv = TinkerServer(device=device).start()
    try:
        cl = TinkerClient(srv.url)
        mid = cl.create_model(base_model=model, lr=1e-5)
        g = torch.Generator().manual_seed(0)
        data = [{"prompt_ids": torch.randint(0, 500, (prompt_len,), generator=g).tolist(),
                 "response_ids": torch.randint(0, 500, (response_len,), generator=g).tolist()} for _ in range(4)]
        out = {}
        t0 = time.perf_counter()
        ids = [cl.submit("asample", model_id=mid, prompt_ids=data[0]["prompt_ids"], num_samples=1,
                         sampling_params={"max_generate_length": response_len, "ignore_eos": True}) for _ in range(requests)]
        toks = sum(len(cl.result(i)["sequences"][0]["tokens"]) for i in ids)
        dt = time.perf_counter() - t0
        out["sample"] = {"requests_per_s": requests / dt, "tokens_per_s": toks / dt}
        t0 = time.perf_counter()
        ids = []
        for _ in range(requests):
            ids.append(cl.submit("forward_backward", model_id=mid, data=data, loss_fn="cross_entropy"))
            ids.append(cl.submit("optim_step", model_id=mid, adam_params={}))
        for i in ids:
            cl.result(i)
        dt = time.perf_counter() - t0
        out["train"] = {"steps_per_s": requests / dt, "tokens_per_s": requests * 4 * response_len / dt}
        return out
    finally:
        srv.shutdown()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-qwen3")
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    print(json.dumps(run(a.model, a.requests, a.device)))


if __name__ == "__main__":
    main()
