"""Stand-alone inference server (reference: R/train/entrypoints/serve.py): one engine behind the HTTP data and control
plane of ``engine/server.py`` (OpenAI-style ``/v1/completions``, token-level ``/generate``, pause / resume, weight
update, ``/metrics``).

    python -m skyrl_isoexec_b200.train.entrypoints.serve [--model qwen3-8b] [--weights DIR_OR_FILE] [--host 127.0.0.1] [--port 8000]
        [--max-num-seqs 64] [--num-kv-pages 0] [--seed 0] [--enable-prefix-caching]

``--weights``: a Hugging Face style directory written by ``models/hf_export.py`` or a ``torch.save`` file with a
``model`` dict; without it the server starts on the seeded random initialisation (for tests).
"""

from __future__ import annotations

import argparse
import os
import time

import torch

from ...engine.llm_engine import EngineConfig, LLMEngine
from ...engine.server import InferenceServer
from ...models.config import get_config
from ...models.decoder import DecoderLM
from ...utils.tokenizer import ByteTokenizer


def build(argv=None) -> InferenceServer:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-qwen3")
    ap.add_argument("--weights", default="")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--num-kv-pages", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--enable-prefix-caching", action="store_true",
                    help="keep full KV pages after their request and reuse them for later requests with the same leading tokens")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    model = DecoderLM(get_config(a.model), device=a.device, seed=a.seed)
    if a.weights:
        if os.path.isdir(a.weights):
            from ...models import hf_export

            hf_export.load_hf(model, a.weights)
        else:
            from ...sync.strategies import load_weights

            load_weights(model, torch.load(a.weights, map_location="cpu", weights_only=False)["model"].items())
    kw = {"max_num_seqs": a.max_num_seqs, "seed": a.seed, "enable_prefix_caching": a.enable_prefix_caching}
    if a.num_kv_pages:
        kw["num_kv_pages"] = a.num_kv_pages
    eng = LLMEngine(model, EngineConfig(**kw))
    return InferenceServer(eng, ByteTokenizer(), host=a.host, port=a.port, model_name=a.model)


def main(argv=None) -> None:
    srv = build(argv).start()
    print(f"serving {srv.model_name} at {srv.url}", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.shutdown()


if __name__ == "__main__":
    main()
