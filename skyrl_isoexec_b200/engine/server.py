"""HTTP inference server over the native engine, plus the client the trainer uses to reach one or many of them
(reference: B/inference_servers/{remote_inference_client,server_group,vllm_server_actor,vllm_router}.py and the
HTTP endpoint of B/inference_engines/inference_engine_client.py).

Server (``InferenceServer``): a stdlib threading HTTP server in front of ONE engine loop thread, which owns the
engine and does continuous batching across all connections.
  data plane     POST /generate               token-in / token-out ({prompt_token_ids, sampling_params, session_id})
                 POST /v1/completions         OpenAI-compatible (``prompt`` may be text or token ids)
                 POST /v1/chat/completions    OpenAI-compatible (needs a tokenizer with a chat template)
  control plane  GET  /health, /get_server_info, /metrics (Prometheus text format)
                 POST /pause {mode: abort|keep|finish}, /resume, /sleep, /wake_up, /reset_prefix_cache,
                      /update_weights {path} (a checkpoint directory or a flat .pt), /shutdown

Client (``RemoteInferenceClient``): routes the data plane over several server URLs (session affinity by hash,
otherwise round-robin), fans the control plane out to all of them, and retries transient failures with
exponential backoff. While servers are paused in ``keep`` mode, data-plane calls wait instead of failing.
"""

from __future__ import annotations

from ..utils.tokenizer import chat_ids

import asyncio
import json
import threading
import time
import urllib.error
import urllib.request
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from .interface import InferenceEngineInterface
from .sampler import SamplingParams

PAUSE_MODES = ("abort", "keep", "finish")


class _Pending:
    __slots__ = ("seqs", "event", "aborted")

    def __init__(self, seqs):
        self.seqs, self.event, self.aborted = seqs, threading.Event(), False


class InferenceServer:
    def __init__(self, llm, tokenizer=None, host: str = "127.0.0.1", port: int = 0, model_name: str = "policy"):
        self.llm, self.tokenizer, self.model_name = llm, tokenizer, model_name
        eos = getattr(tokenizer, "eos_token_id", None)
        if eos is not None and getattr(getattr(llm, "cfg", None), "eos_token_id", 0) is None:
            llm.cfg.eos_token_id = int(eos)
        self._lock = threading.Lock()          # guards the engine (steps, admissions, control verbs)
        self._pending: list[_Pending] = []
        self._stop = threading.Event()
        self._paused_mode: str | None = None
        self.requests_served = 0
        outer = self

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, *a):  # quiet
                pass

            def _reply(self, code, obj):
                body = json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def do_GET(self):
                if self.path == "/health":
                    return self._reply(200, {"status": "ok"})
                if self.path == "/get_server_info":
                    return self._reply(200, outer.info())
                if self.path == "/v1/models":
                    return self._reply(200, {"object": "list", "data": [{"id": outer.model_name, "object": "model"}]})
                if self.path == "/metrics":
                    body = outer.metrics_text().encode()
                    self.send_response(200)
                    self.send_header("Content-Type", "text/plain; version=0.0.4")
                    self.send_header("Content-Length", str(len(body)))
                    self.end_headers()
                    self.wfile.write(body)
                    return None
                self._reply(404, {"error": f"no route {self.path}"})

            def do_POST(self):
                n = int(self.headers.get("Content-Length") or 0)
                try:
                    payload = json.loads(self.rfile.read(n) or b"{}")
                    code, obj = outer.dispatch(self.path, payload)
                except Exception as e:  # noqa: BLE001
                    code, obj = 400, {"error": f"{type(e).__name__}: {e}"}
                self._reply(code, obj)

        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.httpd.daemon_threads = True
        self.host, self.port = self.httpd.server_address[:2]
        self.url = f"http://{self.host}:{self.port}"
        self._threads = [threading.Thread(target=self.httpd.serve_forever, daemon=True),
                         threading.Thread(target=self._engine_loop, daemon=True)]

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> "InferenceServer":
        for t in self._threads:
            t.start()
        return self

    def shutdown(self) -> None:
        self._stop.set()
        self.httpd.shutdown()
        self.httpd.server_close()

    def info(self) -> dict:
        ps = self.llm.model.ps
        return {"model": self.model_name, "tp_size": ps.tp, "dp_size": 1, "pp_size": 1, "paused": self._paused_mode,
                "asleep": bool(getattr(self.llm, "asleep", False)), "requests_served": self.requests_served,
                "max_model_len": self.llm.max_len}

    def metrics_text(self) -> str:
        """Engine counters in the Prometheus text format (the reference scrapes vLLM's /metrics into its tracker,
        R/train/utils/vllm_metrics_scraper.py). Counters are cumulative since the server started."""
        st = dict(getattr(self.llm, "stats", {}) or {})
        rows = [("isoexec_requests_served_total", "counter", self.requests_served),
                ("isoexec_engine_steps_total", "counter", st.get("steps", 0)),
                ("isoexec_tokens_total", "counter", st.get("tokens", 0)),
                ("isoexec_prefill_tokens_total", "counter", st.get("prefill_tokens", 0)),
                ("isoexec_decode_tokens_total", "counter", st.get("decode_tokens", 0)),
                ("isoexec_h2d_bytes_total", "counter", st.get("h2d_bytes", 0)),
                ("isoexec_d2h_bytes_total", "counter", st.get("d2h_bytes", 0)),
                ("isoexec_requests_running", "gauge", len(getattr(self.llm, "running", []) or [])),
                ("isoexec_requests_waiting", "gauge", len(getattr(self.llm, "waiting", []) or [])),
                ("isoexec_paused", "gauge", 0 if self._paused_mode in (None, "", "none") else 1)]
        pc = getattr(self.llm, "prefix_cache", None)
        if pc is not None:
            rows += [("isoexec_prefix_cache_hits_total", "counter", pc.hits), ("isoexec_prefix_cache_misses_total", "counter", pc.misses),
                     ("isoexec_prefix_cache_hit_tokens_total", "counter", pc.hit_tokens), ("isoexec_prefix_cache_evicted_total", "counter", pc.evicted),
                     ("isoexec_prefix_cache_pages", "gauge", len(pc))]
        out = []
        for name, kind, val in rows:
            out.append(f"# TYPE {name} {kind}")
            out.append(f'{name}{{model="{self.model_name}"}} {float(val):g}')
        return "\n".join(out) + "\n"

    # ------------------------------------------------------------------ the engine loop (one thread owns the engine)
    def _engine_loop(self) -> None:
        while not self._stop.is_set():
            with self._lock:
                busy = self.llm.scheduler.has_work() and self._paused_mode != "keep" and not getattr(self.llm, "asleep", False)
                if busy:
                    self.llm.step()
                done = [p for p in self._pending if p.aborted or all(s.finished for s in p.seqs)]
                for p in done:
                    self._pending.remove(p)
            for p in done:
                p.event.set()
            if not busy:
                time.sleep(0.001)

    def _submit(self, prompts: list[list[int]], sp: SamplingParams, timeout: float = 3600.0, mm: list | None = None):
        if self._paused_mode in ("abort", "finish"):
            raise RuntimeError("server is paused; resume before sending requests")
        with self._lock:
            seqs = [self.llm.add_request(p, sp, i, **({"mm": mm[i]} if mm is not None and mm[i] is not None else {}))
                    for i, p in enumerate(prompts)]
            self.llm.link_samples(seqs)            # n > 1 samples of a prompt share its KV pages
            pend = _Pending(seqs)
            self._pending.append(pend)
        if not pend.event.wait(timeout):
            raise TimeoutError("generation did not finish in time")
        self.requests_served += len(prompts)
        return seqs, pend.aborted

    # ------------------------------------------------------------------ routes
    def dispatch(self, path: str, body: dict):
        if path == "/generate":
            return 200, self._generate(body)
        if path == "/v1/completions":
            return 200, self._completions(body)
        if path == "/v1/chat/completions":
            return 200, self._chat(body)
        if path == "/v1/chat/completions/render":
            return 200, self._render(body)
        if path == "/pause":
            return 200, self.pause(body.get("mode", "keep"))
        if path == "/resume":
            self._paused_mode = None
            self.llm.resume_generation()
            return 200, {"ok": True}
        if path in ("/sleep", "/wake_up", "/reset_prefix_cache"):
            with self._lock:
                getattr(self.llm, path[1:])(*([body.get("tags")] if path != "/reset_prefix_cache" else []))
            return 200, {"ok": True}
        if path == "/update_weights":
            return 200, self._update_weights(body)
        if path == "/update_weights_layerwise":
            return 200, self._update_weights_layerwise(body)
        if path == "/shutdown":
            threading.Thread(target=self.shutdown, daemon=True).start()
            return 200, {"ok": True}
        return 404, {"error": f"no route {path}"}

    def pause(self, mode: str) -> dict:
        """abort: running requests end now with what they have (stop_reason "abort");
        keep: requests stay queued with their KV state and continue after /resume;
        finish: no new requests are admitted, running ones run to completion."""
        if mode not in PAUSE_MODES:
            raise ValueError(f"pause mode {mode!r} not in {PAUSE_MODES}")
        with self._lock:                       # a step in flight finishes before the pause takes effect
            self._paused_mode = mode
            self.llm.pause_generation()
        aborted = 0
        if mode == "abort":
            with self._lock:
                for p in self._pending:
                    for s in p.seqs:
                        if not s.finished:
                            s.finished, s.stop_reason = True, "abort"
                            self.llm.scheduler.finish(s)
                            aborted += 1
                    p.aborted = True
        elif mode == "finish":
            while True:
                with self._lock:
                    if not self._pending:
                        break
                time.sleep(0.002)
        return {"ok": True, "mode": mode, "aborted": aborted}

    def _update_weights(self, body: dict) -> dict:
        import torch

        from ..sync.strategies import load_weights

        path = body["path"]
        with self._lock:
            if self.llm.scheduler.has_work() and self._paused_mode is None:
                raise RuntimeError("pause the server before updating weights")
            sd = torch.load(path, weights_only=False, map_location="cpu")
            sd = sd.get("model", sd)
            n = load_weights(self.llm.model, sd.items())
            self.llm.reset_prefix_cache()
        return {"ok": True, "tensors": n}

    def _update_weights_layerwise(self, body: dict) -> dict:
        """Reload from a ``.safetensors`` file with this model's parameter names, a group of layers at a time: only
        ``layers_per_step`` layers' tensors are held on the host at once (a full ``torch.load`` holds the whole model),
        and full-shape tensors are cut to this engine's shard as they are read."""
        from safetensors import safe_open

        from ..sync.strategies import load_weights

        per = max(1, int(body.get("layers_per_step", 4)))
        with self._lock:
            if self.llm.scheduler.has_work() and self._paused_mode is None:
                raise RuntimeError("pause the server before updating weights")
            n, steps, peak = 0, 0, 0
            with safe_open(body["path"], framework="pt", device="cpu") as f:
                groups: dict = {}
                for k in f.keys():
                    parts = k.split(".")
                    g = int(parts[1]) // per if parts[0] == "layers" and len(parts) > 1 and parts[1].isdigit() else -1
                    groups.setdefault(g, []).append(k)
                for g in sorted(groups):
                    held = {k: f.get_tensor(k) for k in groups[g]}
                    peak = max(peak, sum(t.numel() * t.element_size() for t in held.values()))
                    n += load_weights(self.llm.model, held.items())
                    steps += 1
                    del held
            self.llm.reset_prefix_cache()
        return {"ok": True, "tensors": n, "steps": steps, "peak_host_bytes": peak}

    def _encode(self, prompt):
        if isinstance(prompt, list) and (not prompt or isinstance(prompt[0], int)):
            return prompt
        if self.tokenizer is None:
            raise ValueError("text prompts need a tokenizer; send token ids")
        if isinstance(prompt, str):
            return self.tokenizer.encode(prompt)
        return chat_ids(self.tokenizer, prompt)

    def _generate(self, body: dict) -> dict:
        ids = body["prompt_token_ids"]
        ids = ids if ids and isinstance(ids[0], list) else [ids]
        mm = body.get("mm_features")
        if mm is not None:                       # per prompt: the ``features`` of /v1/chat/completions/render, or null
            from .renderer import decode_features

            mm = [decode_features(f) for f in mm]
        seqs, aborted = self._submit(ids, SamplingParams.from_dict(body.get("sampling_params")), mm=mm)
        out = {"response_ids": [s.output_ids for s in seqs], "response_logprobs": [s.logprobs for s in seqs],
               "stop_reasons": [s.stop_reason for s in seqs], "aborted": aborted}
        if any(s.prompt_logprobs is not None for s in seqs):
            out["prompt_logprobs"] = [s.prompt_logprobs for s in seqs]
        return out

    def _render(self, body: dict) -> dict:
        """Token ids of a conversation with every image a run of placeholder tokens, and the images' patches in a
        JSON-safe form (``engine/renderer.py``); what the answer's ``features`` hold goes back in ``/generate`` as
        ``mm_features``."""
        from .renderer import encode_features, render_conversation

        if self.tokenizer is None:
            raise ValueError("rendering a conversation needs a tokenizer")
        r = render_conversation(body["messages"], self.tokenizer, self.llm.mcfg, body.get("add_generation_prompt", True))
        return {"token_ids": r["token_ids"], "features": encode_features(r["features"])}

    def _openai_params(self, body: dict) -> SamplingParams:
        d = {"max_generate_length": body.get("max_tokens", 16), "temperature": body.get("temperature", 1.0),
             "top_p": body.get("top_p", 1.0)}
        for k in ("top_k", "min_p", "seed", "stop_token_ids", "ignore_eos"):
            if k in body:
                d[k] = body[k]
        return SamplingParams.from_dict(d)

    def _completions(self, body: dict) -> dict:
        prompts = body["prompt"]
        batch = prompts if isinstance(prompts, list) and prompts and isinstance(prompts[0], (list, str)) else [prompts]
        n = int(body.get("n", 1))
        ids = [self._encode(p) for p in batch for _ in range(n)]
        seqs, _ = self._submit(ids, self._openai_params(body))
        want_lp = body.get("logprobs") is not None
        choices = []
        for i, s in enumerate(seqs):
            c = {"index": i, "text": self.tokenizer.decode(s.output_ids) if self.tokenizer is not None else "",
                 "token_ids": s.output_ids, "finish_reason": "length" if s.stop_reason == "length" else "stop"}
            if want_lp:
                c["logprobs"] = {"token_logprobs": s.logprobs}
            choices.append(c)
        usage = {"prompt_tokens": sum(len(p) for p in ids), "completion_tokens": sum(len(s.output_ids) for s in seqs)}
        usage["total_tokens"] = usage["prompt_tokens"] + usage["completion_tokens"]
        return {"id": "cmpl-" + uuid.uuid4().hex[:12], "object": "text_completion", "created": int(time.time()),
                "model": self.model_name, "choices": choices, "usage": usage}

    def _chat(self, body: dict) -> dict:
        ids = [self._encode(body["messages"]) for _ in range(int(body.get("n", 1)))]
        seqs, _ = self._submit(ids, self._openai_params({**body, "max_tokens": body.get("max_tokens", body.get("max_completion_tokens", 16))}))
        choices = [{"index": i, "message": {"role": "assistant", "content": self.tokenizer.decode(s.output_ids)},
                    "finish_reason": "length" if s.stop_reason == "length" else "stop"} for i, s in enumerate(seqs)]
        return {"id": "chatcmpl-" + uuid.uuid4().hex[:12], "object": "chat.completion", "created": int(time.time()),
                "model": self.model_name, "choices": choices}


class ServerGroup:
    """Several servers in one process (one per engine), started and stopped together."""

    def __init__(self, engines: list, tokenizer=None, host: str = "127.0.0.1"):
        self.servers = [InferenceServer(e, tokenizer, host) for e in engines]

    def start(self) -> list[str]:
        return [s.start().url for s in self.servers]

    def shutdown(self) -> None:
        for s in self.servers:
            s.shutdown()


class RemoteInferenceClient(InferenceEngineInterface):
    def __init__(self, urls: list[str], max_retries: int = 4, backoff_s: float = 0.05, timeout_s: float = 3600.0):
        self.urls, self.max_retries, self.backoff_s, self.timeout_s = list(urls), max_retries, backoff_s, timeout_s
        self._rr = 0
        self.retries = 0

    # ------------------------------------------------------------------ transport
    def _post(self, url: str, path: str, body: dict | None = None, method: str = "POST") -> dict:
        data = json.dumps(body or {}).encode() if method == "POST" else None
        last = None
        for attempt in range(self.max_retries + 1):
            try:
                req = urllib.request.Request(url + path, data=data, method=method, headers={"Content-Type": "application/json"})
                with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
                    return json.loads(r.read())
            except urllib.error.HTTPError as e:           # the server answered: not transient
                raise RuntimeError(f"{url}{path}: HTTP {e.code}: {e.read().decode(errors='replace')[:300]}") from None
            except (urllib.error.URLError, ConnectionError, TimeoutError) as e:
                last = e
                self.retries += 1
                time.sleep(self.backoff_s * (2 ** attempt))
        raise ConnectionError(f"{url}{path}: no answer after {self.max_retries + 1} attempts: {last}")

    def scrape_metrics(self) -> dict:
        """GET /metrics of every server, summed per metric name: ``{"engine/<name>": value}`` for the tracker."""
        import urllib.request

        tot: dict = {}
        for u in self.urls:
            with urllib.request.urlopen(u + "/metrics", timeout=10) as r:
                for line in r.read().decode().splitlines():
                    if line and not line.startswith("#"):
                        name, val = line.rsplit(" ", 1)
                        key = "engine/" + name.split("{", 1)[0]
                        tot[key] = tot.get(key, 0.0) + float(val)
        return tot

    def _pick(self, session_id=None) -> str:
        if session_id is not None:
            return self.urls[hash(str(session_id)) % len(self.urls)]
        self._rr += 1
        return self.urls[self._rr % len(self.urls)]

    # ------------------------------------------------------------------ data plane
    async def generate(self, input_batch):
        ids = input_batch["prompt_token_ids"]
        sess = input_batch.get("session_ids") or [None] * len(ids)
        by_url: dict = {}
        for i, (p, s) in enumerate(zip(ids, sess)):
            by_url.setdefault(self._pick(s), []).append(i)
        loop = asyncio.get_running_loop()

        mm = input_batch.get("mm_features")
        if mm is not None:
            from .renderer import encode_features

            mm = [f if f is None or "kwargs_data" in f else encode_features(f) for f in mm]

        def call(url, idx):
            body = {"prompt_token_ids": [ids[i] for i in idx], "sampling_params": input_batch.get("sampling_params")}
            if mm is not None:
                body["mm_features"] = [mm[i] for i in idx]
            return idx, self._post(url, "/generate", body)

        parts = await asyncio.gather(*[loop.run_in_executor(None, call, u, ix) for u, ix in by_url.items()])
        n = len(ids)
        out = {"responses": [""] * n, "response_ids": [None] * n, "stop_reasons": [None] * n, "response_logprobs": [None] * n,
               "prompt_logprobs": None, "rollout_expert_indices": None}
        for idx, r in parts:
            for j, i in enumerate(idx):
                out["response_ids"][i], out["response_logprobs"][i] = r["response_ids"][j], r["response_logprobs"][j]
                out["stop_reasons"][i] = r["stop_reasons"][j]
                if r.get("prompt_logprobs") is not None:
                    if out["prompt_logprobs"] is None:
                        out["prompt_logprobs"] = [None] * n
                    out["prompt_logprobs"][i] = r["prompt_logprobs"][j]
        return out

    async def completion(self, request_payload: dict) -> dict:
        return self._post(self._pick(request_payload.get("session_id")), "/v1/completions", request_payload)

    async def chat_completion(self, request_payload: dict) -> dict:
        return self._post(self._pick(request_payload.get("session_id")), "/v1/chat/completions", request_payload)

    async def render_chat_completion(self, request_payload: dict) -> dict:
        """Messages may hold images as data URLs only (the request is JSON)."""
        from .renderer import decode_features

        r = self._post(self._pick(None), "/v1/chat/completions/render", request_payload.get("json", request_payload))
        return {"token_ids": r["token_ids"], "features": decode_features(r.get("features"))}

    # ------------------------------------------------------------------ control plane (fan-out)
    def _all(self, path: str, body: dict | None = None) -> list[dict]:
        return [self._post(u, path, body) for u in self.urls]

    async def wake_up(self, *a, tags=None, **kw):
        return self._all("/wake_up", {"tags": tags})

    async def sleep(self, *a, tags=None, **kw):
        return self._all("/sleep", {"tags": tags})

    async def reset_prefix_cache(self):
        return self._all("/reset_prefix_cache")

    async def pause_generation(self, mode: str = "keep"):
        return self._all("/pause", {"mode": mode})

    async def resume_generation(self):
        return self._all("/resume")

    async def init_weight_update_communicator(self, init_info):
        return True

    async def update_named_weights(self, request):
        """``request``: {"path": checkpoint file every server can read}."""
        return self._all("/update_weights", request)

    def server_info(self) -> list[dict]:
        return [self._post(u, "/get_server_info", method="GET") for u in self.urls]

    async def teardown(self):
        for u in self.urls:
            try:
                self._post(u, "/shutdown")
            except Exception:  # noqa: BLE001
                pass

    def tp_size(self) -> int:
        return int(self.server_info()[0]["tp_size"])

    def dp_size(self) -> int:
        return len(self.urls)
