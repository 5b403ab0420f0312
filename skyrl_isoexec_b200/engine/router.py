"""A routing front end for several inference servers (reference: the router process of R/backends/skyrl_train/
inference_servers/, which sits between the generator and the per-engine HTTP servers).

    python -m skyrl_isoexec_b200.engine.router --backends http://127.0.0.1:8001,http://127.0.0.1:8002 [--port 8000]

One address for the data plane and the control plane:

* ``/generate``, ``/v1/completions``, ``/v1/chat/completions`` go to ONE backend: the one a ``session_id`` (body field or
  ``X-Session-Id`` header) was pinned to, so that the turns of a conversation meet the same engine, otherwise the
  healthy backend with the fewest requests in flight (ties: round robin). ``/generate`` with several prompts and no
  session is split over the healthy backends in contiguous pieces and the answers are joined in order.
* ``/pause``, ``/resume``, ``/update_weights``, ``/update_weights_layerwise``, ``/sleep``, ``/wake_up`` fan out to EVERY
  backend; the answer lists each backend's reply and the call fails if any backend failed (a weight update that reached
  only some engines must not look like a success).
* ``/health`` is 200 while at least one backend is healthy; ``/get_server_info`` and ``/metrics`` aggregate.

A backend that refuses a connection is marked unhealthy, skipped by the data plane, and probed again (``/health``) every
``probe_s`` seconds; a request that hit it is retried once on another backend.
"""

from __future__ import annotations

import json
import threading
import time
import urllib.error
import urllib.request
from concurrent.futures import ThreadPoolExecutor
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

_FANOUT = {"/pause", "/resume", "/update_weights", "/update_weights_layerwise", "/sleep", "/wake_up", "/reset_prefix_cache"}
_ONE = {"/generate", "/v1/completions", "/v1/chat/completions", "/v1/chat/completions/render"}


class Router:
    def __init__(self, backends: list[str], host: str = "127.0.0.1", port: int = 0, probe_s: float = 2.0, timeout_s: float = 3600.0):
        assert backends, "a router needs at least one backend"
        self.backends = [b.rstrip("/") for b in backends]
        self.healthy = {b: True for b in self.backends}
        self.inflight = {b: 0 for b in self.backends}
        self.served = {b: 0 for b in self.backends}
        self.sessions: dict[str, str] = {}
        self.probe_s, self.timeout_s = probe_s, timeout_s
        self._lock = threading.Lock()
        self._rr = 0
        self._stop = threading.Event()
        self._pool = ThreadPoolExecutor(max_workers=max(4, 2 * len(self.backends)))
        outer = self

        class H(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def _reply(self, code, obj, ctype="application/json"):
                body = obj if isinstance(obj, bytes) else json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Type", ctype)
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def do_GET(self):
                code, obj, ctype = outer.get(self.path)
                self._reply(code, obj, ctype)

            def do_POST(self):
                n = int(self.headers.get("Content-Length") or 0)
                try:
                    body = json.loads(self.rfile.read(n) or b"{}")
                except json.JSONDecodeError:
                    return self._reply(400, {"error": "body is not JSON"})
                code, obj = outer.post(self.path, body, self.headers.get("X-Session-Id"))
                self._reply(code, obj)

        self.httpd = ThreadingHTTPServer((host, port), H)
        self.httpd.daemon_threads = True
        self.url = "http://%s:%d" % self.httpd.server_address[:2]
        self._threads = [threading.Thread(target=self.httpd.serve_forever, daemon=True), threading.Thread(target=self._probe_loop, daemon=True)]

    def start(self) -> "Router":
        for t in self._threads:
            t.start()
        return self

    def shutdown(self) -> None:
        self._stop.set()
        self.httpd.shutdown()
        self.httpd.server_close()
        self._pool.shutdown(wait=False)

    # ------------------------------------------------------------------ backends
    def _call(self, backend: str, path: str, body: dict | None, method: str = "POST"):
        """(status code, decoded answer). Connection failures raise ConnectionError and mark the backend unhealthy."""
        data = json.dumps(body or {}).encode() if method == "POST" else None
        req = urllib.request.Request(backend + path, data=data, method=method, headers={"Content-Type": "application/json"})
        try:
            with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
                raw = r.read()
                return r.status, (json.loads(raw) if r.headers.get("Content-Type", "").startswith("application/json") else raw.decode())
        except urllib.error.HTTPError as e:
            raw = e.read()
            try:
                return e.code, json.loads(raw)
            except json.JSONDecodeError:
                return e.code, {"error": raw.decode(errors="replace")[:300]}
        except (urllib.error.URLError, ConnectionError, TimeoutError) as e:
            with self._lock:
                self.healthy[backend] = False
            raise ConnectionError(f"{backend}{path}: {e}") from None

    def _probe_loop(self) -> None:
        while not self._stop.wait(self.probe_s):
            for b in self.backends:
                if not self.healthy[b]:
                    try:
                        code, _ = self._call(b, "/health", None, "GET")
                        if code == 200:
                            with self._lock:
                                self.healthy[b] = True
                    except ConnectionError:
                        pass

    def _pick(self, session: str | None, exclude: set | None = None) -> str | None:
        with self._lock:
            live = [b for b in self.backends if self.healthy[b] and b not in (exclude or ())]
            if not live:
                return None
            if session is not None:
                pinned = self.sessions.get(session)
                if pinned in live:
                    return pinned
            self._rr += 1
            least = min(self.inflight[b] for b in live)
            cands = [b for b in live if self.inflight[b] == least]
            b = cands[self._rr % len(cands)]
            if session is not None:
                self.sessions[session] = b
            return b

    def _one(self, path: str, body: dict, session: str | None):
        tried: set = set()
        for _ in range(2):                                   # the first choice, then one other backend
            b = self._pick(session, tried)
            if b is None:
                break
            tried.add(b)
            with self._lock:
                self.inflight[b] += 1
            try:
                code, obj = self._call(b, path, body)
                with self._lock:
                    self.served[b] += 1
                return code, obj
            except ConnectionError:
                with self._lock:
                    if session is not None and self.sessions.get(session) == b:
                        del self.sessions[session]           # the conversation moves with its next turn
                continue
            finally:
                with self._lock:
                    self.inflight[b] -= 1
        return 503, {"error": "no healthy backend"}

    # ------------------------------------------------------------------ routes
    def post(self, path: str, body: dict, header_session: str | None = None):
        session = body.get("session_id", header_session)
        session = None if session is None else str(session)
        if path in _FANOUT:
            futs = {b: self._pool.submit(self._safe, b, path, body) for b in self.backends}
            res = {b: f.result() for b, f in futs.items()}
            ok = all(code == 200 for code, _ in res.values())
            return (200 if ok else 502), {"ok": ok, "backends": {b: {"status": c, "reply": o} for b, (c, o) in res.items()}}
        if path == "/generate" and session is None and isinstance(body.get("prompt_token_ids"), list) and len(body["prompt_token_ids"]) > 1 \
                and body.get("mm_features") is None:
            return self._split_generate(body)
        if path in _ONE:
            return self._one(path, body, session)
        return 404, {"error": f"no route {path}"}

    def _safe(self, b: str, path: str, body: dict):
        try:
            return self._call(b, path, body)
        except ConnectionError as e:
            return 503, {"error": str(e)}

    def _split_generate(self, body: dict):
        prompts = body["prompt_token_ids"]
        with self._lock:
            live = [b for b in self.backends if self.healthy[b]]
        if not live:
            return 503, {"error": "no healthy backend"}
        k = min(len(live), len(prompts))
        per = -(-len(prompts) // k)
        pieces = [(live[i], prompts[i * per:(i + 1) * per]) for i in range(k) if prompts[i * per:(i + 1) * per]]
        futs = [self._pool.submit(self._one, "/generate", dict(body, prompt_token_ids=p), None) for _, p in pieces]
        out: dict = {}
        for f in futs:
            code, obj = f.result()
            if code != 200:
                return code, obj
            for key, val in obj.items():
                if isinstance(val, list):
                    out.setdefault(key, []).extend(val)
                else:
                    out.setdefault(key, val)
        return 200, out

    def get(self, path: str):
        if path == "/health":
            n = sum(self.healthy.values())
            return (200 if n else 503), {"status": "ok" if n else "down", "healthy_backends": n, "backends": len(self.backends)}, "application/json"
        if path == "/get_server_info":
            infos = {}
            for b in self.backends:
                code, obj = self._safe_get(b, "/get_server_info")
                infos[b] = obj if code == 200 else {"error": obj}
            return 200, {"router": {"inflight": dict(self.inflight), "served": dict(self.served), "healthy": dict(self.healthy),
                                    "sessions": len(self.sessions)}, "backends": infos}, "application/json"
        if path == "/metrics":
            tot: dict = {}
            for b in self.backends:
                code, text = self._safe_get(b, "/metrics")
                if code != 200 or not isinstance(text, str):
                    continue
                for line in text.splitlines():
                    if line and not line.startswith("#"):
                        name, val = line.rsplit(" ", 1)
                        tot[name] = tot.get(name, 0.0) + float(val)
            lines = [f"{k} {v:g}" for k, v in sorted(tot.items())]
            lines += [f'router_requests_served{{backend="{b}"}} {n}' for b, n in self.served.items()]
            lines += [f'router_backend_healthy{{backend="{b}"}} {int(h)}' for b, h in self.healthy.items()]
            return 200, ("\n".join(lines) + "\n").encode(), "text/plain; version=0.0.4"
        return 404, {"error": f"no route {path}"}, "application/json"

    def _safe_get(self, b: str, path: str):
        try:
            return self._call(b, path, None, "GET")
        except ConnectionError as e:
            return 503, str(e)


def main(argv=None) -> None:
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--backends", required=True, help="comma-separated base URLs of the inference servers")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--probe-s", type=float, default=2.0)
    a = ap.parse_args(argv)
    r = Router([b for b in a.backends.split(",") if b], a.host, a.port, a.probe_s).start()
    print(f"router at {r.url} -> {len(r.backends)} backends", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        r.shutdown()


if __name__ == "__main__":
    main()
