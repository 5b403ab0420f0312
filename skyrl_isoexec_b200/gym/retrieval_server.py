"""A retrieval server for the search environments (the reference's examples start a dense or BM25 retriever behind
``POST /retrieve`` and point ``environment.skyrl_gym.search.search_url`` at it; this is the BM25 one, dependency-free):

    python -m skyrl_isoexec_b200.gym.retrieval_server --corpus corpus.jsonl [--host 127.0.0.1] [--port 8000]

``corpus.jsonl`` has one document per line, either a JSON string or an object with ``contents`` (or ``text``; an optional
``title`` is put in front). Request: ``{"query": str | [str, ...], "topk": 3, "return_scores": true}``; answer:
``{"result": [[{"document": {"id", "contents"}, "score"}, ...], ...]}``, one list per query.
"""

from __future__ import annotations

import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from .tools import SearchToolGroup


def load_corpus(path: str) -> list[str]:
    docs = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            if not line.strip():
                continue
            d = json.loads(line)
            if isinstance(d, str):
                docs.append(d)
            else:
                body = d.get("contents") or d.get("text") or ""
                docs.append((d["title"] + "\n" + body) if d.get("title") else body)
    return docs


class RetrievalServer:
    def __init__(self, corpus: list[str], host: str = "127.0.0.1", port: int = 0):
        self.index = SearchToolGroup(corpus)
        self.requests = 0
        self.fail_next = 0                  # tests: answer this many requests with 503 first
        outer = self

        class H(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def _reply(self, code, obj):
                body = json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def do_GET(self):
                self._reply(200 if self.path == "/health" else 404, {"status": "ok", "documents": len(outer.index.docs)})

            def do_POST(self):
                n = int(self.headers.get("Content-Length") or 0)
                raw = self.rfile.read(n)
                outer.requests += 1
                if outer.fail_next > 0:
                    outer.fail_next -= 1
                    return self._reply(503, {"error": "busy"})
                if self.path != "/retrieve":
                    return self._reply(404, {"error": f"no route {self.path}"})
                try:
                    body = json.loads(raw or b"{}")
                    queries = body["query"] if isinstance(body["query"], list) else [body["query"]]
                    topk = int(body.get("topk", 3))
                except (KeyError, ValueError, TypeError) as e:
                    return self._reply(400, {"error": f"bad request: {e}"})
                out = []
                for q in queries:
                    hits = outer.index.search(str(q), topk)
                    out.append([dict({"document": {"id": h["doc_id"], "contents": h["text"]}},
                                     **({"score": h["score"]} if body.get("return_scores", True) else {})) for h in hits])
                self._reply(200, {"result": out})

        self.httpd = ThreadingHTTPServer((host, port), H)
        self.httpd.daemon_threads = True
        self.url = "http://%s:%d/retrieve" % self.httpd.server_address[:2]
        self._thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)

    def start(self) -> "RetrievalServer":
        self._thread.start()
        return self

    def shutdown(self) -> None:
        self.httpd.shutdown()
        self.httpd.server_close()


def main(argv=None) -> None:
    import argparse
    import time

    ap = argparse.ArgumentParser()
    ap.add_argument("--corpus", required=True)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    a = ap.parse_args(argv)
    srv = RetrievalServer(load_corpus(a.corpus), a.host, a.port).start()
    print(f"retrieval server at {srv.url} over {len(srv.index.docs)} documents", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.shutdown()


if __name__ == "__main__":
    main()
