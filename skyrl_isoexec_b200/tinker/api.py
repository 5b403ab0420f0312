"""HTTP front end of the Tinker-style API (reference: R/tinker/api.py FastAPI app + SQLModel tables, R/tinker/engine.py).

Every mutating call returns a ``request_id`` at once; the work is queued in a SQLite table (so queued requests
survive a restart of the front end) and executed in order by one engine thread; ``/api/v1/retrieve_future`` returns
``{status: pending|completed|failed, result}``.

  POST /api/v1/create_model        {base_model, model_overrides?, lr?, lora_config?: {rank, alpha}}   -> {model_id}
                                   (with ``lora_config`` the model is an ADAPTER: models created on the same base with the same
                                   overrides share one set of base weights, which never train; each trains its own factors)
  POST /api/v1/forward_backward    {model_id, data, loss_fn}
  POST /api/v1/forward             {model_id, data}
  POST /api/v1/optim_step          {model_id, adam_params}
  POST /api/v1/asample             {model_id, prompt_ids | chunks, num_samples, sampling_params}   (chunks: encoded_text / image)
  POST /api/v1/save_weights | load_weights {model_id, path}
  POST /api/v1/retrieve_future     {request_id}
  POST /api/v1/list_checkpoints    {model_id}                            -> every completed save of the model
  POST /api/v1/checkpoint_archive  {model_id, path}                      -> {archive_id, bytes, sha256}: a .tar.gz of the save
  GET  /api/v1/download/<archive_id>                                     -> the archive's bytes
  GET  /api/v1/telemetry                                                 -> per-verb counts / failures / latency, queue depth
  GET  /api/v1/healthz, /api/v1/get_server_capabilities
  REST-style forms of the same, with the reference's paths: GET / ; POST /api/v1/client/config ; GET /api/v1/samplers/<id> ;
  GET /api/v1/training_runs[/<model_id>] ; GET /api/v1/training_runs/<model_id>/checkpoints and /api/v1/models/<model_id>/checkpoints ;
  GET /api/v1/training_runs/<model_id>/checkpoints/<checkpoint>/archive | download (<checkpoint>: file name or index of the
  save) ; POST /api/v1/telemetry (events a client reports; stored, counted in GET /api/v1/telemetry)

A front end restarted on an existing database file reloads its models from their stored specs, re-applies the last
completed ``save_weights`` of each when the file is still there, and keeps queued requests; requests that were
pending for a model that cannot be rebuilt are marked failed with that reason
(reference: R/tinker/api.py:730-1375, checkpoint archive and download routes, request telemetry).
"""

from __future__ import annotations

import hashlib
import json
import os
import sqlite3
import tarfile
import tempfile
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from .backend import LOSS_FNS, SkyRLTrainBackend

_ROUTES = {"forward_backward": "forward_backward", "forward": "forward", "optim_step": "optim_step", "asample": "sample",
           "save_weights": "save_weights", "load_weights": "load_weights", "save_weights_for_sampler": "save_weights_for_sampler"}


class TinkerServer:
    def __init__(self, db_path: str = ":memory:", host: str = "127.0.0.1", port: int = 0, device: str | None = None):
        self.db = sqlite3.connect(db_path, check_same_thread=False)
        self.db.execute("create table if not exists futures (id text primary key, seq integer, model_id text, payload text, "
                        "status text, result text, created real)")
        self.db.execute("create table if not exists models (id text primary key, spec text)")
        self.db.execute("create table if not exists sessions (id text primary key, kind text, model_id text, meta text, "
                        "created real, heartbeat real)")
        self.db.execute("create table if not exists checkpoints (model_id text, path text, kind text, step integer, bytes integer, "
                        "created real)")
        self.db.execute("create table if not exists archives (id text primary key, model_id text, src text, file text, bytes integer, "
                        "sha256 text, created real)")
        self.db.execute("create table if not exists client_events (session_id text, name text, payload text, created real)")
        cols = [r[1] for r in self.db.execute("pragma table_info(futures)")]
        if "finished" not in cols:
            self.db.execute("alter table futures add column finished real")
        self._dblock = threading.Lock()
        self.device = device
        self.models: dict[str, SkyRLTrainBackend] = {}
        self.shared_bases: dict[str, SkyRLTrainBackend] = {}     # (base model, overrides, seed) -> the backend its adapters share
        self.adapter_of: dict[str, str] = {}                     # adapter model id -> key of its shared base
        self._stop = threading.Event()
        self._wake = threading.Event()
        self._seq = int(self.db.execute("select coalesce(max(seq), 0) from futures").fetchone()[0])
        self.recovered = self._recover()
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
                if self.path == "/api/v1/healthz":
                    return self._reply(200, {"status": "ok"})
                if self.path == "/api/v1/get_server_capabilities":
                    from ..models.config import PRESETS

                    return self._reply(200, {"supported_models": sorted(PRESETS), "loss_fns": sorted(LOSS_FNS)})
                if self.path == "/api/v1/telemetry":
                    return self._reply(200, outer.telemetry())
                if self.path == "/":
                    return self._reply(200, {"name": "skyrl_isoexec_b200 tinker API", "api": "/api/v1", "models": len(outer.models)})
                rest = outer.rest_get(self.path)
                if rest is not None:
                    kind, val = rest
                    if kind == "json":
                        return self._reply(200, val)
                    if kind == "missing":
                        return self._reply(404, {"error": val})
                    self.path = "/api/v1/download/" + val          # kind == "download": stream the archive below
                if self.path.startswith("/api/v1/download/"):
                    f = outer.archive_file(self.path.rsplit("/", 1)[-1])
                    if f is None:
                        return self._reply(404, {"error": "unknown archive"})
                    self.send_response(200)
                    self.send_header("Content-Type", "application/gzip")
                    self.send_header("Content-Length", str(os.path.getsize(f)))
                    self.end_headers()
                    with open(f, "rb") as fh:
                        while True:
                            buf = fh.read(1 << 20)
                            if not buf:
                                break
                            self.wfile.write(buf)
                    return None
                self._reply(404, {"error": "no route"})

            def do_POST(self):
                n = int(self.headers.get("Content-Length") or 0)
                try:
                    body = json.loads(self.rfile.read(n) or b"{}")
                    self._reply(200, outer.post(self.path, body))
                except KeyError as e:
                    self._reply(404, {"error": f"unknown {e}"})
                except Exception as e:  # noqa: BLE001
                    self._reply(400, {"error": f"{type(e).__name__}: {e}"})

        self.httpd = ThreadingHTTPServer((host, port), H)
        self.httpd.daemon_threads = True
        self.url = "http://%s:%d" % self.httpd.server_address[:2]
        self._threads = [threading.Thread(target=self.httpd.serve_forever, daemon=True), threading.Thread(target=self._loop, daemon=True)]

    def start(self):
        for t in self._threads:
            t.start()
        return self

    def shutdown(self):
        self._stop.set()
        self._wake.set()
        self.httpd.shutdown()
        self.httpd.server_close()

    # ------------------------------------------------------------------ restart, checkpoints, telemetry
    def _recover(self) -> dict:
        """Rebuild the models a previous front end left in the database; fail what cannot continue."""
        out = {"models": [], "failed_requests": 0}
        for mid, spec in self.db.execute("select id, spec from models").fetchall():
            sp = json.loads(spec)
            try:
                if sp.get("lora_config"):
                    self._add_adapter(mid, sp)
                    b = self.models[mid]
                else:
                    b = SkyRLTrainBackend(sp["base_model"], sp["model_overrides"], self.device, sp["lr"], sp["seed"])
                last = self.db.execute("select path from checkpoints where model_id = ? and kind = 'save_weights' order by created desc limit 1",
                                       (mid,)).fetchone()
                if last and os.path.exists(last[0]):
                    b.handle({"type": "load_weights", "path": last[0], **({"tenant": mid} if sp.get("lora_config") else {})})
                self.models[mid] = b
                out["models"].append(mid)
            except Exception as e:  # noqa: BLE001
                cur = self.db.execute("update futures set status = 'failed', result = ?, finished = ? where model_id = ? and status = 'pending'",
                                      (json.dumps({"error": f"front end restarted and the model could not be rebuilt: {type(e).__name__}: {e}"}),
                                       time.time(), mid))
                out["failed_requests"] += cur.rowcount
        self.db.commit()
        return out

    def _checkpoint_of(self, model_id: str, ref: str) -> str | None:
        """A recorded save of the model named by its file / directory name or by its index in save order."""
        with self._dblock:
            rows = [r[0] for r in self.db.execute("select path from checkpoints where model_id = ? order by created", (model_id,))]
        if ref.lstrip("-").isdigit() and -len(rows) <= int(ref) < len(rows):
            return rows[int(ref)]
        for p_ in reversed(rows):
            if os.path.basename(p_.rstrip("/")) == ref:
                return p_
        return None

    def rest_get(self, path: str):
        """The reference's REST paths. Returns None (not one of them), ("json", obj), ("missing", why) or ("download", archive id)."""
        parts = [x for x in path.split("?")[0].split("/") if x]
        if parts[:2] != ["api", "v1"]:
            return None
        parts = parts[2:]
        try:
            if parts == ["training_runs"]:
                return "json", self.post("/api/v1/training_runs", {})
            if len(parts) == 2 and parts[0] == "training_runs":
                runs = [r for r in self.post("/api/v1/training_runs", {})["training_runs"] if r["model_id"] == parts[1]]
                return ("json", runs[0]) if runs else ("missing", f"no training run {parts[1]!r}")
            if len(parts) == 3 and parts[0] in ("training_runs", "models") and parts[2] == "checkpoints":
                return "json", self.post("/api/v1/list_checkpoints", {"model_id": parts[1]})
            if len(parts) == 5 and parts[0] == "training_runs" and parts[2] == "checkpoints" and parts[4] in ("archive", "download"):
                ck = self._checkpoint_of(parts[1], parts[3])
                if ck is None:
                    return "missing", f"no checkpoint {parts[3]!r} of {parts[1]!r}"
                arc = self.post("/api/v1/checkpoint_archive", {"model_id": parts[1], "path": ck})
                return ("json", arc) if parts[4] == "archive" else ("download", arc["archive_id"])
            if len(parts) == 2 and parts[0] == "samplers":
                with self._dblock:
                    row = self.db.execute("select model_id, meta, created, heartbeat from sessions where id = ? and kind = 'sampling_session'",
                                          (parts[1],)).fetchone()
                if row is None:
                    return "missing", f"no sampler {parts[1]!r}"
                b = self.models.get(row[0])
                return "json", {"sampler_id": parts[1], "model_id": row[0], "created": row[2], "heartbeat": row[3], **json.loads(row[1]),
                                "sampler_version": getattr(b, "sampler_version", 0) if b is not None else None}
        except KeyError as e:
            return "missing", f"unknown {e}"
        return None

    def archive_file(self, archive_id: str) -> str | None:
        with self._dblock:
            row = self.db.execute("select file from archives where id = ?", (archive_id,)).fetchone()
        return row[0] if row and os.path.exists(row[0]) else None

    def telemetry(self) -> dict:
        with self._dblock:
            rows = self.db.execute("select payload, status, created, finished from futures").fetchall()
            sessions = self.db.execute("select count(*) from sessions").fetchone()[0]
        per: dict = {}
        for payload, status, created, finished in rows:
            kind = json.loads(payload).get("type", "?")
            d = per.setdefault(kind, {"count": 0, "pending": 0, "failed": 0, "latency_s_sum": 0.0, "latency_s_max": 0.0})
            d["count"] += 1
            d["pending"] += status == "pending"
            d["failed"] += status == "failed"
            if finished:
                d["latency_s_sum"] += finished - created
                d["latency_s_max"] = max(d["latency_s_max"], finished - created)
        with self._dblock:
            events = dict(self.db.execute("select name, count(*) from client_events group by name").fetchall())
        return {"requests": per, "queue_depth": sum(d["pending"] for d in per.values()), "models": len(self.models), "sessions": sessions,
                "client_events": events}

    # ------------------------------------------------------------------ front end
    def post(self, path: str, body: dict) -> dict:
        verb = path.rsplit("/", 1)[-1]
        if path.endswith("/client/config"):
            return {"poll_interval_s": 0.01, "request_timeout_s": 600.0, "future_retention": "database", "api_prefix": "/api/v1"}
        if verb == "telemetry":
            evs = body.get("events") or ([body] if body.get("name") else [])
            with self._dblock:
                for ev in evs:
                    self.db.execute("insert into client_events values (?, ?, ?, ?)",
                                    (body.get("session_id"), str(ev.get("name", "event")), json.dumps(ev), time.time()))
                self.db.commit()
            return {"status": "accepted", "events": len(evs)}
        if verb == "list_checkpoints":
            with self._dblock:
                rows = self.db.execute("select path, kind, step, bytes, created from checkpoints where model_id = ? order by created",
                                       (body["model_id"],)).fetchall()
            return {"checkpoints": [dict(path=p_, kind=k, step=st, bytes=b, created=c, exists=os.path.exists(p_)) for p_, k, st, b, c in rows]}
        if verb == "checkpoint_archive":
            with self._dblock:
                known = self.db.execute("select 1 from checkpoints where model_id = ? and path = ?", (body["model_id"], body["path"])).fetchone()
            if not known or not os.path.exists(body["path"]):
                raise KeyError(f"checkpoint {body['path']!r} of {body['model_id']!r}")       # only recorded saves are served
            aid = "arc-" + uuid.uuid4().hex[:12]
            fd, tmp = tempfile.mkstemp(prefix=aid + "-", suffix=".tar.gz")
            os.close(fd)
            with tarfile.open(tmp, "w:gz") as tf:
                tf.add(body["path"], arcname=os.path.basename(body["path"].rstrip("/")))
            h = hashlib.sha256()
            with open(tmp, "rb") as fh:
                for buf in iter(lambda: fh.read(1 << 20), b""):
                    h.update(buf)
            size = os.path.getsize(tmp)
            with self._dblock:
                self.db.execute("insert into archives values (?, ?, ?, ?, ?, ?, ?)", (aid, body["model_id"], body["path"], tmp, size, h.hexdigest(), time.time()))
                self.db.commit()
            return {"archive_id": aid, "bytes": size, "sha256": h.hexdigest(), "download": f"/api/v1/download/{aid}"}
        # ---- sessions: bookkeeping only (who is connected, which sampler weights a sampling session reads)
        if verb in ("create_session", "create_sampling_session"):
            if verb == "create_sampling_session" and body.get("model_id") not in self.models:
                raise KeyError(f"model_id {body.get('model_id')!r}")
            sid = ("sess-" if verb == "create_session" else "samp-") + uuid.uuid4().hex[:10]
            now = time.time()
            with self._dblock:
                self.db.execute("insert into sessions values (?, ?, ?, ?, ?, ?)",
                                (sid, verb[len("create_"):], body.get("model_id"), json.dumps({k: v for k, v in body.items() if k != "model_id"}), now, now))
                self.db.commit()
            return {"session_id": sid}
        if verb == "session_heartbeat":
            with self._dblock:
                cur = self.db.execute("update sessions set heartbeat = ? where id = ?", (time.time(), body["session_id"]))
                self.db.commit()
            if cur.rowcount == 0:
                raise KeyError(body["session_id"])
            return {"ok": True}
        if verb == "get_info":
            if body.get("model_id") not in self.models:
                raise KeyError(f"model_id {body.get('model_id')!r}")
            with self._dblock:
                spec = json.loads(self.db.execute("select spec from models where id = ?", (body["model_id"],)).fetchone()[0])
                pending = self.db.execute("select count(*) from futures where model_id = ? and status = 'pending'", (body["model_id"],)).fetchone()[0]
            b = self.models[body["model_id"]]
            return {"model_id": body["model_id"], "spec": spec, "step": b.step_count, "pending_requests": pending,
                    "num_parameters": int(b.model.store.flat.numel()), "sampler_version": getattr(b, "sampler_version", 0)}
        if verb == "unload_model":
            if body.get("model_id") not in self.models:
                raise KeyError(f"model_id {body.get('model_id')!r}")
            with self._dblock:
                busy = self.db.execute("select count(*) from futures where model_id = ? and status = 'pending'", (body["model_id"],)).fetchone()[0]
            if busy:
                raise RuntimeError(f"{busy} requests of {body['model_id']} are still pending")
            del self.models[body["model_id"]]
            with self._dblock:
                self.db.execute("delete from models where id = ?", (body["model_id"],))
                self.db.commit()
            return {"unloaded": body["model_id"]}
        if verb == "training_runs":
            with self._dblock:
                rows = self.db.execute("select id, spec from models").fetchall()
            return {"training_runs": [{"model_id": i, "spec": json.loads(sp), "step": self.models[i].step_count} for i, sp in rows if i in self.models]}
        if verb == "weights_info":
            import torch

            sd = torch.load(body["path"], weights_only=False, map_location="cpu")
            return {"path": body["path"], "step": int(sd.get("step", 0)), "num_tensors": len(sd["model"]),
                    "num_parameters": int(sum(v.numel() for v in sd["model"].values())), "has_optimizer": sd.get("optimizer") is not None}
        if verb == "create_model":
            mid = "model-" + uuid.uuid4().hex[:10]
            spec = {"base_model": body.get("base_model", "tiny-qwen3"), "model_overrides": body.get("model_overrides") or {},
                    "lr": body.get("lr", 1e-5), "seed": body.get("seed", 0)}
            lora = body.get("lora_config") or None
            if lora and int(lora.get("rank", 0)) > 0:
                spec["lora_config"] = {"rank": int(lora["rank"]), "alpha": float(lora.get("alpha", 16.0))}
                self._add_adapter(mid, spec)
            else:
                self.models[mid] = SkyRLTrainBackend(spec["base_model"], spec["model_overrides"], self.device, spec["lr"], spec["seed"])
            with self._dblock:
                self.db.execute("insert into models values (?, ?)", (mid, json.dumps(spec)))
                self.db.commit()
            return {"model_id": mid}
        if verb == "retrieve_future":
            with self._dblock:
                row = self.db.execute("select status, result from futures where id = ?", (body["request_id"],)).fetchone()
            if row is None:
                raise KeyError(body["request_id"])
            return {"status": row[0], "result": json.loads(row[1]) if row[1] else None}
        if verb not in _ROUTES:
            raise KeyError(path)
        if body.get("model_id") not in self.models:
            raise KeyError(f"model_id {body.get('model_id')!r}")
        rid = "req-" + uuid.uuid4().hex[:12]
        payload = dict(body, type=_ROUTES[verb])
        if body["model_id"] in self.adapter_of:
            payload["tenant"] = body["model_id"]
        with self._dblock:
            self._seq += 1
            self.db.execute("insert into futures (id, seq, model_id, payload, status, result, created) values (?, ?, ?, ?, 'pending', null, ?)",
                            (rid, self._seq, body["model_id"], json.dumps(payload), time.time()))
            self.db.commit()
        self._wake.set()
        return {"request_id": rid}

    def _add_adapter(self, mid: str, spec: dict) -> None:
        """An adapter model: it lives on the shared backend of its (base model, overrides, seed); the first one builds it."""
        key = json.dumps([spec["base_model"], spec["model_overrides"], spec["seed"]], sort_keys=True)
        if key not in self.shared_bases:
            self.shared_bases[key] = SkyRLTrainBackend(spec["base_model"], spec["model_overrides"], self.device, spec["lr"], spec["seed"])
        be = self.shared_bases[key]
        be.add_tenant(mid, spec["lora_config"]["rank"], spec["lora_config"]["alpha"], lr=spec["lr"], seed=len(be.tenants))
        self.models[mid] = be
        self.adapter_of[mid] = key

    # ------------------------------------------------------------------ engine loop: strictly in arrival order
    def _loop(self) -> None:
        while not self._stop.is_set():
            with self._dblock:
                row = self.db.execute("select id, model_id, payload from futures where status = 'pending' order by seq limit 1").fetchone()
            if row is None:
                self._wake.wait(0.05)
                self._wake.clear()
                continue
            rid, mid, payload = row
            req = json.loads(payload)
            try:
                res, status = self.models[mid].handle(req), "completed"
            except Exception as e:  # noqa: BLE001
                res, status = {"error": f"{type(e).__name__}: {e}"}, "failed"
            with self._dblock:
                self.db.execute("update futures set status = ?, result = ?, finished = ? where id = ?", (status, json.dumps(res), time.time(), rid))
                if status == "completed" and req["type"] in ("save_weights", "save_weights_for_sampler") and req.get("path"):
                    p_ = req["path"]
                    size = os.path.getsize(p_) if os.path.isfile(p_) else sum(
                        os.path.getsize(os.path.join(d, f)) for d, _, fs in os.walk(p_) for f in fs) if os.path.exists(p_) else 0
                    self.db.execute("insert into checkpoints values (?, ?, ?, ?, ?, ?)",
                                    (mid, p_, req["type"], int(self.models[mid].step_count), int(size), time.time()))
                self.db.commit()


class TinkerClient:
    """Blocking convenience client (stdlib only)."""

    def __init__(self, url: str, poll_s: float = 0.01, timeout_s: float = 600.0):
        self.url, self.poll_s, self.timeout_s = url, poll_s, timeout_s

    def _post(self, verb: str, body: dict) -> dict:
        import urllib.error
        import urllib.request

        req = urllib.request.Request(f"{self.url}/api/v1/{verb}", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
        try:
            with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
                return json.loads(r.read())
        except urllib.error.HTTPError as e:
            raise RuntimeError(f"{verb}: HTTP {e.code}: {e.read().decode(errors='replace')[:300]}") from None

    def create_model(self, **kw) -> str:
        return self._post("create_model", kw)["model_id"]

    def submit(self, verb: str, **body) -> str:
        return self._post(verb, body)["request_id"]

    def result(self, request_id: str) -> dict:
        t0 = time.time()
        while time.time() - t0 < self.timeout_s:
            r = self._post("retrieve_future", {"request_id": request_id})
            if r["status"] == "completed":
                return r["result"]
            if r["status"] == "failed":
                raise RuntimeError(r["result"]["error"])
            time.sleep(self.poll_s)
        raise TimeoutError(request_id)

    def call(self, verb: str, **body) -> dict:
        return self.result(self.submit(verb, **body))


def main(argv=None) -> None:
    """``python -m skyrl_isoexec_b200.tinker.api [--host 127.0.0.1] [--port 8000] [--db tinker.db] [--device cuda]``"""
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--db", default=":memory:")
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    srv = TinkerServer(db_path=a.db, host=a.host, port=a.port, device=a.device).start()
    print(f"tinker API at {srv.url}/api/v1", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.shutdown()


if __name__ == "__main__":
    main()
