"""Tinker-style API end to end on CPU: futures, ordering, a supervised step that lowers the loss, sampling,
RL-style importance-sampling update, save / load."""
import pytest
import torch

from skyrl_isoexec_b200.tinker.api import TinkerClient, TinkerServer


def test_tinker_training_loop_over_http(tmp_path):
    srv = TinkerServer(db_path=str(tmp_path / "q.db"), device="cpu").start()
    try:
        cl = TinkerClient(srv.url)
        mid = cl.create_model(base_model="tiny-qwen3", lr=3e-3)
        g = torch.Generator().manual_seed(0)
        data = [{"prompt_ids": torch.randint(0, 500, (5,), generator=g).tolist(),
                 "response_ids": torch.randint(0, 500, (8,), generator=g).tolist()} for _ in range(4)]
        # queue several requests before any result is read: they run in order
        ids = []
        for _ in range(4):
            ids.append(cl.submit("forward_backward", model_id=mid, data=data, loss_fn="cross_entropy"))
            ids.append(cl.submit("optim_step", model_id=mid, adam_params={"learning_rate": 3e-3}))
        res = [cl.result(i) for i in ids]
        losses = [r["loss"] for r in res[0::2]]
        assert [r["step"] for r in res[1::2]] == [1, 2, 3, 4] and losses[-1] < losses[0]
        assert res[0]["num_tokens"] == 32
        # sample, then an RL update on the samples with their own logprobs (ratio 1 at the start)
        s = cl.call("asample", model_id=mid, prompt_ids=data[0]["prompt_ids"], num_samples=3,
                    sampling_params={"max_generate_length": 6, "ignore_eos": True})
        assert len(s["sequences"]) == 3 and all(len(x["tokens"]) == 6 and len(x["logprobs"]) == 6 for x in s["sequences"])
        rl = [{"prompt_ids": data[0]["prompt_ids"], "response_ids": x["tokens"], "logprobs": x["logprobs"], "advantages": a}
              for x, a in zip(s["sequences"], (1.0, -0.5, 0.25))]
        fwd = cl.call("forward", model_id=mid, data=rl)
        assert fwd["logprobs"] == [x["logprobs"] for x in s["sequences"]]            # engine == trainer, bit for bit
        out = cl.call("forward_backward", model_id=mid, data=rl, loss_fn="importance_sampling")
        assert abs(out["loss"] - (-(1.0 - 0.5 + 0.25) * 6)) < 1e-4                    # sum of -ratio*A with ratio == 1
        path = str(tmp_path / "w" / "ckpt.pt")
        cl.call("save_weights", model_id=mid, path=path)
        cl.call("optim_step", model_id=mid, adam_params={})
        assert cl.call("load_weights", model_id=mid, path=path)["step"] == 4
        # sessions, sampler publication, introspection
        sess = cl._post("create_session", {"user": "t"})["session_id"]
        assert cl._post("session_heartbeat", {"session_id": sess})["ok"]
        samp = cl._post("create_sampling_session", {"model_id": mid, "base": "latest"})["session_id"]
        assert sess.startswith("sess-") and samp.startswith("samp-")
        pub = cl.call("save_weights_for_sampler", model_id=mid, path=str(tmp_path / "w" / "sampler.pt"))
        assert pub["sampler_version"] == 1 and pub["step"] == 4
        info = cl._post("get_info", {"model_id": mid})
        assert info["step"] == 4 and info["sampler_version"] == 1 and info["pending_requests"] == 0 and info["num_parameters"] > 0
        wi = cl._post("weights_info", {"path": path})
        assert wi["step"] == 4 and wi["has_optimizer"] and wi["num_parameters"] > 0
        assert not cl._post("weights_info", {"path": pub["path"]})["has_optimizer"]
        assert [r["model_id"] for r in cl._post("training_runs", {})["training_runs"]] == [mid]
        with pytest.raises(RuntimeError, match="loss_fn"):
            cl.call("forward_backward", model_id=mid, data=rl, loss_fn="nope")
        with pytest.raises(RuntimeError, match="404"):
            cl.submit("optim_step", model_id="model-missing")
        assert cl._post("unload_model", {"model_id": mid})["unloaded"] == mid
        assert cl._post("training_runs", {})["training_runs"] == []
        with pytest.raises(RuntimeError, match="404"):
            cl._post("get_info", {"model_id": mid})
    finally:
        srv.shutdown()


def test_tinker_checkpoint_archive_download_telemetry_and_restart(tmp_path):
    """Saves are recorded, can be packed and downloaded; telemetry counts requests; a front end restarted on the same
    database file rebuilds the model from its last save and keeps serving it."""
    import hashlib
    import io
    import json
    import tarfile
    import urllib.request

    db = str(tmp_path / "t.db")
    srv = TinkerServer(db_path=db, device="cpu").start()
    try:
        cl = TinkerClient(srv.url)
        mid = cl.create_model(base_model="tiny-qwen3", lr=3e-3)
        data = [{"prompt_ids": [5, 6, 7], "response_ids": [8, 9, 10, 11]}]
        cl.call("forward_backward", model_id=mid, data=data, loss_fn="cross_entropy")
        cl.call("optim_step", model_id=mid)
        path = str(tmp_path / "w1.pt")
        cl.call("save_weights", model_id=mid, path=path)
        want = cl.call("forward", model_id=mid, data=data)["logprobs"]
        cks = cl._post("list_checkpoints", {"model_id": mid})["checkpoints"]
        assert len(cks) == 1 and cks[0]["path"] == path and cks[0]["step"] == 1 and cks[0]["bytes"] > 0 and cks[0]["exists"]
        with pytest.raises(RuntimeError):
            cl._post("checkpoint_archive", {"model_id": mid, "path": str(tmp_path / "not_a_save.pt")})     # only recorded saves are served
        arc = cl._post("checkpoint_archive", {"model_id": mid, "path": path})
        with urllib.request.urlopen(srv.url + arc["download"]) as r:
            blob = r.read()
        assert len(blob) == arc["bytes"] and hashlib.sha256(blob).hexdigest() == arc["sha256"]
        with tarfile.open(fileobj=io.BytesIO(blob), mode="r:gz") as tf:
            assert tf.getnames() == ["w1.pt"]
        with urllib.request.urlopen(srv.url + "/api/v1/telemetry") as r:
            tel = json.loads(r.read())
        assert tel["requests"]["forward_backward"]["count"] == 1 and tel["requests"]["save_weights"]["failed"] == 0
        assert tel["queue_depth"] == 0 and tel["models"] == 1 and tel["requests"]["optim_step"]["latency_s_max"] > 0
    finally:
        srv.shutdown()
    srv2 = TinkerServer(db_path=db, device="cpu").start()
    try:
        assert srv2.recovered["models"] == [mid]
        cl2 = TinkerClient(srv2.url)
        got = cl2.call("forward", model_id=mid, data=data)["logprobs"]
        assert got == want                                   # the rebuilt model carries the saved weights
        info = cl2._post("get_info", {"model_id": mid})
        assert info["step"] == 1
    finally:
        srv2.shutdown()


def test_tinker_rest_paths_of_the_reference(tmp_path):
    """The REST-style routes: runs, checkpoints by name or index with archive / download, sampler lookup, client config,
    client-reported telemetry."""
    import io
    import json
    import tarfile
    import urllib.error
    import urllib.request

    srv = TinkerServer(db_path=str(tmp_path / "r.db"), device="cpu").start()

    def get(path):
        with urllib.request.urlopen(srv.url + path, timeout=60) as r:
            raw = r.read()
            return json.loads(raw) if r.headers.get("Content-Type", "").startswith("application/json") else raw

    try:
        cl = TinkerClient(srv.url)
        mid = cl.create_model(base_model="tiny-qwen3")
        cl.call("save_weights", model_id=mid, path=str(tmp_path / "a.pt"))
        cl.call("save_weights", model_id=mid, path=str(tmp_path / "b.pt"))
        assert get("/")["models"] == 1
        assert [r["model_id"] for r in get("/api/v1/training_runs")["training_runs"]] == [mid]
        assert get(f"/api/v1/training_runs/{mid}")["model_id"] == mid
        cks = get(f"/api/v1/training_runs/{mid}/checkpoints")["checkpoints"]
        assert [c["path"].rsplit("/", 1)[-1] for c in cks] == ["a.pt", "b.pt"] == [c["path"].rsplit("/", 1)[-1] for c in get(f"/api/v1/models/{mid}/checkpoints")["checkpoints"]]
        arc = get(f"/api/v1/training_runs/{mid}/checkpoints/b.pt/archive")
        blob = get(f"/api/v1/training_runs/{mid}/checkpoints/-1/download")            # the last save, by index
        with tarfile.open(fileobj=io.BytesIO(blob), mode="r:gz") as tf:
            assert tf.getnames() == ["b.pt"]
        assert arc["bytes"] > 0 and arc["download"].startswith("/api/v1/download/")
        with pytest.raises(urllib.error.HTTPError):
            get(f"/api/v1/training_runs/{mid}/checkpoints/zzz.pt/archive")
        sid = cl._post("create_sampling_session", {"model_id": mid, "base_model": "tiny-qwen3"})["session_id"]
        smp = get(f"/api/v1/samplers/{sid}")
        assert smp["model_id"] == mid and smp["sampler_version"] == 0
        assert cl._post("client/config", {})["api_prefix"] == "/api/v1"
        assert cl._post("telemetry", {"session_id": sid, "events": [{"name": "step"}, {"name": "step"}, {"name": "error", "msg": "x"}]})["events"] == 3
        assert get("/api/v1/telemetry")["client_events"] == {"step": 2, "error": 1}
    finally:
        srv.shutdown()


def test_tinker_adapters_share_one_base_and_train_apart(tmp_path):
    """Multi-tenant LoRA: two adapter models on one base. Each trains its own factors, each samples under its own merged
    weights, the base never moves, and an adapter's save / load brings its factors back."""
    srv = TinkerServer(db_path=str(tmp_path / "q.db"), device="cpu").start()
    try:
        cl = TinkerClient(srv.url)
        a = cl.create_model(base_model="tiny-qwen3", lr=2e-2, lora_config={"rank": 4, "alpha": 8})
        b = cl.create_model(base_model="tiny-qwen3", lr=2e-2, lora_config={"rank": 2})
        full = cl.create_model(base_model="tiny-qwen3", lr=1e-3)                        # an ordinary model beside them
        be = srv.models[a]
        assert srv.models[b] is be and srv.models[full] is not be and set(be.tenants) == {a, b}
        base0 = {n: t.clone() for n, t in be.model.named_weights()}
        g = torch.Generator().manual_seed(0)
        data = [{"prompt_ids": torch.randint(0, 500, (5,), generator=g).tolist(),
                 "response_ids": torch.randint(0, 500, (8,), generator=g).tolist()} for _ in range(4)]
        prompt = data[0]["prompt_ids"]
        sp = {"max_generate_length": 5, "ignore_eos": True, "temperature": 0.0}
        before = cl.call("asample", model_id=a, prompt_ids=prompt, num_samples=1, sampling_params=sp)["sequences"][0]
        losses = []
        for _ in range(4):                                                              # only adapter a trains
            losses.append(cl.call("forward_backward", model_id=a, data=data, loss_fn="cross_entropy")["loss"])
            assert cl.call("optim_step", model_id=a, adam_params={})["step"] == len(losses)
        assert losses[-1] < losses[0]
        after_a = cl.call("asample", model_id=a, prompt_ids=prompt, num_samples=1, sampling_params=sp)["sequences"][0]
        same_b = cl.call("asample", model_id=b, prompt_ids=prompt, num_samples=1, sampling_params=sp)["sequences"][0]
        assert after_a["logprobs"] != before["logprobs"]                                # a's policy moved
        assert same_b["logprobs"] == before["logprobs"]                                 # b still is the base (its B factors are zero)
        # sampling under an adapter and scoring under it agree bit for bit (the adapter is merged for both)
        fwd = cl.call("forward", model_id=a, data=[{"prompt_ids": prompt, "response_ids": after_a["tokens"]}])
        assert fwd["logprobs"][0] == after_a["logprobs"]
        # the base weights are untouched once no adapter is merged
        be.store.deactivate()
        assert all(torch.equal(t, base0[n]) for n, t in be.model.named_weights())
        # save, train on, load: the factors come back
        path = str(tmp_path / "a.pt")
        cl.call("save_weights", model_id=a, path=path)
        cl.call("forward_backward", model_id=a, data=data, loss_fn="cross_entropy")
        cl.call("optim_step", model_id=a, adam_params={"learning_rate": 5e-2})
        moved = cl.call("asample", model_id=a, prompt_ids=prompt, num_samples=1, sampling_params=sp)["sequences"][0]
        assert cl.call("load_weights", model_id=a, path=path)["step"] == 4
        back = cl.call("asample", model_id=a, prompt_ids=prompt, num_samples=1, sampling_params=sp)["sequences"][0]
        assert back["logprobs"] == after_a["logprobs"] and moved["logprobs"] != after_a["logprobs"]
    finally:
        srv.shutdown()
    # a restarted front end rebuilds the shared base and both adapters, with a's last save applied
    srv2 = TinkerServer(db_path=str(tmp_path / "q.db"), device="cpu").start()
    try:
        assert srv2.models[a] is srv2.models[b] and set(srv2.models[a].tenants) == {a, b}
        cl2 = TinkerClient(srv2.url)
        again = cl2.call("asample", model_id=a, prompt_ids=prompt, num_samples=1, sampling_params=sp)["sequences"][0]
        assert again["logprobs"] == after_a["logprobs"]
    finally:
        srv2.shutdown()
