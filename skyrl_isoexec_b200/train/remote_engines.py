"""The trainer's rollouts on inference servers it does not own (reference: the remote inference engines of
R/backends/skyrl_train/inference_servers/ and examples/train/remote_inference_engine: ``run_engines_locally=false`` with
``remote_urls``).

``RemoteEngines`` stands where the trainer otherwise holds its in-process engine: generation goes through
``engine/server.py::RemoteInferenceClient`` (requests spread over the servers, sessions pinned), and the verbs the training
loop uses map to the servers' control plane:

    wake_up / sleep          nothing: the servers own their memory (the colocated trainer's phase switches do not apply)
    reset_prefix_cache       POST /reset_prefix_cache
    push_weights(model)      the policy's weights at full shapes go to ``{weights_dir}/weights_{version}.safetensors`` (a
                             directory every server can read), every server is paused, reloads them a few layers at a time
                             (POST /update_weights_layerwise), and resumes; the previous file is deleted afterwards

The servers run this framework's engine, so on the same kind of device their rollout logprobs are the trainer's bits; but
the execution contract's in-process hand-shake and ledger do not reach across HTTP, so such a run needs
``trainer.isoexec.enabled=false``: the bit-mismatch metrics are still reported every step, nothing is enforced.
"""

from __future__ import annotations

import os

from ..engine.server import RemoteInferenceClient


class RemoteEngines:
    model = None                       # there is no in-process engine model

    def __init__(self, urls: list[str], weights_dir: str, rank: int = 0):
        if not urls:
            raise ValueError("run_engines_locally=false needs generator.inference_engine.remote_urls")
        self.client = RemoteInferenceClient(list(urls))
        self.weights_dir, self.rank = weights_dir, rank
        self.asleep = False
        self.version = 0
        self.stats = {"weight_pushes": 0, "weight_bytes": 0}
        self.prefix_cache = None
        self._last_file: str | None = None
        infos = [self.client._post(u, "/get_server_info", None, "GET") for u in self.client.urls]
        self.max_len = min(int(i.get("max_model_len", 1 << 30)) for i in infos)

    def wake_up(self, tags=None) -> None:
        self.asleep = False               # the servers own their memory: the trainer's sleep / wake between phases does not reach them

    def sleep(self, tags=None) -> None:
        self.asleep = False

    def reset_prefix_cache(self) -> None:
        if self.rank == 0:
            self.client._all("/reset_prefix_cache")

    def invalidation_counts(self) -> dict:
        return {}

    def push_weights(self, model, write: bool = True) -> int:
        """Collective over the trainer's tensor-parallel group (shards are gathered to full shapes); ``write``: this rank
        writes the file and talks to the servers. Returns the bytes written."""
        from safetensors.torch import save_file

        from ..models.hf_export import full_named_weights

        sd = {}
        for name, t in full_named_weights(model):
            if write:
                sd[name] = t.detach().cpu().contiguous()
        if not write:
            return 0
        os.makedirs(self.weights_dir, exist_ok=True)
        self.version += 1
        path = os.path.join(self.weights_dir, f"weights_{self.version}.safetensors")
        tmp = path + ".tmp"
        save_file(sd, tmp)
        os.replace(tmp, path)
        self.client._all("/pause", {"mode": "keep"})
        try:
            self.client._all("/update_weights_layerwise", {"path": path})
        finally:
            self.client._all("/resume")
        if self._last_file and os.path.exists(self._last_file):
            os.remove(self._last_file)
        self._last_file = path
        n = sum(t.numel() * t.element_size() for t in sd.values())
        self.stats["weight_pushes"] += 1
        self.stats["weight_bytes"] += n
        return n
