"""The compute side of the Tinker API: one model (policy worker + colocated engine) driven by typed requests
(reference: R/backends/skyrl_train_backend.py ``SkyRLTrainBackend``; R/tinker/engine.py request loop).

Requests are plain dicts, processed strictly in arrival order:
  forward_backward {data: [{prompt_ids | chunks, response_ids, advantages?, logprobs?}], loss_fn}  -> per-sequence logprobs, loss
                   (``chunks``: text and image chunks of a multimodal prompt, engine/renderer.py::render_model_input)
  forward          {data}                                                                 -> per-sequence logprobs
  optim_step       {adam_params: {learning_rate}}                                         -> grad norm
  sample           {prompt_ids | chunks, num_samples, sampling_params}                    -> sequences + logprobs
  save_weights / load_weights {path}
"""

from __future__ import annotations

import os

import torch

from ..engine.llm_engine import EngineConfig, LLMEngine
from ..engine.sampler import SamplingParams
from ..models.config import get_config
from ..models.decoder import DecoderLM
from ..train import algorithms as alg
from ..train.batch import TrainingInputBatch, build_sequences
from ..train.policy_worker import OptimizerConfig, PolicyWorker, WorkerConfig

LOSS_FNS = {"cross_entropy": "cross_entropy", "importance_sampling": "importance_sampling", "ppo": "regular", "cispo": "cispo"}


class SkyRLTrainBackend:
    def __init__(self, base_model: str = "tiny-qwen3", model_overrides: dict | None = None, device: str | None = None,
                 lr: float = 1e-5, seed: int = 0, num_kv_pages: int = 64, external_inference_url: str | None = None,
                 external_inference_model: str = "policy", external_timeout_s: float = 600.0):
        # sampling can be served by a separate OpenAI-compatible server (reference: R/tinker/extra/external_inference.py):
        # token-id prompts to POST {url}/v1/completions, sampled ids and logprobs back; training stays in this process
        self.external_url = external_inference_url.rstrip("/") if external_inference_url else None
        self.external_model, self.external_timeout_s = external_inference_model, external_timeout_s
        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.cfg = get_config(base_model, **(model_overrides or {}))
        self.model = DecoderLM(self.cfg, device=dev, seed=seed)
        self.algo = alg.AlgorithmConfig(policy_loss_type="cross_entropy")
        self.worker = PolicyWorker(self.model, WorkerConfig(optimizer=OptimizerConfig(lr=lr, num_warmup_steps=0)), self.algo)
        self.engine = LLMEngine(self.model, EngineConfig(max_num_seqs=64, num_kv_pages=num_kv_pages, seed=seed + 1))
        self.step_count = 0
        # multi-tenant LoRA (reference: docs/content/docs/tinker/multi_tenancy.mdx, B/workers/megatron/adapter_store.py): several
        # model ids share this backend's base weights, each with an adapter of its own that is merged in while its requests
        # run; the base never trains
        self.store = None
        self.tenants: dict = {}             # tenant -> {"trainer": LoRATrainer, "step": int}

    def add_tenant(self, tenant: str, rank: int, alpha: float = 16.0, lr: float = 1e-4, seed: int = 0) -> None:
        from ..train.lora import AdapterStore, LoRAAdapter, LoRAConfig, LoRATrainer

        if self.store is None:
            self.store = AdapterStore(self.model)
        self.store.deactivate()                          # a new adapter is sized on the base weights
        self.store.register(tenant, LoRAAdapter.init(self.model, LoRAConfig(rank=rank, alpha=alpha, lr=lr, seed=seed)))
        self.tenants[tenant] = {"trainer": LoRATrainer(self.worker, self.store, tenant), "step": 0}

    def _switch(self, tenant: str | None) -> None:
        """Merge the adapter of the request's tenant (dropping what the engine cached under another one)."""
        if self.store is None:
            return
        if tenant is not None and tenant not in self.tenants:
            raise KeyError(f"unknown adapter {tenant!r}")
        if self.store.active != tenant:
            if tenant is None:
                self.store.deactivate()
            else:
                self.store.activate(tenant)
            self.engine.reset_prefix_cache()

    def _sample_external(self, prompt_ids: list[int], sp, n: int) -> dict:
        import json
        import urllib.request

        body = {"model": self.external_model, "prompt": prompt_ids, "n": n, "max_tokens": sp.max_generate_length,
                "temperature": sp.temperature, "top_p": sp.top_p, "logprobs": 1}
        if sp.top_k and sp.top_k > 0:
            body["top_k"] = sp.top_k
        if sp.stop_token_ids:
            body["stop_token_ids"] = list(sp.stop_token_ids)
        if sp.ignore_eos:
            body["ignore_eos"] = True
        req = urllib.request.Request(self.external_url + "/v1/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=self.external_timeout_s) as r:
            out = json.loads(r.read())
        seqs = []
        for c in out["choices"]:
            if "token_ids" not in c:
                raise RuntimeError("the external server's completion carries no token_ids: training needs the sampled ids")
            lps = (c.get("logprobs") or {}).get("token_logprobs") or [0.0] * len(c["token_ids"])
            seqs.append({"tokens": list(c["token_ids"]), "logprobs": list(lps),
                         "stop_reason": "length" if c.get("finish_reason") == "length" else "stop"})
        return {"sequences": seqs}

    def _render(self, item: dict) -> tuple[list[int], dict | None]:
        """Prompt ids and image features of a request item: ``prompt_ids`` as given, or ``chunks`` (text and image chunks,
        ``engine/renderer.py::render_model_input``)."""
        if item.get("chunks") is None:
            return list(item["prompt_ids"]), None
        from ..engine.renderer import render_model_input

        r = render_model_input(item["chunks"], self.model.cfg)
        return r["token_ids"], r["features"]

    def _batch(self, data: list[dict]) -> TrainingInputBatch:
        rendered = [self._render(d) for d in data]
        seq, att, rmask = build_sequences([ids for ids, _ in rendered], [d["response_ids"] for d in data])
        B, R = rmask.shape
        adv, old = torch.zeros(B, R), torch.zeros(B, R)
        lmask = rmask.clone()
        for i, d in enumerate(data):
            n = len(d["response_ids"])
            a = d.get("advantages", 1.0)
            adv[i, :n] = torch.tensor(a, dtype=torch.float32) if isinstance(a, (list, tuple)) else float(a)
            if d.get("logprobs") is not None:
                old[i, :n] = torch.tensor(d["logprobs"], dtype=torch.float32)
            if d.get("loss_mask") is not None:          # multi-turn data: observation tokens carry weight 0
                lmask[i, :n] = torch.tensor(d["loss_mask"], dtype=lmask.dtype)
        fields = {"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": lmask,
                  "advantages": adv, "action_log_probs": old, "rollout_logprobs": old.clone()}
        feats = [f for _, f in rendered]
        if any(f is not None for f in feats):
            from ..train.batch import TensorList

            dim = next(f["pixel_values"].shape[1] for f in feats if f is not None)
            fields["pixel_values"] = TensorList([f["pixel_values"] if f else torch.zeros(0, dim) for f in feats])
            fields["image_grid_thw"] = TensorList([f["image_grid_thw"] if f else torch.zeros(0, 3, dtype=torch.int64) for f in feats])
            fields["mm_positions"] = TensorList([torch.tensor(f["positions"] if f else [], dtype=torch.int64) for f in feats])
        return TrainingInputBatch(fields)

    def handle(self, req: dict) -> dict:
        kind = req["type"]
        tenant = req.get("tenant")
        self._switch(tenant)
        if tenant is not None and kind == "optim_step":
            t = self.tenants[tenant]
            lr = (req.get("adam_params") or {}).get("learning_rate")
            if lr is not None:
                for gparam in t["trainer"].opt.param_groups:
                    gparam["lr"] = float(lr)
            self.worker.reduce_gradients()
            gn = t["trainer"].optim_step()
            t["step"] += 1
            self.engine.reset_prefix_cache()
            return {"grad_norm": gn, "step": t["step"]}
        if tenant is not None and kind in ("save_weights", "load_weights"):
            ad = self.store.adapters[tenant]
            if kind == "save_weights":
                os.makedirs(os.path.dirname(req["path"]) or ".", exist_ok=True)
                torch.save({"adapter": ad.state_dict(), "step": self.tenants[tenant]["step"], "opt": self.tenants[tenant]["trainer"].opt.state_dict()}, req["path"])
                return {"path": req["path"]}
            sd = torch.load(req["path"], weights_only=False, map_location="cpu")
            for k in ad.A:
                ad.A[k].copy_(sd["adapter"]["A"][k])
                ad.B[k].copy_(sd["adapter"]["B"][k])
            self.tenants[tenant]["trainer"].opt.load_state_dict(sd["opt"])
            self.tenants[tenant]["step"] = int(sd.get("step", 0))
            self.store.refresh()
            self.engine.reset_prefix_cache()
            return {"step": self.tenants[tenant]["step"]}
        if kind in ("forward", "forward_backward"):
            b = self._batch(req["data"])
            lens = [len(d["response_ids"]) for d in req["data"]]
            if kind == "forward":
                lp = self.worker.forward(b)
                return {"logprobs": [lp[i, :n].tolist() for i, n in enumerate(lens)]}
            loss_fn = req.get("loss_fn", "cross_entropy")
            if loss_fn not in LOSS_FNS:
                raise ValueError(f"loss_fn {loss_fn!r} not in {sorted(LOSS_FNS)}")
            self.algo.policy_loss_type = LOSS_FNS[loss_fn]
            if loss_fn == "cross_entropy" or all(d.get("logprobs") is None for d in req["data"]):
                b.pop("action_log_probs")
            m = self.worker.forward_backward(b)
            return {"loss": m["policy_loss"], "num_tokens": m["loss_tokens"], "clip_ratio": m["ppo_clip_ratio"]}
        if kind == "optim_step":
            lr = (req.get("adam_params") or {}).get("learning_rate")
            if lr is not None:
                self.worker.opt.cfg.lr = float(lr)
            gn = self.worker.optim_step()
            self.step_count += 1
            self.engine.reset_prefix_cache()
            return {"grad_norm": gn, "step": self.step_count}
        if kind == "sample":
            sp = SamplingParams.from_dict(req.get("sampling_params"))
            n = int(req.get("num_samples", 1))
            ids, feats = self._render(req)
            if self.external_url:
                if feats is not None:
                    raise ValueError("image chunks cannot be sampled through an external text-completion server")
                return self._sample_external(ids, sp, n)
            if self.engine.asleep:
                self.engine.wake_up()
            outs = self.engine.generate([ids] * n, sp, mm=[feats] * n if feats is not None else None)
            res = {"sequences": [{"tokens": o.response_ids, "logprobs": o.response_logprobs, "stop_reason": o.stop_reason} for o in outs]}
            if sp.prompt_logprobs is not None:
                res["prompt_logprobs"] = outs[0].prompt_logprobs          # the samples share the prompt
            return res
        if kind == "save_weights_for_sampler":
            # the sampler IS this backend's engine and reads the trainer's parameter buffer: publishing new weights is a
            # version bump plus dropping what the engine cached under the old ones (optionally also a file for others)
            self.sampler_version = getattr(self, "sampler_version", 0) + 1
            self.engine.reset_prefix_cache()
            out = {"sampler_version": self.sampler_version, "step": self.step_count}
            if req.get("path"):
                os.makedirs(os.path.dirname(req["path"]) or ".", exist_ok=True)
                torch.save({"model": {k: v.detach().cpu() for k, v in self.model.named_weights()}, "step": self.step_count}, req["path"])
                out["path"] = req["path"]
            return out
        if kind == "save_weights":
            os.makedirs(os.path.dirname(req["path"]) or ".", exist_ok=True)
            torch.save({"model": {k: v.detach().cpu() for k, v in self.model.named_weights()}, "step": self.step_count,
                        "optimizer": self.worker.opt.state_dict()}, req["path"])
            return {"path": req["path"]}
        if kind == "load_weights":
            from ..sync.strategies import load_weights

            sd = torch.load(req["path"], weights_only=False, map_location="cpu")
            load_weights(self.model, sd["model"].items())
            if sd.get("optimizer") is not None and req.get("with_optimizer", True):
                self.worker.opt.load_state_dict(sd["optimizer"])
            self.step_count = int(sd.get("step", 0))
            return {"step": self.step_count}
        raise ValueError(f"unknown request type {kind!r}")
