"""The RL trainer against inference servers it does not own: generation over HTTP, weights through a shared directory."""
import os

import pytest
import torch

from skyrl_isoexec_b200.train.config import SkyRLTrainConfig, validate_cfg


def test_trainer_rolls_out_on_remote_servers_and_pushes_its_weights(tmp_path):
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.server import ServerGroup
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.remote_engines import RemoteEngines
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    # two servers that start from OTHER weights than the policy: what they generate is the policy's only if the push works
    engines = [LLMEngine(DecoderLM(get_config("tiny-qwen3"), seed=90 + i), EngineConfig(num_kv_pages=32, seed=5 + i)) for i in range(2)]
    group = ServerGroup(engines)
    urls = group.start()
    try:
        ov = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4", "generator.n_samples_per_prompt=2",
              "generator.sampling_params.max_generate_length=8", "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8",
              "data.synthetic_prompts=16", "trainer.max_prompt_length=8", "trainer.num_steps=2", "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}",
              "trainer.resume_mode=none", "trainer.ckpt_interval=0", "trainer.policy.optimizer_config.lr=1e-3", "trainer.isoexec.enabled=false",
              "generator.inference_engine.run_engines_locally=false", "generator.inference_engine.remote_urls=" + str(urls).replace("'", '"')]
        cfg = SkyRLTrainConfig.from_cli_overrides(ov)
        validate_cfg(cfg)
        tr = RayPPOTrainer(cfg, device="cpu")
        tr.train()
        assert isinstance(tr.engine, RemoteEngines) and tr.global_step == 2
        assert tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0            # same kernels on both ends: same bits
        assert tr.engine.stats["weight_pushes"] == 3 and tr.all_metrics["sync/bytes"] > 0      # before the first step and after each
        for e in engines:                                                                      # both servers hold the last update
            assert torch.equal(e.model.store.flat, tr.policy.model.store.flat)
        assert sum(e.stats["tokens"] for e in engines) > 0 and all(e.stats["tokens"] > 0 for e in engines)   # the requests were spread
        files = os.listdir(tmp_path / "remote_weights")
        assert files == ["weights_3.safetensors"]                                              # older files are removed
    finally:
        group.shutdown()
    # what the configuration check says
    bad = SkyRLTrainConfig.from_cli_overrides(["generator.inference_engine.run_engines_locally=false"])
    with pytest.raises(ValueError, match="remote_urls"):
        validate_cfg(bad)
    with pytest.raises(ValueError, match="isoexec.enabled=false"):
        validate_cfg(SkyRLTrainConfig.from_cli_overrides(["generator.inference_engine.run_engines_locally=false",
                                                          'generator.inference_engine.remote_urls=["http://127.0.0.1:1"]']))


def test_http_endpoint_in_front_of_the_trainers_engine_keeps_the_contract(tmp_path):
    import json
    import urllib.request

    from skyrl_isoexec_b200.train.callbacks import TrainingCallback
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    ov = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=2", "trainer.policy_mini_batch_size=2", "generator.n_samples_per_prompt=2",
          "generator.sampling_params.max_generate_length=8", "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8",
          "data.synthetic_prompts=8", "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=16", "trainer.num_steps=2",
          "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}", "trainer.resume_mode=none", "trainer.ckpt_interval=0",
          "generator.inference_engine.enable_http_endpoint=true"]
    seen = {}

    class External(TrainingCallback):                      # an outside client of the same endpoint, between two steps
        def on_step_end(self, trainer, inp, control):
            trainer.engine.wake_up()
            req = urllib.request.Request(trainer.http_endpoint_url + "/generate", data=json.dumps(
                {"prompt_token_ids": [[5, 6, 7]], "sampling_params": {"max_generate_length": 3, "ignore_eos": True}}).encode(),
                headers={"Content-Type": "application/json"})
            seen[trainer.global_step] = json.loads(urllib.request.urlopen(req, timeout=60).read())["response_ids"][0]
            trainer.engine.sleep()

    tr = RayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(ov), device="cpu", callbacks=[External()])
    try:
        tr.train()
        assert tr.http_endpoint_url.startswith("http://127.0.0.1:") and tr.global_step == 2
        assert tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0 and tr.adapter_engine.ledger.verdict()["ok"]
        assert len(seen[1]) == 3 and len(seen[2]) == 3 and tr.http_server.requests_served >= 2 * 4 + 2
    finally:
        tr.http_server.shutdown()


def test_trainer_through_a_router_in_front_of_two_servers(tmp_path):
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.router import Router
    from skyrl_isoexec_b200.engine.server import ServerGroup
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    engines = [LLMEngine(DecoderLM(get_config("tiny-qwen3"), seed=70 + i), EngineConfig(num_kv_pages=32, seed=9 + i)) for i in range(2)]
    group = ServerGroup(engines)
    router = Router(group.start()).start()
    try:
        ov = ["trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4", "generator.n_samples_per_prompt=2",
              "generator.sampling_params.max_generate_length=6", "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8",
              "data.synthetic_prompts=16", "trainer.max_prompt_length=8", "trainer.num_steps=1", "trainer.logger=jsonl", f"trainer.ckpt_path={tmp_path}",
              "trainer.resume_mode=none", "trainer.ckpt_interval=0", "trainer.isoexec.enabled=false",
              "generator.inference_engine.run_engines_locally=false", f"generator.inference_engine.external_proxy_url={router.url}"]
        tr = RayPPOTrainer(SkyRLTrainConfig.from_cli_overrides(ov), device="cpu")
        tr.train()
        assert tr.all_metrics["policy/rollout_train_logprob_bit_mismatches"] == 0
        assert all(torch.equal(e.model.store.flat, tr.policy.model.store.flat) for e in engines)       # the push fanned out to both
        assert all(e.stats["tokens"] > 0 for e in engines)                                              # and so did the requests
    finally:
        router.shutdown()
        group.shutdown()
