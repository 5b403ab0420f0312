"""Rollout engine in another process, reached over ``torch.distributed`` object messages.

``DistEngineServer.serve()`` runs on the rollout rank and answers requests from
``DistEngineClient`` (an ``InferenceEngineInterface``) on the trainer rank: generate, sleep /
wake, weight-sync init (where the contract hashes are compared and a mismatch is sent back as
an error and raised on BOTH sides), weight update, shutdown. The reference does the same over
Ray actor calls / HTTP (B/inference_engines/ray_wrapped_inference_engine.py,
B/inference_servers/remote_inference_client.py); here the control plane is the process group
the two sides already share, so the CPU/gloo configuration needs nothing else.
"""

from __future__ import annotations

import asyncio
import traceback

import torch.distributed as dist

from ..core.process import ContractMismatch
from .interface import InferenceEngineInterface, NativeInferenceEngine


def _send(obj, dst: int, group=None) -> None:
    dist.send_object_list([obj], dst=dst, group=group)


def _recv(src: int, group=None):
    box = [None]
    dist.recv_object_list(box, src=src, group=group)
    return box[0]


class DistEngineServer:
    def __init__(self, engine: NativeInferenceEngine, client_rank: int, group=None):
        self.engine, self.client, self.group = engine, client_rank, group

    def serve(self) -> None:
        while True:
            verb, payload = _recv(self.client, self.group)
            if verb == "shutdown":
                _send(("ok", None), self.client, self.group)
                return
            try:
                if verb == "generate":
                    res = asyncio.run(self.engine.generate(payload))
                elif verb == "sleep":
                    res = asyncio.run(self.engine.sleep())
                elif verb == "wake_up":
                    res = asyncio.run(self.engine.wake_up())
                elif verb == "init_weight_update_communicator":
                    res = asyncio.run(self.engine.init_weight_update_communicator(payload))
                elif verb == "update_named_weights":
                    _send(("go", None), self.client, self.group)   # receiver is about to enter the collective
                    res = asyncio.run(self.engine.update_named_weights(payload))
                elif verb == "reset_prefix_cache":
                    res = asyncio.run(self.engine.reset_prefix_cache())
                elif verb == "stats":
                    res = dict(self.engine.llm.stats)
                else:
                    raise ValueError(f"unknown verb {verb!r}")
                _send(("ok", res), self.client, self.group)
            except ContractMismatch as e:
                _send(("contract_mismatch", str(e)), self.client, self.group)
                raise
            except Exception as e:  # noqa: BLE001
                _send(("error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"), self.client, self.group)


class DistEngineClient(InferenceEngineInterface):
    def __init__(self, server_rank: int, group=None, tp: int = 1):
        self.server, self.group, self._tp = server_rank, group, tp

    def _call(self, verb, payload=None, pre_reply=None):
        _send((verb, payload), self.server, self.group)
        if pre_reply is not None:
            tag, _ = _recv(self.server, self.group)
            assert tag == "go"
            pre_reply()
        tag, res = _recv(self.server, self.group)
        if tag == "contract_mismatch":
            raise ContractMismatch(res)
        if tag == "error":
            raise RuntimeError(f"remote engine failed: {res}")
        return res

    async def generate(self, input_batch):
        return self._call("generate", dict(input_batch))

    async def wake_up(self, *a, **kw):
        return self._call("wake_up")

    async def sleep(self, *a, **kw):
        return self._call("sleep")

    async def init_weight_update_communicator(self, init_info):
        return self._call("init_weight_update_communicator", init_info)

    async def update_named_weights(self, request, send_fn=None):
        """``send_fn`` runs the sender's half of the collective once the server has entered its half."""
        return self._call("update_named_weights", request, pre_reply=send_fn)

    async def reset_prefix_cache(self):
        return self._call("reset_prefix_cache")

    async def teardown(self):
        return self._call("shutdown")

    def stats(self):
        return self._call("stats")

    def tp_size(self):
        return self._tp
