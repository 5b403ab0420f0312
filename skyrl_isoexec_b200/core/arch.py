"""Architecture as a first-class dimension of a composition (reference: ISO/core/arch.py:27-88).
A leaf summed with the tcgen05 k-step differs in its low bits from one summed on another tensor
core generation, so the arch label is part of every ImplRef and of the handshake."""

from __future__ import annotations

from dataclasses import dataclass

import torch


def detect_arch(device=None) -> str:
    """"sm100" on a Blackwell GPU, "cpu" for CPU tensors; any other GPU is refused."""
    dev = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    if dev.type != "cuda":
        return "cpu"
    major, minor = torch.cuda.get_device_capability(dev)
    if major == 10:
        return "sm100"
    raise RuntimeError(f"unsupported GPU architecture sm{major}{minor}: this framework is written for sm_100a only")


@dataclass(frozen=True)
class HardwareTarget:
    arch: str
    device_name: str = ""

    @staticmethod
    def current(device=None) -> "HardwareTarget":
        a = detect_arch(device)
        name = torch.cuda.get_device_name(device) if a != "cpu" else "cpu"
        return HardwareTarget(a, name)

    @staticmethod
    def assert_homogeneous(targets: list["HardwareTarget"]) -> "HardwareTarget":
        archs = {t.arch for t in targets}
        if len(archs) != 1:
            raise RuntimeError(f"heterogeneous architectures in one job: {sorted(archs)}; bitwise parity cannot hold")
        return targets[0]
