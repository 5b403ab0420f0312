"""Per-process ExecutionContract, the handshake hash and contract delivery.

Each process (trainer rank or rollout engine) builds its contract once from the registry and
the model's selections, optionally writes it as an artifact (``ISOEXEC_CONTRACT_PATH``),
cross-checks ``ISOEXEC_CONTRACT_HASH`` when the launcher supplied one, and exposes
``contract_hash()``: the ``numerical_policy`` identity folded with named *extensions*
(reference: ISO/core/process_contract.py:25-49,78-137,150-226; ISO/core/contract_delivery.py:21-104).
Trainer and engine exchange that hash on the weight-sync init message and refuse to start on a
mismatch. An extension whose digest function raises contributes ``EXTENSION-ERROR:<Type>`` so a
broken side can never fake agreement.
"""

from __future__ import annotations

import hashlib
import json
import os
import tempfile
from typing import Callable

from ..contract import model as M
from ..contract.codec import from_canonical_json, to_canonical_json
from ..contract.digest import compute_identities
from ..contract.rules import validate_or_raise

ENV_CONTRACT_PATH = "ISOEXEC_CONTRACT_PATH"
ENV_CONTRACT_HASH = "ISOEXEC_CONTRACT_HASH"
ENV_NEGATIVE_CONTROL = "ISOEXEC_HANDSHAKE_NEGATIVE_CONTROL"


class ContractMismatch(RuntimeError):
    pass


class ContractDeliveryError(RuntimeError):
    pass


_extensions: dict[str, Callable[[], str]] = {}
_process_contract: M.ExecutionContract | None = None


def register_contract_extension(name: str, digest_fn: Callable[[], str]) -> None:
    _extensions[name] = digest_fn


def clear_contract_extensions() -> None:
    _extensions.clear()


def composite_hash(base: str, extensions: dict[str, Callable[[], str]] | None = None) -> str:
    ext = _extensions if extensions is None else extensions
    if not ext:
        return base
    digests = {}
    for name in sorted(ext):
        try:
            digests[name] = str(ext[name]())
        except Exception as e:  # noqa: BLE001 - a failing extension must poison the hash, not vanish
            digests[name] = f"EXTENSION-ERROR:{type(e).__name__}"
    blob = json.dumps({"base": base, "extensions": digests}, sort_keys=True, separators=(",", ":"))
    return hashlib.sha256(blob.encode("utf-8")).hexdigest()


def write_contract(contract: M.ExecutionContract, path: str) -> None:
    """Atomic artifact write (temp file + rename)."""
    d = os.path.dirname(os.path.abspath(path)) or "."
    os.makedirs(d, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=d, prefix=".contract.", suffix=".json")
    try:
        with os.fdopen(fd, "wb") as f:
            f.write(to_canonical_json(contract))
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)


def load_contract(path: str) -> M.ExecutionContract:
    """Load + self-consistency (stored identities == recomputed) + env hash cross-check."""
    with open(path, "rb") as f:
        c = from_canonical_json(f.read())
    if compute_identities(c) != c.identities:
        raise ContractDeliveryError(f"{path}: stored identities do not match the content")
    want = os.environ.get(ENV_CONTRACT_HASH)
    if want and want != c.identities.numerical_policy:
        raise ContractDeliveryError(f"{path}: numerical_policy {c.identities.numerical_policy[:12]} != "
                                    f"{ENV_CONTRACT_HASH} {want[:12]}")
    return c


def expected_installed_keys(contract: M.ExecutionContract, side: str) -> set[tuple[str, str]]:
    """(op, site) pairs the contract says must be installed on ``side`` ("trainer" | "engine")."""
    role = {c.id: c.runtime_role for c in contract.cases}
    return {(op, cid) for e in contract.composition for cid in e.cases if role[cid] == side for op in e.region}


def set_process_contract(contract: M.ExecutionContract) -> M.ExecutionContract:
    global _process_contract
    validate_or_raise(contract)
    _process_contract = contract
    path = os.environ.get(ENV_CONTRACT_PATH)
    if path:
        write_contract(contract, path)
    want = os.environ.get(ENV_CONTRACT_HASH)
    if want and want != contract.identities.numerical_policy:
        raise ContractDeliveryError(f"built contract {contract.identities.numerical_policy[:12]} != "
                                    f"{ENV_CONTRACT_HASH} {want[:12]}")
    return contract


def get_process_contract() -> M.ExecutionContract:
    if _process_contract is None:
        raise RuntimeError("no process contract: call set_process_contract(build...) at model construction")
    return _process_contract


def reset_process_contract() -> None:
    global _process_contract
    _process_contract = None


def contract_hash(contract: M.ExecutionContract | None = None) -> str:
    c = contract or get_process_contract()
    h = composite_hash(c.identities.numerical_policy)
    if os.environ.get(ENV_NEGATIVE_CONTROL) == "1":
        # live negative control: corrupt the stamped hash so the handshake must refuse
        h = hashlib.sha256(("negative-control:" + h).encode()).hexdigest()
    return h


def contract_hash_or_none() -> str | None:
    """The stamped hash, or None in a process that has built no contract (tools, unit tests of a transport)."""
    return contract_hash() if _process_contract is not None else None


def assert_contract_agreement(mine: str, theirs: str | None, who: str = "peer") -> None:
    if theirs is None:
        raise ContractMismatch(f"{who} sent no contract hash: refusing to run without a handshake")
    if mine != theirs:
        raise ContractMismatch(f"execution contract mismatch with {who}: local {mine[:16]}.. != remote {theirs[:16]}.. "
                               "(the two sides would not compute the same bits)")


def assert_init_info_contract(init_info, contract: M.ExecutionContract | None = None) -> None:
    """Receiver side of the weight-sync init message."""
    assert_contract_agreement(contract_hash(contract), getattr(init_info, "contract_hash", None), "trainer")
