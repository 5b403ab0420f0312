"""Gate-signature table: per (model, numerical-policy hash, arch) the admitted steady-state
signature of a healthy run (mean |rollout - train| logprob diff band, entropy), each backed by a
proof reference; admission without a proof ref is refused (reference: ISO/core/signatures.py:48-131).
Under this framework's contract the admitted band is exactly zero."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Signature:
    model: str
    policy_hash: str
    arch: str
    mean_abs_diff_lo: float
    mean_abs_diff_hi: float
    entropy: float | None
    proof_ref: str


class SignatureTable:
    def __init__(self):
        self._rows: dict[tuple[str, str, str], Signature] = {}

    def admit(self, model: str, policy_hash: str, arch: str, mean_abs_diff_band: tuple[float, float],
              entropy: float | None = None, proof_ref: str = "") -> Signature:
        if not proof_ref or not proof_ref.strip():
            raise ValueError("a gate signature needs a proof_ref (the run or test that produced it)")
        lo, hi = mean_abs_diff_band
        if lo < 0 or hi < lo:
            raise ValueError(f"invalid band {mean_abs_diff_band}")
        sig = Signature(model, policy_hash, arch, lo, hi, entropy, proof_ref)
        self._rows[(model, policy_hash, arch)] = sig
        return sig

    def lookup(self, model: str, policy_hash: str, arch: str) -> Signature | None:
        return self._rows.get((model, policy_hash, arch))

    def check(self, model: str, policy_hash: str, arch: str, mean_abs_diff: float) -> tuple[bool, str]:
        sig = self.lookup(model, policy_hash, arch)
        if sig is None:
            return False, "no admitted signature for this (model, contract, arch)"
        ok = sig.mean_abs_diff_lo <= mean_abs_diff <= sig.mean_abs_diff_hi
        return ok, "" if ok else f"mean diff {mean_abs_diff:.3e} outside [{sig.mean_abs_diff_lo:.3e}, {sig.mean_abs_diff_hi:.3e}]"


def bitwise_table(model: str, policy_hash: str, arch: str, proof_ref: str) -> SignatureTable:
    t = SignatureTable()
    t.admit(model, policy_hash, arch, (0.0, 0.0), proof_ref=proof_ref)
    return t
