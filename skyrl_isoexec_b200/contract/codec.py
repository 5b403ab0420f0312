"""Canonical JSON codec for the ExecutionContract: sorted keys, compact separators, UTF-8, no
JSON floats (a float constant is a ``BitPattern`` or a decimal string), unknown fields refused,
schema version "2" only. The canonical bytes are what the identity hashes are taken over
(reference wire rules: ISO/contract/serialize.py:23-48,154-156,264-298). Encoding and decoding
are driven by ``model.SCHEMA`` rather than written per class.
"""

from __future__ import annotations

import json

from .model import SCHEMA, SCHEMA_VERSION, BitPattern, ExecutionContract

SUPPORTED_SCHEMA_VERSIONS = frozenset({SCHEMA_VERSION})


class SerializationError(Exception):
    pass


class UnknownFieldError(SerializationError):
    pass


def refuse_floats(obj, path: str = "$") -> None:
    if isinstance(obj, float):
        raise SerializationError(f"raw float at {path}; carry it as a BitPattern or a decimal string")
    if isinstance(obj, dict):
        for k, v in obj.items():
            refuse_floats(v, f"{path}.{k}")
    elif isinstance(obj, (list, tuple)):
        for i, v in enumerate(obj):
            refuse_floats(v, f"{path}[{i}]")


def canonical_bytes(plain) -> bytes:
    refuse_floats(plain)
    return json.dumps(plain, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode("utf-8")


def _enc_value(v):
    return {"bits": v.bits, "dtype": v.dtype} if isinstance(v, BitPattern) else v


def _dec_value(v, ctx):
    if isinstance(v, dict):
        if set(v) != {"bits", "dtype"}:
            raise UnknownFieldError(f"{ctx}: a constant object must be exactly {{bits, dtype}}, got {sorted(v)}")
        return BitPattern(v["bits"], v["dtype"])
    return v


def to_plain(obj):
    """Dataclass -> plain JSON structure following SCHEMA."""
    out = {}
    for name, kind in SCHEMA[type(obj)]:
        v = getattr(obj, name)
        if kind == "scalar":
            out[name] = v
        elif kind == "list":
            out[name] = list(v)
        elif kind == "map":
            out[name] = {k: _enc_value(x) for k, x in v}
        elif kind[0] == "obj":
            out[name] = to_plain(v)
        elif kind[0] == "opt":
            out[name] = None if v is None else to_plain(v)
        elif kind[0] == "objs":
            out[name] = [to_plain(x) for x in v]
    return out


def from_plain(cls, d, ctx: str = "$"):
    if not isinstance(d, dict):
        raise SerializationError(f"{ctx}: expected an object for {cls.__name__}")
    names = [n for n, _ in SCHEMA[cls]]
    unknown = set(d) - set(names)
    if unknown:
        raise UnknownFieldError(f"{ctx}: unknown field(s) {sorted(unknown)} for {cls.__name__}")
    missing = set(names) - set(d)
    if missing:
        raise SerializationError(f"{ctx}: missing field(s) {sorted(missing)} for {cls.__name__}")
    kw = {}
    for name, kind in SCHEMA[cls]:
        v, c = d[name], f"{ctx}.{name}"
        if kind == "scalar":
            kw[name] = v
        elif kind == "list":
            kw[name] = tuple(v)
        elif kind == "map":
            kw[name] = tuple(sorted((k, _dec_value(x, c)) for k, x in v.items()))
        elif kind[0] == "obj":
            kw[name] = from_plain(kind[1], v, c)
        elif kind[0] == "opt":
            kw[name] = None if v is None else from_plain(kind[1], v, c)
        elif kind[0] == "objs":
            kw[name] = tuple(from_plain(kind[1], x, f"{c}[{i}]") for i, x in enumerate(v))
    return cls(**kw)


def to_canonical_json(contract: ExecutionContract) -> bytes:
    return canonical_bytes(to_plain(contract))


def from_canonical_json(data: bytes | str) -> ExecutionContract:
    try:
        plain = json.loads(data, parse_float=_no_float)
    except ValueError as e:
        raise SerializationError(f"not valid JSON: {e}") from e
    if not isinstance(plain, dict):
        raise SerializationError("top level must be an object")
    ver = plain.get("schema_version")
    if ver not in SUPPORTED_SCHEMA_VERSIONS:
        raise SerializationError(f"unsupported schema_version {ver!r}; this build reads {sorted(SUPPORTED_SCHEMA_VERSIONS)}")
    return from_plain(ExecutionContract, plain)


def _no_float(s):
    raise SerializationError(f"JSON float {s!r} in a contract document")
