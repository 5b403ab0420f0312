"""Path-scheme aware file helpers (reference: B/utils/io/ local / S3 / GCS). Only the local scheme is available
offline; remote schemes raise with the name of the missing client instead of failing somewhere deeper."""

from __future__ import annotations

import contextlib
import os
import shutil
import tempfile

_REMOTE = {"s3": "boto3 / s3fs", "gs": "gcsfs", "gcs": "gcsfs", "hdfs": "pyarrow.fs"}


def scheme(path: str) -> str:
    return path.split("://", 1)[0] if "://" in path else "file"


def _local(path: str) -> str:
    s = scheme(path)
    if s == "file":
        return path[len("file://"):] if path.startswith("file://") else path
    raise RuntimeError(f"{s}:// paths need {_REMOTE.get(s, 'a remote filesystem client')}, which is not installed here")


def exists(path: str) -> bool:
    return os.path.exists(_local(path))


def makedirs(path: str) -> None:
    os.makedirs(_local(path), exist_ok=True)


def list_dir(path: str) -> list[str]:
    return sorted(os.listdir(_local(path)))


def remove(path: str) -> None:
    p = _local(path)
    if os.path.isdir(p):
        shutil.rmtree(p)
    elif os.path.exists(p):
        os.remove(p)


@contextlib.contextmanager
def open_file(path: str, mode: str = "r"):
    p = _local(path)
    if any(m in mode for m in "wa"):
        os.makedirs(os.path.dirname(p) or ".", exist_ok=True)
    with open(p, mode) as f:
        yield f


@contextlib.contextmanager
def atomic_write(path: str, mode: str = "w"):
    """Write to a temporary sibling and rename: a reader never sees a torn checkpoint marker."""
    p = _local(path)
    os.makedirs(os.path.dirname(p) or ".", exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=os.path.dirname(p) or ".", prefix=".tmp-")
    try:
        with os.fdopen(fd, mode) as f:
            yield f
        os.replace(tmp, p)
    except BaseException:
        with contextlib.suppress(OSError):
            os.remove(tmp)
        raise


@contextlib.contextmanager
def local_work_dir(path: str):
    """A local directory standing for ``path`` (identity for local paths)."""
    p = _local(path)
    os.makedirs(p, exist_ok=True)
    yield p


# ----------------------------------------------------------------------------- archives (reference: R/utils/storage.py)
@contextlib.contextmanager
def pack_and_upload(dest: str, rank: int | None = None):
    """Yield an empty temporary directory; on a clean exit its content becomes the archive ``dest`` (tar inside gzip at
    level 0: checkpoint tensors do not compress, speed matters). With ``rank`` given and a ``dest + ".probe"`` file
    present, the filesystem is shared between the ranks and only rank 0 writes. The archive appears atomically."""
    import gzip
    import tarfile

    with tempfile.TemporaryDirectory() as tmp:
        yield tmp
        if rank not in (None, 0) and exists(dest + ".probe"):
            return
        with atomic_write(dest, "wb") as f:
            with gzip.GzipFile(fileobj=f, mode="wb", compresslevel=0) as gz:
                with tarfile.open(fileobj=gz, mode="w:") as tar:
                    tar.add(tmp, arcname="")


@contextlib.contextmanager
def download_and_unpack(source: str):
    """Yield a temporary directory holding the content of the archive ``source``. Members that would land outside the
    directory, links and device files are refused (tarfile's ``data`` filter)."""
    import tarfile

    with tempfile.TemporaryDirectory() as tmp:
        with open_file(source, "rb") as f:
            with tarfile.open(fileobj=f, mode="r:gz") as tar:
                tar.extractall(tmp, filter="data")
        yield tmp


def download_file(source: str):
    """The whole file as an in-memory binary stream positioned at 0."""
    import io as _io

    with open_file(source, "rb") as f:
        return _io.BytesIO(f.read())
