"""Path-scheme aware file helpers (reference: R/backends/skyrl_train/utils/io/io.py: local, S3 and GCS through fsspec).

A path without a scheme, or with ``file://``, is local and goes through ``os``. Every other scheme (``s3://``, ``gs://``,
``gcs://``, ``hdfs://``, ``memory://``, ``local://`` ...) goes through ``fsspec.filesystem(scheme)``: it works when the
client package of that scheme is installed (``s3fs``, ``gcsfs``, ``pyarrow``), and raises with the name of the missing
package otherwise. ``memory://`` (fsspec's in-process store) and ``local://`` (the local disk, but through the whole
remote code path) need no client, which is what the tests use.

Directory-shaped work on a remote path is staged: ``local_work_dir`` yields a temporary directory and uploads it on exit,
``local_read_dir`` downloads into one. A call that fails with an error that looks transient (timeouts, throttling, expired
tokens) is retried with back-off; filesystem instances are re-made on the retry so that refreshed credentials are seen.
"""

from __future__ import annotations

import contextlib
import os
import shutil
import tempfile
import time

_CLIENTS = {"s3": "s3fs", "s3a": "s3fs", "gs": "gcsfs", "gcs": "gcsfs", "hdfs": "pyarrow", "abfs": "adlfs", "az": "adlfs"}
_TRANSIENT = ("timeout", "timed out", "throttl", "slowdown", "expiredtoken", "requestexpired", "temporar", "connection reset", "503", "500")
RETRIES, BACKOFF_S = 4, 0.5


def scheme(path: str) -> str:
    return path.split("://", 1)[0] if "://" in path else "file"


def is_cloud_path(path: str) -> bool:
    """True for every path that is reached through fsspec instead of ``os``."""
    return scheme(str(path)) != "file"


def _local(path: str) -> str:
    return path[len("file://"):] if path.startswith("file://") else path


def _fs(path: str, fresh: bool = False):
    s = scheme(path)
    try:
        import fsspec

        return fsspec.filesystem(s, skip_instance_cache=fresh) if fresh else fsspec.filesystem(s)
    except (ImportError, ValueError) as e:
        need = _CLIENTS.get(s)
        raise RuntimeError(f"{s}:// paths need {need or 'an fsspec client for that scheme'}, which is not installed here ({e})") from None


def _retry(path: str, fn):
    """``fn(fs, stripped path)`` with retries on errors that look transient."""
    last = None
    for attempt in range(RETRIES):
        fs = _fs(path, fresh=attempt > 0)
        try:
            return fn(fs, fs._strip_protocol(path))
        except (FileNotFoundError, IsADirectoryError, NotADirectoryError, PermissionError):
            raise
        except Exception as e:  # noqa: BLE001 - the clients raise their own classes; the text decides
            if not any(t in (type(e).__name__ + " " + str(e)).lower() for t in _TRANSIENT):
                raise
            last = e
            time.sleep(BACKOFF_S * (2 ** attempt))
    raise last


def exists(path: str) -> bool:
    if not is_cloud_path(path):
        return os.path.exists(_local(path))
    return bool(_retry(path, lambda fs, p: fs.exists(p)))


def isdir(path: str) -> bool:
    if not is_cloud_path(path):
        return os.path.isdir(_local(path))
    return bool(_retry(path, lambda fs, p: fs.isdir(p)))


def makedirs(path: str) -> None:
    if not is_cloud_path(path):
        os.makedirs(_local(path), exist_ok=True)
    else:
        _retry(path, lambda fs, p: fs.makedirs(p, exist_ok=True))


def list_dir(path: str) -> list[str]:
    """Names (not paths) of the entries of a directory, sorted."""
    if not is_cloud_path(path):
        return sorted(os.listdir(_local(path)))
    return sorted({str(e).rstrip("/").rsplit("/", 1)[-1] for e in _retry(path, lambda fs, p: fs.ls(p, detail=False))} - {""})


def remove(path: str) -> None:
    if not is_cloud_path(path):
        p = _local(path)
        if os.path.isdir(p):
            shutil.rmtree(p)
        elif os.path.exists(p):
            os.remove(p)
        return
    _retry(path, lambda fs, p: fs.rm(p, recursive=True) if fs.exists(p) else None)


@contextlib.contextmanager
def open_file(path: str, mode: str = "r"):
    if not is_cloud_path(path):
        p = _local(path)
        if any(m in mode for m in "wa"):
            os.makedirs(os.path.dirname(p) or ".", exist_ok=True)
        with open(p, mode) as f:
            yield f
        return
    with _retry(path, lambda fs, p: fs.open(p, mode)) as f:
        yield f


@contextlib.contextmanager
def atomic_write(path: str, mode: str = "w"):
    """Write to a temporary sibling and rename: a reader never sees a torn checkpoint marker. On an object store the
    object appears when the writer closes it, which is atomic already."""
    if is_cloud_path(path):
        with open_file(path, mode) as f:
            yield f
        return
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


def _walk(root: str):
    for d, _dirs, files in os.walk(root):
        for name in files:
            full = os.path.join(d, name)
            yield full, os.path.relpath(full, root).replace(os.sep, "/")


def upload_file(local_path: str, dest: str) -> None:
    if not is_cloud_path(dest):
        os.makedirs(os.path.dirname(_local(dest)) or ".", exist_ok=True)
        shutil.copyfile(local_path, _local(dest))
        return
    _retry(dest, lambda fs, p: (fs.makedirs(p.rsplit("/", 1)[0], exist_ok=True) if "/" in p else None, fs.put_file(local_path, p)))


def upload_directory(local_dir: str, dest: str, only: list[str] | None = None) -> int:
    """Every file under ``local_dir`` (or just the relative paths in ``only``) to the same relative path under ``dest``.
    Returns the number of files sent."""
    n = 0
    for full, rel in _walk(local_dir):
        if only is not None and rel not in only:
            continue
        upload_file(full, dest.rstrip("/") + "/" + rel)
        n += 1
    return n


def download_file_to(source: str, local_path: str) -> None:
    os.makedirs(os.path.dirname(local_path) or ".", exist_ok=True)
    if not is_cloud_path(source):
        shutil.copyfile(_local(source), local_path)
        return
    _retry(source, lambda fs, p: fs.get_file(p, local_path))


def download_directory(source: str, local_dir: str) -> int:
    """The tree under ``source`` into ``local_dir``; returns the number of files fetched."""
    if not is_cloud_path(source):
        shutil.copytree(_local(source), local_dir, dirs_exist_ok=True)
        return sum(1 for _ in _walk(local_dir))
    root = _fs(source)._strip_protocol(source).rstrip("/")
    files = [str(f) for f in _retry(source, lambda fs, p: fs.find(p))]
    for f in files:
        rel = f[len(root):].lstrip("/") if f.startswith(root) else f.rsplit("/", 1)[-1]
        dst = os.path.join(local_dir, rel)
        os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
        _retry(source, lambda fs, _p, f=f, dst=dst: fs.get_file(f, dst))
    return len(files)


@contextlib.contextmanager
def local_work_dir(path: str):
    """A local directory standing for ``path``: the path itself when local, else a temporary directory whose content is
    uploaded to ``path`` on a clean exit."""
    if not is_cloud_path(path):
        p = _local(path)
        os.makedirs(p, exist_ok=True)
        yield p
        return
    with tempfile.TemporaryDirectory(prefix="isoexec-up-") as tmp:
        yield tmp
        upload_directory(tmp, path)


@contextlib.contextmanager
def local_read_dir(path: str):
    """A local directory with the content of ``path``: the path itself when local, else a temporary download."""
    if not is_cloud_path(path):
        if not os.path.exists(_local(path)):
            raise FileNotFoundError(f"path does not exist: {path}")
        yield _local(path)
        return
    with tempfile.TemporaryDirectory(prefix="isoexec-down-") as tmp:
        if download_directory(path, tmp) == 0:
            raise FileNotFoundError(f"nothing under {path}")
        yield tmp


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
