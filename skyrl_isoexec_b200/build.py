"""Build the native library in-tree: every ``csrc/*.cu`` -> ``lib/libisoexec_b200.so``.

The kernels are plain CUDA (no torch headers) behind ``extern "C"`` launchers, so a
full rebuild takes seconds and cross-compiles for sm_100a on a box without a GPU.
Python reaches the launchers through ``ctypes`` (``skyrl_isoexec_b200.ops._native``).

Usage: ``python -m skyrl_isoexec_b200.build [--force] [--verbose]``
"""

from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "lib" / "obj"
LIB = PKG / "lib" / "libisoexec_b200.so"
CPU_SRC = PKG / "csrc_cpu" / "ops_cpu.cpp"
CPU_LIB = PKG / "lib" / "libisoexec_cpu.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return exe


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if stale) and return the path of the shared library."""
    srcs = sources()
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    stamp = OBJ / "stamp.txt"
    want = _digest(srcs + headers)
    if not force and LIB.exists() and stamp.exists() and stamp.read_text() == want:
        return LIB
    OBJ.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    link = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(want)
    return LIB


def build_cpu(force: bool = False) -> Path:
    """Compile the CPU oracle / CPU-route library (g++, OpenMP, no FMA contraction)."""
    stamp = OBJ / "stamp_cpu.txt"
    want = hashlib.sha256(CPU_SRC.read_bytes()).hexdigest()
    if not force and CPU_LIB.exists() and stamp.exists() and stamp.read_text() == want:
        return CPU_LIB
    OBJ.mkdir(parents=True, exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
           "-fvisibility=hidden", str(CPU_SRC), "-o", str(CPU_LIB)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(want)
    return CPU_LIB


def build_all(force: bool = False, verbose: bool = False) -> tuple[Path, Path]:
    return build(force, verbose), build_cpu(force)


if __name__ == "__main__":
    for path in build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv):
        print(path)
