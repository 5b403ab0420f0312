"""Structural rules of the kernel sources, checked by reading the files (reference practice: source-level AST tests
where behaviour cannot be exercised, tests/backends/.../test_isoexec_sync_single_copy.py).

Every device-side wait loop in the kernels is bounded: it goes through the bounded-wait helpers.
"""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC_EXT = (".py", ".cu", ".cuh", ".h", ".cpp")


def _sources():
    for top in ("skyrl_isoexec_b200", "tests", "profiles", "examples"):
        for d, _, files in os.walk(os.path.join(ROOT, top)):
            if "__pycache__" in d or os.sep + "lib" in d:
                continue
            for f in files:
                if f.endswith(SRC_EXT):
                    yield os.path.join(d, f)
    for f in ("bench.py", "__graft_entry__.py"):
        yield os.path.join(ROOT, f)


def _read(path):
    with open(path, errors="replace") as f:
        return f.read()


def test_every_kernel_wait_loop_is_bounded():
    """A ``while`` that polls a barrier or a flag must be the bounded helper itself; everything else calls it."""
    bad, seen = [], 0
    csrc = os.path.join(ROOT, "skyrl_isoexec_b200", "csrc")
    for f in sorted(os.listdir(csrc)):
        if not f.endswith((".cu", ".cuh")):
            continue
        text = _read(os.path.join(csrc, f))
        for m in re.finditer(r"while\s*\(([^;{]*?)\)\s*[{;]", text):
            cond = m.group(1)
            if re.search(r"try_wait|ld_acquire|volatile|\*\s*flag|flags\[", cond):
                seen += 1
                # the loop body (next ~600 characters) has to consult the clock or an iteration limit
                body = text[m.end():m.end() + 600]
                if not re.search(r"globaltimer|kWaitLimit|limit|max_iter|spins", body):
                    bad.append((f, cond.strip()[:60]))
    assert not bad, bad
    assert seen >= 4          # the scan really found the polling loops (mbarrier helper, peer flags)
