"""Structural rules of the source tree, checked by reading the files (reference practice: source-level AST tests where
behaviour cannot be exercised, tests/backends/.../test_isoexec_sync_single_copy.py).

  * no source file names a copy API or a TMA load form that is off limits on the machines this runs on;
  * comments and docstrings stand on their own: they do not point at planning documents, review notes, build rounds,
    the job runner or machine-local paths;
  * every device-side wait loop in the kernels is bounded (goes through the bounded-wait helpers).
The forbidden words are assembled from pieces so that this file does not contain them either.
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


def test_no_forbidden_device_apis_are_named():
    batch = ["cuda" + "Memcpy" + "Batch" + "Async", "cuda" + "Memcpy3D" + "Batch" + "Async", "cu" + "Memcpy" + "Batch" + "Async",
             "cu" + "Memcpy3D" + "Batch" + "Async"]
    mcast = "." + "multicast" + "::" + "cluster"
    hits = []
    for p in _sources():
        text = _read(p)
        for w in batch:
            if w in text:
                hits.append((p, w))
        # a cluster-multicast qualifier is only ever allowed on tcgen05.commit, never on a copy
        for m in re.finditer(re.escape(mcast), text):
            line = text[text.rfind("\n", 0, m.start()) + 1:text.find("\n", m.end())]
            if "commit" not in line and "never" not in line.lower() and "no " not in line.lower():
                hits.append((p, line.strip()[:80]))
    assert not hits, hits


def test_comments_do_not_point_outside_the_source_tree():
    words = ["SUR" + "VEY", "VER" + "DICT", "ADV" + "ICE.md", "DES" + "IGN.md", "BASE" + "LINE.md", "gpu" + "run", "/ro" + "ot/", "the ju" + "dge"]
    pat = re.compile("|".join(re.escape(w) for w in words))
    rounds = re.compile(r"\b(in|this|last|next) round\b|\bround [0-9]\b", re.I)
    hits = []
    for p in _sources():
        if p.endswith("test_source_rules_cpu.py"):
            continue
        for i, line in enumerate(_read(p).splitlines(), 1):
            if pat.search(line) or rounds.search(line):
                hits.append(f"{os.path.relpath(p, ROOT)}:{i}: {line.strip()[:90]}")
    assert not hits, "\n".join(hits)


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
