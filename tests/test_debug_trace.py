"""Digest properties and the comparator's fault matrix: a two-sided fake pipeline with injected
divergence, one test per guarantee (first divergence, contamination, missing records, rank
awareness, ladder level, format refusal, torch-free CLI)."""
import json
import os
import subprocess
import sys

import torch

from skyrl_isoexec_b200.debug import compare, thash, trace


def test_digest_is_order_invariant_over_rows_and_sensitive_to_bits():
    x = torch.randn(17, 33)
    perm = torch.randperm(17)
    assert thash.digest(x) == thash.digest(x[perm])
    y = x.clone()
    y[3, 5] = -y[3, 5]
    assert thash.digest(x) != thash.digest(y)
    z = torch.zeros(4, 4)
    nz = z.clone()
    nz[0, 0] = -0.0
    assert thash.digest(z) != thash.digest(nz)                      # signed zero is visible
    assert thash.row_digests(x)[perm].tolist() == thash.row_digests(x[perm]).tolist()
    b = x.bfloat16()
    assert thash.digest(b) == thash.digest(b.clone())


def test_ladder_tells_how_many_low_bits_differ():
    x = torch.randn(8, 16)
    y = x.clone()
    yi = y.view(torch.int32)
    yi[2, 3] ^= 0b11                                                 # flip the two lowest mantissa bits
    lx, ly = thash.ladder(x), thash.ladder(y)
    assert lx["0"] != ly["0"] and lx["1"] != ly["1"] and lx["2"] == ly["2"] and lx["8"] == ly["8"]


def _pipeline(directory, side, rank, inject=None, drop=None, keys=None, regions=("embed", "layer0.out", "layer1.out", "final_norm")):
    """A fake forward: each region is a deterministic function of the previous one."""
    tr = trace.Tracer(directory, side, rank)
    keys = keys or [("s0", i) for i in range(6)]
    tr.begin_forward("trainer_score" if side == "trainer" else "engine_decode", keys)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(len(keys), 8, generator=g)
    for r in regions:
        x = x * 1.5 + 0.25
        if inject == r:
            x = x.clone()
            x.view(torch.int32)[1, 2] ^= 1
        if drop != r:
            tr.record(r, x)
    tr.close()
    return tr.path


def test_clean_traces_compare_equal(tmp_path):
    a = _pipeline(str(tmp_path / "a"), "trainer", 0)
    b = _pipeline(str(tmp_path / "b"), "engine", 0)
    code, rep = compare.compare(a, b)
    assert code == 0 and rep["first_divergence"] is None and rep["regions"] == 4 and rep["compared_rows"] == 24


def test_first_divergence_and_contamination(tmp_path):
    a = _pipeline(str(tmp_path / "a"), "trainer", 0)
    b = _pipeline(str(tmp_path / "b"), "engine", 0, inject="layer0.out")
    code, rep = compare.compare(a, b)
    assert code == 2
    assert rep["first_divergence"]["region"] == "layer0.out" and rep["first_divergence"]["rows_differing"] == 1
    assert rep["first_divergence"]["example_row"] == ["s0", 1]
    assert rep["contaminated"] == ["layer1.out", "final_norm"]     # downstream of the first, not separate findings


def test_missing_region_and_rows_are_reported(tmp_path):
    a = _pipeline(str(tmp_path / "a"), "trainer", 0)
    b = _pipeline(str(tmp_path / "b"), "engine", 0, drop="layer1.out", keys=[("s0", i) for i in range(4)])
    code, rep = compare.compare(a, b)
    assert code == 0 and rep["missing_regions"] == ["layer1.out"]
    assert rep["missing_rows"]["embed"] == 2


def test_disjoint_rows_are_inconclusive_not_clean(tmp_path):
    a = _pipeline(str(tmp_path / "a"), "trainer", 0, keys=[("s0", i) for i in range(4)])
    b = _pipeline(str(tmp_path / "b"), "engine", 0, keys=[("s9", i) for i in range(4)])
    assert compare.compare(a, b)[0] == 3


def test_same_side_different_ranks_are_not_compared(tmp_path):
    a = _pipeline(str(tmp_path / "a"), "trainer", 0)
    b = _pipeline(str(tmp_path / "b"), "trainer", 1, inject="embed")
    code, rep = compare.compare(a, b)
    assert code == 3 and "ranks" in rep["note"]


def test_format_refusal_and_torch_free_cli(tmp_path):
    bad = tmp_path / "bad.jsonl"
    bad.write_text('{"format":"something-else"}\n')
    good = _pipeline(str(tmp_path / "a"), "trainer", 0)
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    # the CLI must work with torch made unimportable
    prog = ("import sys; sys.modules['torch'] = None\n"
            "from skyrl_isoexec_b200.debug.compare import main\n"
            f"sys.exit(main([{str(good)!r}, {str(bad)!r}]))")
    r = subprocess.run([sys.executable, "-c", prog], env=env, capture_output=True, text=True)
    assert r.returncode == 1 and "bad input" in r.stderr
    prog2 = prog.replace(repr(str(bad)), repr(str(good)))
    r = subprocess.run([sys.executable, "-c", prog2], env=env, capture_output=True, text=True)
    assert r.returncode == 0 and json.loads(r.stdout)["compared_rows"] == 24


def test_model_doors_record_when_tracer_is_active(tmp_path):
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM, ForwardCtx
    from skyrl_isoexec_b200.ops import functional as F

    cfg = get_config("tiny-qwen3")
    m = DecoderLM(cfg)
    tr = trace.install("trainer", 0, str(tmp_path))
    try:
        tr.begin_forward("trainer_score", [("s", i) for i in range(20)])
        ids = torch.randint(0, cfg.vocab_size, (20,))
        with torch.no_grad():
            m(ids, ForwardCtx(torch.arange(20, dtype=torch.int32), F.AttnMeta.packed([20], 4, 2, "cpu")))
    finally:
        trace.uninstall()
    _, recs = compare.load(tr.path)
    assert [r["region"] for r in recs] == ["layer0.out", "layer1.out", "final_norm"] and "rows" in recs[0]
