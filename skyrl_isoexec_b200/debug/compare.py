"""Offline comparator for two debug traces: where and how do the two runtimes diverge.
Standard library only, so it runs on a machine without torch (reference: ISO/debug/compare.py:291-707).

    python -m skyrl_isoexec_b200.debug TRACE_A.jsonl TRACE_B.jsonl

Exit codes: 0 clean (every common row of every common region agrees), 2 divergence found,
3 inconclusive (nothing comparable: no common regions or no common rows), 1 bad input.

Guarantees: the FIRST divergence is reported in trace A's region order (causal order of the
forward); later differing regions are listed as *contaminated* (downstream of the first); regions
or rows present on one side only are listed as missing, never silently skipped; the ladder level
at which a differing row starts to agree tells how many low mantissa bits differ; records of
different ranks are never compared with one another.
"""

import json
import sys

FORMAT = "isoexec-trace-1"


class TraceFormatError(Exception):
    pass


def load(path):
    try:
        with open(path) as f:
            lines = [ln for ln in f.read().splitlines() if ln.strip()]
    except OSError as e:
        raise TraceFormatError(f"{path}: {e}")
    if not lines:
        raise TraceFormatError(f"{path}: empty trace")
    try:
        head = json.loads(lines[0])
        recs = [json.loads(ln) for ln in lines[1:]]
    except ValueError as e:
        raise TraceFormatError(f"{path}: not JSONL ({e})")
    if not isinstance(head, dict) or head.get("format") != FORMAT:
        raise TraceFormatError(f"{path}: unknown trace format {head.get('format') if isinstance(head, dict) else head!r}")
    for r in recs:
        if not isinstance(r, dict) or "region" not in r or "digest" not in r:
            raise TraceFormatError(f"{path}: record without region/digest")
    return head, recs


def _rows_by_key(rec):
    """{(key tuple): {k: digest}} for a record that carries row digests."""
    if "rows" not in rec or "row_keys" not in rec:
        return None
    out = {}
    for j, key in enumerate(rec["row_keys"]):
        out[tuple(key)] = {k: v[j] for k, v in rec["rows"].items()}
    return out


def _collect(recs):
    """region -> {row key -> ladder digests}, merged over every record of the region (first write wins)."""
    order, table, whole = [], {}, {}
    for r in recs:
        reg = r["region"]
        if reg not in table:
            order.append(reg)
            table[reg] = {}
            whole[reg] = []
        rows = _rows_by_key(r)
        if rows is None:
            whole[reg].append(r["digest"])
        else:
            for k, v in rows.items():
                table[reg].setdefault(k, v)
    return order, table, whole


def _agree_level(a, b, ladder):
    for k in ladder:
        if a.get(str(k)) == b.get(str(k)):
            return k
    return None


def compare(path_a, path_b):
    ha, ra = load(path_a)
    hb, rb = load(path_b)
    report = {"a": path_a, "b": path_b, "first_divergence": None, "contaminated": [], "missing_regions": [],
              "missing_rows": {}, "compared_rows": 0, "regions": 0, "rank_a": ha.get("rank"), "rank_b": hb.get("rank")}
    if ha.get("side") == hb.get("side") and ha.get("rank") != hb.get("rank"):
        report["note"] = "same side, different ranks: records are shards of one tensor, not comparable"
        return 3, report
    ladder = ha.get("ladder", [0])
    order_a, tab_a, whole_a = _collect(ra)
    order_b, tab_b, whole_b = _collect(rb)
    report["missing_regions"] = [r for r in order_a if r not in tab_b] + [r for r in order_b if r not in tab_a]
    for reg in order_a:
        if reg not in tab_b:
            continue
        rows_a, rows_b = tab_a[reg], tab_b[reg]
        common = [k for k in rows_a if k in rows_b]
        only = (len(rows_a) - len(common)) + (len(rows_b) - len(common))
        if only:
            report["missing_rows"][reg] = only
        if not common:
            # fall back to whole-tensor digests when both sides recorded exactly one
            if len(whole_a[reg]) == 1 and len(whole_b[reg]) == 1:
                report["regions"] += 1
                report["compared_rows"] += 1
                if whole_a[reg][0].get("0") != whole_b[reg][0].get("0"):
                    lvl = _agree_level(whole_a[reg][0], whole_b[reg][0], ladder)
                    entry = {"region": reg, "rows_differing": 1, "rows_compared": 1, "agree_from_ladder_level": lvl, "example_row": None}
                    if report["first_divergence"] is None:
                        report["first_divergence"] = entry
                    else:
                        report["contaminated"].append(reg)
            continue
        report["regions"] += 1
        report["compared_rows"] += len(common)
        bad = [k for k in common if rows_a[k].get("0") != rows_b[k].get("0")]
        if bad:
            levels = [_agree_level(rows_a[k], rows_b[k], ladder) for k in bad]
            worst = None if any(l is None for l in levels) else max(levels)
            entry = {"region": reg, "rows_differing": len(bad), "rows_compared": len(common),
                     "agree_from_ladder_level": worst, "example_row": list(bad[0])}
            if report["first_divergence"] is None:
                report["first_divergence"] = entry
            else:
                report["contaminated"].append(reg)
    if report["first_divergence"] is not None:
        return 2, report
    if report["compared_rows"] == 0:
        return 3, report
    return 0, report


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        sys.stderr.write("usage: python -m skyrl_isoexec_b200.debug TRACE_A TRACE_B\n")
        return 1
    try:
        code, rep = compare(argv[0], argv[1])
    except TraceFormatError as e:
        sys.stderr.write(f"bad input: {e}\n")
        return 1
    print(json.dumps(rep, indent=1))
    return code
