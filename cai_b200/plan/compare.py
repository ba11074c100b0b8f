"""Compare two op timelines of the same plan, kernel kind by kernel kind.

Typical use: the measured timeline of a step (``python -m cai_b200.trainer ... --trace measured.csv``) against the one
the calibrated backend predicts for the same plan (``bin/trainer plan topo --backend calibrated --trace predicted.csv``).
Ops are matched by their index in the plan; the table lists, per op kind and stream, the summed durations of both files
and their ratio, largest absolute difference first: the kernels that are off their model are where to look next.

    python -m cai_b200.plan.compare measured.csv predicted.csv
"""
from __future__ import annotations

import argparse
import csv
import json
from collections import defaultdict


def load(path):
    """``{op_index: (kind, stream, duration in us)}`` from a CSV (reference schema) or a Trace Event JSON file."""
    out = {}
    if str(path).endswith(".json"):
        with open(path) as f:
            doc = json.load(f)
        names = {e["tid"]: e["args"]["name"] for e in doc["traceEvents"] if e.get("ph") == "M"}
        for e in doc["traceEvents"]:
            if e.get("ph") == "X":
                out[int(e["args"]["op"])] = (e["name"], names.get(e["tid"], str(e["tid"])), float(e["dur"]))
        return out
    with open(path) as f:
        for r in csv.DictReader(f):
            out[int(r["op_index"])] = (r["kind"], r["stream"], float(r["dur_us"]))
    return out


def compare(a_path, b_path):
    a, b = load(a_path), load(b_path)
    common = sorted(set(a) & set(b))
    rows = defaultdict(lambda: [0, 0.0, 0.0])
    mismatched = 0
    for i in common:
        if a[i][0] != b[i][0]:
            mismatched += 1
            continue
        r = rows[(a[i][0], a[i][1])]
        r[0] += 1
        r[1] += a[i][2]
        r[2] += b[i][2]
    table = [{"kind": k, "stream": s, "ops": n, "a_ms": x / 1e3, "b_ms": y / 1e3, "ratio": (x / y if y else float("inf"))}
             for (k, s), (n, x, y) in rows.items()]
    table.sort(key=lambda r: -abs(r["a_ms"] - r["b_ms"]))
    return table, {"only_a": len(set(a) - set(b)), "only_b": len(set(b) - set(a)), "kind_mismatch": mismatched}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("a", help="first timeline (e.g. measured), CSV or Trace Event JSON")
    ap.add_argument("b", help="second timeline (e.g. predicted)")
    a = ap.parse_args(argv)
    table, odd = compare(a.a, a.b)
    print(f"{'kind':<20} {'stream':<11} {'ops':>5} | {'a ms':>9} | {'b ms':>9} | a / b")
    for r in table:
        print(f"{r['kind']:<20} {r['stream']:<11} {r['ops']:5d} | {r['a_ms']:9.3f} | {r['b_ms']:9.3f} | {r['ratio']:5.2f}")
    ta, tb = sum(r["a_ms"] for r in table), sum(r["b_ms"] for r in table)
    print(f"{'sum of op durations':<38} | {ta:9.3f} | {tb:9.3f} | {ta / tb if tb else float('inf'):5.2f}")
    if any(odd.values()):
        print(f"unmatched: {odd}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
