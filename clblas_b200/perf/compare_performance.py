#!/usr/bin/env python
"""Side-by-side table of two performance tables in the reference's CSV schema.

Text counterpart of the reference's plotting script (src/scripts/perf/plotPerformance.py, which overlays the GFLOPS
curves of several CSV files): for every problem size of the first table it prints the row of the second table with the
nearest size and the ratio of the two GFLOPS columns.

    python clblas_b200/perf/compare_performance.py doc/performance/B200/clblas_b200_dgemm_col_nt.csv published.csv
"""
from __future__ import annotations

import csv
import sys


def load(path: str) -> list[tuple[int, float, str]]:
    rows = []
    with open(path, newline="") as f:
        for r in csv.DictReader(f):
            try:
                rows.append((int(r["m"]), float(r["GFLOPS"]), r.get("label", "")))
            except (KeyError, ValueError):
                continue
    return rows


def main(argv: list[str]) -> int:
    if len(argv) != 3:
        print(__doc__, file=sys.stderr)
        return 2
    a, b = load(argv[1]), load(argv[2])
    if not a or not b:
        print("no rows with m and GFLOPS columns", file=sys.stderr)
        return 1
    print(f"# A = {argv[1]}\n# B = {argv[2]}")
    print(f"{'m (A)':>8} {'GFLOPS A':>12} {'m (B)':>8} {'GFLOPS B':>12} {'A / B':>8}")
    for m, ga, _ in a:
        mb, gb, _ = min(b, key=lambda r: abs(r[0] - m))
        print(f"{m:8d} {ga:12.1f} {mb:8d} {gb:12.1f} {ga / gb if gb else float('inf'):8.1f}")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
