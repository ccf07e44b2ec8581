#!/usr/bin/env python
"""Performance sweep around the native client, writing the reference's CSV schema.

Counterpart of the reference's sweep driver (src/scripts/perf/measurePerformance.py) for the B200
library: size arguments take the same list / range syntax ("1024", "512-8192:512", "15,2048-3000"),
every combination is run through `clblas_b200_client`, and one row per run is written with the
header of the reference's published tables (doc/performance/**.csv):

    m,n,k,lda,ldb,ldc,offa,offb,offc,alpha,beta,order,transa,transb,side,uplo,diag,function,device,library,numQueues,label,GFLOPS

    python clblas_b200/perf/measure_performance.py -f gemm -r s --transb transpose -s 512-8192:512 \
        --label sgemm_col_nt_b200 -o sgemm_col_nt_b200.csv
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CLIENT = os.path.join(HERE, "..", "lib", "clblas_b200_client")
HEADER = ("m,n,k,lda,ldb,ldc,offa,offb,offc,alpha,beta,order,transa,transb,side,uplo,diag,function,device,library,"
          "numQueues,label,GFLOPS")


def expand(spec: str) -> list[int]:
    """'1024' -> [1024]; '100-800:100' -> 100, 200, ..., 800; comma-separated pieces are concatenated."""
    out: list[int] = []
    for piece in spec.split(","):
        m = re.fullmatch(r"(\d+)(?:-(\d+)(?::(\d+))?)?", piece.strip())
        if not m:
            raise ValueError(f"bad size specification: {piece!r}")
        lo = int(m.group(1))
        hi = int(m.group(2)) if m.group(2) else lo
        step = int(m.group(3)) if m.group(3) else (hi - lo or 1)
        out.extend(range(lo, hi + 1, step))
    return out


TRANS = {"none": 0, "transpose": 1, "conj": 2}


def main() -> int:
    ap = argparse.ArgumentParser(description="Measure performance of the clblas_b200 library")
    ap.add_argument("-s", "--square", help="sizes used for m, n and k together")
    ap.add_argument("-m", "--sizem"), ap.add_argument("-n", "--sizen"), ap.add_argument("-k", "--sizek")
    ap.add_argument("-f", "--function", default="gemm", choices=["gemm", "trsm", "trmm", "syrk", "syr2k", "symm"])
    ap.add_argument("-r", "--precision", default="s", choices=["s", "d", "c", "z"])
    ap.add_argument("--order", default="column", choices=["row", "column"])
    ap.add_argument("--transa", default="none", choices=list(TRANS)), ap.add_argument("--transb", default="none", choices=list(TRANS))
    ap.add_argument("--side", default="left", choices=["left", "right"])
    ap.add_argument("--uplo", default="upper", choices=["upper", "lower"])
    ap.add_argument("--diag", default="unit", choices=["unit", "nonunit"])
    ap.add_argument("--alpha", type=float, default=1.0), ap.add_argument("--beta", type=float, default=1.0)
    ap.add_argument("--path", type=int, default=0, help="clblasB200SetGemmPath value (4 = 3xTF32 SGEMM)")
    ap.add_argument("-p", "--profile", type=int, default=10), ap.add_argument("--apiCallCount", type=int, default=10)
    ap.add_argument("--label", default="b200")
    ap.add_argument("-o", "--output", default="-")
    a = ap.parse_args()

    if a.square:
        sizes = [(v, v, v) for v in expand(a.square)]
    else:
        ms, ns = expand(a.sizem or "1024"), expand(a.sizen or "1024")
        ks = expand(a.sizek or "1024")
        sizes = [(m, n, k) for m in ms for n in ns for k in ks]
    if not os.path.exists(CLIENT):
        print(f"{CLIENT} is missing: run python clblas_b200/build.py", file=sys.stderr)
        return 2
    out = sys.stdout if a.output == "-" else open(a.output, "w")
    print(HEADER, file=out)
    for m, n, k in sizes:
        cmd = [CLIENT, "-f", a.function, "-r", a.precision, "-m", str(m), "-n", str(n), "-k", str(k),
               "-o", "1" if a.order == "column" else "0", "--transposeA", str(TRANS[a.transa]),
               "--transposeB", str(TRANS[a.transb]), "--side", "0" if a.side == "left" else "1",
               "--uplo", "0" if a.uplo == "upper" else "1", "--diag", "0" if a.diag == "unit" else "1",
               "--alpha", str(a.alpha), "--beta", str(a.beta), "-p", str(a.profile), "--apiCallCount", str(a.apiCallCount),
               "--path", str(a.path)]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
        g = re.search(r"Gflops < .* >: ([0-9.eE+-]+)", r.stdout)
        if r.returncode != 0 or not g:
            print(f"run failed for m={m} n={n} k={k}: {r.stderr.strip()[-200:]}", file=sys.stderr)
            continue
        print(f"{m},{n},{k},0,0,0,0,0,0,{a.alpha:g},{a.beta:g},{a.order},{a.transa},{a.transb},{a.side},{a.uplo},{a.diag},"
              f"{a.precision}{a.function},gpu,clblas_b200,1,{a.label},{float(g.group(1)):.2f}", file=out)
        out.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
