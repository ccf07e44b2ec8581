#!/usr/bin/env python
"""Benchmark of the level-3 hot path on B200, in the protocol of the reference's client
(src/client/client.cpp:497, :574-592: untimed warm-up, then back-to-back enqueued calls timed as a
block; GFLOP/s = 2*M*N*K / t, src/client/clfunc_xgemm.hpp:95-98; TRSM M*(M+1)*N / t,
src/client/clfunc_xtrsm.hpp:70-80) with CUDA events in place of gettimeofday.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload sgemm32768|dgemm8192|...] [--no-also]
    python bench.py --impl reference ...     # the reference's own CPU code on the host cores

One step = one call of the workload through the clBLAS-shaped C ABI.  The default workload is the
SGEMM column-major N/T, M=N=K=32768, U[-1,1], alpha=1, beta=0 (three 4 GiB matrices).  With N > 1 ranks
(torchrun, one process per GPU) the fixed problem is split: rank r owns a column block of op(B) and C
(boundaries multiples of 128) and A is broadcast from rank 0 inside every step by the library's sharded
entry point (NCCL in panels on a second stream, panel products behind events) -- strong scaling, so the
1 -> N ratio of `value` is the speed-up.  Rank 0 prints ONE JSON line.  Besides the headline it carries

* "also": short, separately timed records of the other workloads -- DGEMM T/N 8192^3 (per-rank columns fixed:
  weak), SGEMM N/T 8192^3 (weak), DTRSM 8192 x 16384 (right-hand sides split: strong) at every N; SGEMM N/N
  1024^3 and the ragged row-major SGEMM at N = 1 -- and "timed_region_s_total", the sum of all timed regions;
* "parity": after the timed regions the result of one more call is checked on every rank's shard against a
  float64 host evaluation of sampled rows x columns of the SAME device data (first / last rows and columns
  always included; C pre-filled with NaN where beta = 0; NaN in the triangle of A that must not be read),
  as a fraction of the bound 4*K*u (GEMM, on |alpha||A||B| + |beta||C|) or 4*M*u (TRSM, backward error);
  the worst fraction over the ranks is printed and the process exits non-zero when it exceeds 1.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NOMINAL = {"fp32": 148 * 128 * 2 * 1.965e9 / 1e12, "fp64": 148 * 64 * 2 * 1.965e9 / 1e12}
# enums of src/clBLAS.h:78-113 (the package is not imported at module level: the reference arm must not map it)
ROW_MAJOR, COL_MAJOR, NO_TRANS, TRANS = 0, 1, 0, 1
LEFT, LOWER, NON_UNIT = 0, 1, 1

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum), captured with ncu
# at the workload's full size where the capture is one pass (profiles/dram_traffic_full_size.md).  None where no
# capture of that workload exists: the 32768^3 SGEMM (12 GB, launches of over a second) is beyond what a capture may
# hold, and its traffic cannot be scaled from a smaller case (8192^3 -> 16384^3: 8x the flops, 26x the bytes).  The
# DTRSM figure is the sum over the 43 launches of one call.
NCU_TRAFFIC_BYTES = {
    "sgemm1024": int(12.63e6),
    "dgemm8192": int(6.107e9 + 509.2e6 + 620.1e6 + 12.4e6),
    "sgemm_ragged": int(94.89e6 + 18.84e6),
    "dtrsm8192": int(7.93e9 + 1.75e9),
    "sgemm32768": None,
    "sgemm8192": int(3.257e9 + 263.6e6),
}
NCU_TRAFFIC_BYTES_3XTF32 = {"sgemm8192": int(2.70e9 + 256.35e6)}
ALIASES = {"cfg1": "sgemm1024", "cfg2": "dgemm8192", "cfg3": "sgemm_ragged", "cfg4": "dtrsm8192", "cfg5": "sgemm32768"}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------

def plan_shards(total, parts, align=128):
    """Same arithmetic as clblasB200PlanShards (equal shares rounded up to the alignment)."""
    units = (total + align - 1) // align
    per = (units + parts - 1) // parts
    return [min(i * per * align, total) for i in range(parts)] + [total]


def _dt(prec):
    import torch
    return torch.float32 if prec == "s" else torch.float64


class GemmWorkload:
    kind = "gemm"

    def __init__(self, name, prec, order, transA, transB, M, N, K, alpha, beta, lda, ldb, ldc, offs=(0, 0, 0),
                 dist_kind="uniform", scaling="weak", sets=1, desc=""):
        self.name, self.prec, self.order, self.transA, self.transB = name, prec, order, transA, transB
        self.M, self.N, self.K, self.alpha, self.beta = M, N, K, alpha, beta
        self.lda, self.ldb, self.ldc, self.offs = lda, ldb, ldc, offs
        self.dist_kind, self.scaling, self.sets, self.desc = dist_kind, scaling, sets, desc
        self.pipe = "fp32" if prec == "s" else "fp64"
        self.metric = ("SGEMM" if prec == "s" else "DGEMM") + " TFLOP/s"

    def local_n(self, rank, world):
        if world == 1 or self.scaling == "weak":
            return self.N
        b = plan_shards(self.N, world)
        return b[rank + 1] - b[rank]

    def flops(self, world):
        n_total = self.N * world if self.scaling == "weak" else self.N
        return 2.0 * self.M * n_total * self.K

    def local_flops(self, rank, world):
        return 2.0 * self.M * self.local_n(rank, world) * self.K

    def min_bytes(self, n_local=None):
        n = self.N if n_local is None else n_local
        e = 4 if self.prec == "s" else 8
        return (self.M * self.K + self.K * n + self.M * n * (2 if self.beta != 0 else 1)) * e

    def ldb_local(self, nl, world):
        """A rank's block of a transposed B (stored N x K) in a split problem is held on its own, nl rows per column."""
        if world > 1 and self.scaling == "strong" and self.order == COL_MAJOR and self.transB != NO_TRANS:
            return max(nl, 1)
        return self.ldb

    def _stored(self, trans, rows, cols):
        tra = (self.order == COL_MAJOR and trans == NO_TRANS) or (self.order == ROW_MAJOR and trans != NO_TRANS)
        return (rows, cols) if tra else (cols, rows)

    def lengths(self, nl, world=1):
        def length(trans, rows, cols, ld, off):
            inner, outer = self._stored(trans, rows, cols)
            return off + (outer - 1) * ld + inner
        return (length(self.transA, self.M, self.K, self.lda, self.offs[0]),
                length(self.transB, self.K, max(nl, 1), self.ldb_local(nl, world), self.offs[1]),
                length(NO_TRANS, self.M, max(nl, 1), self.ldc, self.offs[2]))

    def alloc(self, rank, world, device, host=False):
        """Flat buffers for A (stored), B_local, C_local in the workload's own layout."""
        import torch
        dt = _dt(self.prec)
        gen = torch.Generator(device=device)
        gen.manual_seed(12345 + rank)
        out = []
        for n in self.lengths(self.local_n(rank, world), world):
            if self.dist_kind == "normal":
                t = torch.empty(n, dtype=dt, device=device).normal_(generator=gen)
            else:
                t = torch.empty(n, dtype=dt, device=device).uniform_(-1.0, 1.0, generator=gen)
            out.append(t.cpu().pin_memory() if host else t)
        return out

    def call(self, cb, bufs, rank, world, comm=None):
        A, B, C = bufs
        nl = self.local_n(rank, world)
        if world == 1:
            fn = cb.clblasSgemm if self.prec == "s" else cb.clblasDgemm
            return fn(self.order, self.transA, self.transB, self.M, nl, self.K, self.alpha, A, self.offs[0], self.lda,
                      B, self.offs[1], self.ldb, self.beta, C, self.offs[2], self.ldc)
        fn = cb.clblasB200SgemmSharded if self.prec == "s" else cb.clblasB200DgemmSharded
        return fn(self.order, self.transA, self.transB, self.M, nl, self.K, self.alpha, A, self.offs[0], self.lda,
                  B, self.offs[1], self.ldb_local(nl, world), self.beta, C, self.offs[2], self.ldc, comm, 0)

    def call_local(self, cb, bufs, rank, world):
        """This rank's product alone (no collective): what the roofline figure is measured on."""
        return self.call(cb, bufs, 0, 1) if world == 1 or self.scaling == "weak" else \
            (cb.clblasSgemm if self.prec == "s" else cb.clblasDgemm)(
                self.order, self.transA, self.transB, self.M, self.local_n(rank, world), self.K, self.alpha, bufs[0], self.offs[0],
                self.lda, bufs[1], self.offs[1], self.ldb_local(self.local_n(rank, world), world), self.beta, bufs[2], self.offs[2], self.ldc)

    def call_host(self, cb, bufs):
        A, B, C = bufs
        fn = cb.clblasB200SgemmHost if self.prec == "s" else cb.clblasB200DgemmHost
        return fn(self.order, self.transA, self.transB, self.M, self.N, self.K, self.alpha, A, self.offs[0], self.lda,
                  B, self.offs[1], self.ldb, self.beta, C, self.offs[2], self.ldc)

    def parity(self, cb, bufs, rank, world, comm):
        """One more call on a poisoned C, then sampled entries against float64 on the host.  Returns error / bound."""
        import torch
        A, B, C = bufs
        nl = self.local_n(rank, world)
        if nl == 0:
            self.call(cb, bufs, rank, world, comm)
            return 0.0
        dev = C.device
        gen = torch.Generator(device=dev)
        gen.manual_seed(999 + rank)
        if self.beta == 0:
            C.fill_(float("nan"))                      # beta = 0 must never read C
        else:
            C.uniform_(-1.0, 1.0, generator=gen)
        C0 = C.clone()
        cb.check(self.call(cb, bufs, rank, world, comm), "parity call")
        torch.cuda.synchronize()
        r = np.random.Generator(np.random.Philox(key=[4711, rank]))
        rows = np.unique(np.concatenate([r.choice(self.M, size=min(40, self.M), replace=False), [0, self.M - 1]]))
        cols = np.unique(np.concatenate([r.choice(nl, size=min(40, nl), replace=False), [0, nl - 1]]))
        ri, ci = torch.from_numpy(rows).to(dev), torch.from_numpy(cols).to(dev)
        kk = torch.arange(self.K, device=dev)
        colmaj = self.order == COL_MAJOR

        def gather(buf, off, ld, trans, idx, other):
            # op(X)(i, k): column-major NoTrans -> i + k*ld; a transposition or row-major storage exchanges the two
            first_is_inner = (trans == NO_TRANS) == colmaj
            ii, oo = idx[:, None], other[None, :]
            flat = off + (ii + oo * ld if first_is_inner else oo + ii * ld)
            return buf[flat].cpu().numpy().astype(np.float64)

        Ar = gather(A, self.offs[0], self.lda, self.transA, ri, kk)                              # rows x K
        Bc = gather(B, self.offs[1], self.ldb_local(nl, world), NO_TRANS if self.transB != NO_TRANS else TRANS, ci, kk)   # cols x K
        idx = self.offs[2] + (ri[:, None] + ci[None, :] * self.ldc if colmaj else ci[None, :] + ri[:, None] * self.ldc)
        got = C[idx].cpu().numpy().astype(np.float64)
        exact = self.alpha * (Ar @ Bc.T)
        denom = abs(self.alpha) * (np.abs(Ar) @ np.abs(Bc).T)
        if self.beta != 0:
            c0 = C0[idx].cpu().numpy().astype(np.float64)
            exact += self.beta * c0
            denom += abs(self.beta) * np.abs(c0)
        u = 2.0 ** -24 if self.prec == "s" else 2.0 ** -53
        ratio = float(np.max(np.abs(got - exact) / np.where(denom == 0, np.finfo(np.float64).tiny, denom)) / (4.0 * self.K * u))
        if self.beta == 0 and self.ldc == (self.M if colmaj else nl) and bool(torch.isnan(C[self.offs[2]:self.offs[2] + self.M * nl]).any()):
            ratio = float("inf")                       # an entry of C was not written
        if not np.isfinite(ratio):
            ratio = 1e30
        return ratio

    def config(self, world):
        set_bytes = sum(self.lengths(self.N)) * (4 if self.prec == "s" else 8)
        return {"workload": f"{self.name}: {self.desc}", "M": self.M, "N": self.N * (world if self.scaling == "weak" else 1),
                "K": self.K, "alpha": self.alpha, "beta": self.beta, "lda": self.lda, "ldb": self.ldb, "ldc": self.ldc,
                "offsets": list(self.offs),
                "l2": "inputs larger than L2" if set_bytes > 130e6 else "rotating buffer sets larger than L2",
                "buffer_sets": self.sets,
                "parallelism": f"column blocks of C over {world} GPUs, A broadcast over NCCL inside every step" if world > 1 else "1 GPU"}


class TrsmWorkload:
    kind, name, prec, scaling, pipe, metric = "trsm", "dtrsm8192", "d", "strong", "fp64", "DTRSM TFLOP/s"
    sets = 1

    def __init__(self):
        self.M, self.N, self.alpha = 8192, 16384, 1.0
        self.desc = "DTRSM column-major Left/Lower/NoTrans/NonUnit, A 8192x8192, B 8192x16384"

    def local_n(self, rank, world):
        b = plan_shards(self.N, world)
        return b[rank + 1] - b[rank]

    def flops(self, world):
        return float(self.M) * (self.M + 1) * self.N

    def local_flops(self, rank, world):
        return float(self.M) * (self.M + 1) * self.local_n(rank, world)

    def min_bytes(self, n_local=None):
        n = self.N if n_local is None else n_local
        return (self.M * (self.M + 1) // 2 + 2 * self.M * n) * 8

    def alloc(self, rank, world, device, host=False):
        import torch
        M, nl = self.M, self.local_n(rank, world)
        gen = torch.Generator(device=device)
        gen.manual_seed(12345)                               # the same A on every rank (rank 0's is the one that counts)
        A = torch.empty(M * M, dtype=torch.float64, device=device).uniform_(-1.0, 1.0, generator=gen) / M
        Av = A.view(M, M)                                   # Av[j, i] = A(i, j) column-major
        Av.diagonal().uniform_(1.0, 2.0, generator=gen)
        iu = torch.triu_indices(M, M, offset=1, device=device)
        Av[iu[1], iu[0]] = float("nan")                      # strictly upper part: must never be read
        del iu
        gen.manual_seed(12345 + 7 * (rank + 1))
        B = torch.empty(M * max(nl, 1), dtype=torch.float64, device=device).normal_(generator=gen)
        if host:
            return [A.cpu().pin_memory(), B.cpu().pin_memory()]
        return [A, B]

    def call(self, cb, bufs, rank, world, comm=None):
        A, B = bufs
        nl = self.local_n(rank, world)
        if world == 1:
            return cb.clblasDtrsm(COL_MAJOR, LEFT, LOWER, NO_TRANS, NON_UNIT, self.M, nl, self.alpha, A, 0, self.M, B, 0, self.M)
        return cb.clblasB200DtrsmSharded(COL_MAJOR, LEFT, LOWER, NO_TRANS, NON_UNIT, self.M, nl, self.alpha, A, 0, self.M,
                                         B, 0, self.M, comm, 0)

    def call_local(self, cb, bufs, rank, world):
        return cb.clblasDtrsm(COL_MAJOR, LEFT, LOWER, NO_TRANS, NON_UNIT, self.M, self.local_n(rank, world), self.alpha,
                              bufs[0], 0, self.M, bufs[1], 0, self.M)

    def call_host(self, cb, bufs):
        A, B = bufs
        return cb.clblasB200DtrsmHost(COL_MAJOR, LEFT, LOWER, NO_TRANS, NON_UNIT, self.M, self.N, self.alpha, A, 0, self.M, B, 0, self.M)

    def parity(self, cb, bufs, rank, world, comm):
        """Fresh right-hand sides, one more solve, entrywise backward error of sampled columns against the bound."""
        import torch
        A, B = bufs
        M, nl = self.M, self.local_n(rank, world)
        if nl == 0:
            self.call(cb, bufs, rank, world, comm)
            return 0.0
        gen = torch.Generator(device=B.device)
        gen.manual_seed(31337 + rank)
        B.normal_(generator=gen)
        B0 = B.clone()
        if world > 1 and rank != 0:
            A.fill_(float("nan"))                      # everything this rank uses of A must come from the broadcast
        cb.check(self.call(cb, bufs, rank, world, comm), "parity call")
        torch.cuda.synchronize()
        if not bool(torch.isfinite(B[: M * nl]).all()):
            return 1e30                                # the NaN triangle of A was read
        r = np.random.Generator(np.random.Philox(key=[4712, rank]))
        cols = np.unique(np.concatenate([r.choice(nl, size=min(24, nl), replace=False), [0, nl - 1]]))
        ci = torch.from_numpy(cols).to(B.device)
        X = B.view(-1, M)[ci].cpu().numpy().T
        R = B0.view(-1, M)[ci].cpu().numpy().T
        T = np.tril(np.nan_to_num(A.view(M, M).cpu().numpy().T, nan=0.0))
        res = np.abs(self.alpha * R - T @ X)
        den = np.abs(T) @ np.abs(X) + abs(self.alpha) * np.abs(R)
        return float(np.max(res / np.where(den == 0, np.finfo(np.float64).tiny, den)) / (4.0 * M * 2.0 ** -53))

    def config(self, world):
        return {"workload": f"{self.name}: {self.desc}", "M": self.M, "N": self.N, "alpha": self.alpha,
                "lda": self.M, "ldb": self.M, "l2": "inputs larger than L2", "buffer_sets": 1,
                "parallelism": f"right-hand-side columns over {world} GPUs, A broadcast over NCCL inside every step" if world > 1 else "1 GPU"}


def workloads():
    CM, RM, N_, T_ = COL_MAJOR, ROW_MAJOR, NO_TRANS, TRANS
    return {
        "sgemm1024": GemmWorkload("sgemm1024", "s", CM, N_, N_, 1024, 1024, 1024, 1.5, 0.5, 1024, 1024, 1024, sets=16,
                                  desc="SGEMM column-major N/N 1024^3, U[-1,1], alpha=1.5 beta=0.5"),
        "dgemm8192": GemmWorkload("dgemm8192", "d", CM, T_, N_, 8192, 8192, 8192, 1.0, 1.0, 8192, 8192, 8192, dist_kind="normal",
                                  scaling="weak", desc="DGEMM column-major T/N 8192^3, normal(0,1), alpha=beta=1, tight ld"),
        "sgemm_ragged": GemmWorkload("sgemm_ragged", "s", RM, T_, N_, 4099, 3001, 1537, -2.0, 0.25, 4099 + 16, 3001 + 32, 3001 + 8,
                                     offs=(7, 13, 5), sets=2,
                                     desc="SGEMM row-major T/N M=4099 N=3001 K=1537, padded ld, offsets 7/13/5, alpha=-2 beta=0.25"),
        "dtrsm8192": TrsmWorkload(),
        # the shape the reference publishes its own curves on (column-major N/T, m=n=k=ld, alpha=beta=1,
        # doc/performance/clBLAS_2.6.0/S9150/README.txt:21-35) at the size the FP32 target is stated for
        "sgemm8192": GemmWorkload("sgemm8192", "s", CM, N_, T_, 8192, 8192, 8192, 1.0, 1.0, 8192, 8192, 8192, scaling="weak",
                                  desc="SGEMM column-major N/T 8192^3, U[-1,1], alpha=beta=1"),
        "sgemm32768": GemmWorkload("sgemm32768", "s", CM, N_, T_, 32768, 32768, 32768, 1.0, 0.0, 32768, 32768, 32768,
                                   scaling="strong", desc="SGEMM column-major N/T 32768^3, U[-1,1], alpha=1 beta=0"),
    }


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def mark(self):
        return time.perf_counter()

    def summary(self, t0=None, t1=None):
        sm, smmax, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ts, ln in list(self.lines):
            if (t0 is not None and ts < t0) or (t1 is not None and ts > t1 + 0.15):
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0])); smmax.append(float(f[1])); power.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[4:8]):
                if val == "Active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples" if self.proc else "nvidia-smi unavailable"]}
        busy = [c for c, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": max(smmax), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm)}

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()


# ------------------------------------------------------------------------------------------------
# CPU legs: the reference's own CPU code (oracle/_ref) or its C restatement (oracle port)
# ------------------------------------------------------------------------------------------------

def cpu_reference_sample(wl, seconds_target=12.0, threads=None):
    """Times the reference's CPU implementation of the workload's routine on a bounded sample of the
    workload: a block of rows of the result (GEMM) or of right-hand-side columns (TRSM), each host
    thread working on its own slice through the reference's code.  Returns (TFLOP/s, cores, kind, text)."""
    import oracle
    from concurrent.futures import ThreadPoolExecutor
    oracle.build()
    kind = "reference" if oracle.have_ref() else "port"
    impl = "ref" if kind == "reference" else "port"
    os.environ.setdefault("OMP_NUM_THREADS", "1")
    threads = threads or os.cpu_count() or 1
    dt = np.float32 if wl.prec == "s" else np.float64
    g = np.random.Generator(np.random.Philox(key=[12345, 99]))

    if wl.kind == "trsm":
        n = 1024                                   # order of the sampled triangle
        A = np.tril(g.uniform(-1, 1, (n, n)) / n, -1) + np.diag(g.uniform(1, 2, n))
        Ab = np.asfortranarray(A).ravel(order="F").astype(dt)

        def work(cols):
            B = g.standard_normal(n * cols).astype(dt)
            t0 = time.perf_counter()
            oracle.trsm(oracle.ColumnMajor, oracle.Left, oracle.Lower, oracle.NoTrans, oracle.NonUnit, n, cols, 1.0,
                        Ab, 0, n, B, 0, n, impl=impl)
            return time.perf_counter() - t0

        probe = work(1)
        cols = max(1, int(seconds_target / max(probe, 1e-6)))
        cols = min(cols, 64)
        t0 = time.perf_counter()
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(work, [cols] * threads))
        el = time.perf_counter() - t0
        flops = float(n) * (n + 1) * cols * threads
        text = f"{threads} threads x (DTRSM Left/Lower order {n}, {cols} right-hand sides) through NaiveBlas::trsm"
        return flops / el / 1e12, threads, kind, text

    K = min(wl.K, 2048)
    cols = 64
    Bm = g.uniform(-1, 1, K * cols).astype(dt)

    def work(rows):
        A = g.uniform(-1, 1, rows * K).astype(dt)
        C = np.zeros(rows * cols, dtype=dt)
        t0 = time.perf_counter()
        # column-major rows x cols x K, A stored K x rows (T) or rows x K (N) as in the workload
        ta = oracle.Trans if wl.transA != 0 else oracle.NoTrans
        lda = K if ta == oracle.Trans else rows
        oracle.gemm(oracle.ColumnMajor, ta, oracle.NoTrans, rows, cols, K, wl.alpha, A, 0, lda, Bm, 0, K, wl.beta,
                    C, 0, rows, impl=impl)
        return time.perf_counter() - t0

    probe = work(8)
    rows = max(8, int(8 * seconds_target / max(probe, 1e-6)))
    rows = min(rows, 4096)
    t0 = time.perf_counter()
    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(work, [rows] * threads))
    el = time.perf_counter() - t0
    flops = 2.0 * rows * cols * K * threads
    text = f"{threads} threads x ({rows}x{cols}x{K} block of the workload's GEMM) through NaiveBlas::gemm"
    return flops / el / 1e12, threads, kind, text


def cpu_blas_sample(wl):
    """Netlib-interface BLAS of the host (the interface the reference test-suite links as its oracle,
    src/tests/correctness/blas-lapack.c:70, :124), all cores, on a bounded slice: informational."""
    try:
        from scipy.linalg import blas
    except Exception:
        return None
    dt = np.float32 if wl.prec == "s" else np.float64
    g = np.random.Generator(np.random.Philox(key=[12345, 98]))
    n = 4096
    if wl.kind == "trsm":
        A = np.asfortranarray(np.tril(g.uniform(-1, 1, (n, n)) / n, -1) + np.diag(g.uniform(1, 2, n)))
        B = np.asfortranarray(g.standard_normal((n, n)))
        blas.dtrsm(1.0, A, B, lower=1)
        t0 = time.perf_counter()
        blas.dtrsm(1.0, A, B, lower=1)
        el = time.perf_counter() - t0
        return {"value": float(n) * (n + 1) * n / el / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(),
                "lib": "scipy.linalg.blas (OpenBLAS)", "sample": f"dtrsm Left/Lower {n}x{n}, {n} right-hand sides"}
    A = np.asfortranarray(g.uniform(-1, 1, (n, n)).astype(dt))
    B = np.asfortranarray(g.uniform(-1, 1, (n, n)).astype(dt))
    f = blas.sgemm if wl.prec == "s" else blas.dgemm
    f(1.0, A, B)
    t0 = time.perf_counter()
    f(1.0, A, B, trans_a=1 if wl.transA else 0)
    el = time.perf_counter() - t0
    return {"value": 2.0 * n ** 3 / el / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(),
            "lib": "scipy.linalg.blas (OpenBLAS)", "sample": f"{'s' if wl.prec == 's' else 'd'}gemm {n}^3"}


def base_line(args, wl, world):
    """Keys shared by both arms (the reference arm must describe the same metric and configuration)."""
    return {"metric": wl.metric, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None,
            "dtype": "f32" if wl.prec == "s" else "f64", "data": "synthetic", "config": wl.config(world)}


def run_reference_arm(args, wl, world):
    """The reference's own CPU implementation of the routine (NaiveBlas compiled from the reference tree when it was
    built, else its C restatement) on all host cores; every step times a bounded block of the workload.  Loads
    nothing of the CUDA library."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    for _ in range(1 if args.warmup else 0):
        cpu_reference_sample(wl, seconds_target=2.0)
    vals, text, kind, cores = [], None, None, 0
    per_step = max(2.0, min(20.0, 120.0 / max(args.steps, 1)))
    t_all = time.perf_counter()
    for _ in range(args.steps):
        v, cores, kind, text = cpu_reference_sample(wl, seconds_target=per_step)
        vals.append(v)
    wall = time.perf_counter() - t_all
    value = float(np.mean(vals))
    line = dict(base_line(args, wl, world), impl="reference", value=value, ms_per_step=wall / args.steps * 1e3, gpu_launches=0,
                cpu_baseline={"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": text},
                e2e={"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------

class Runner:
    def __init__(self, args, cb, torch, dist, rank, world, local_rank, device, comm, sampler):
        self.args, self.cb, self.torch, self.dist = args, cb, torch, dist
        self.rank, self.world, self.local_rank, self.device, self.comm, self.sampler = rank, world, local_rank, device, comm, sampler
        self.timed_s = 0.0

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if self.world == 1:
            return v
        t = self.torch.tensor([v], device=self.device, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def gather(self, v):
        if self.world == 1:
            return [v]
        out = [None] * self.world
        self.dist.all_gather_object(out, v)
        return out

    def timed(self, fn, steps, warmup):
        """W untimed calls, then K calls timed with CUDA events on the launching stream between two barriers;
        returns (ms per step, max over ranks; launches of the region; wall-clock marks for the clock record)."""
        torch = self.torch
        for i in range(warmup):
            self.cb.check(fn(i), "warm-up call")
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = self.cb.launch_count()
        t0 = self.sampler.mark()
        e0.record()
        st = 0
        for i in range(steps):
            st = fn(warmup + i)
        e1.record()
        self.barrier()
        t1 = self.sampler.mark()
        self.cb.check(st, "timed call")
        ms = self.max_over_ranks(e0.elapsed_time(e1))
        self.timed_s += ms * 1e-3
        return ms / steps, self.cb.launch_count() - launches0, (t0, t1)

    def measure(self, wl, steps, warmup):
        """Device-resident throughput of one workload, the roofline figure of its dominant kernel and a parity check."""
        cb, torch = self.cb, self.torch
        sets = [wl.alloc(self.rank, self.world, self.device) for _ in range(wl.sets)]
        ms_per_step, launches, (t0, t1) = self.timed(lambda i: wl.call(cb, sets[i % len(sets)], self.rank, self.world, self.comm),
                                                     steps, warmup)
        value = wl.flops(self.world) / (ms_per_step * 1e-3) / 1e12
        kernel = cb.last_gemm_variant()
        clocks = self.sampler.summary(t0, t1) if self.rank == 0 else None

        # this rank's product alone (no collective): the roofline numerator.  On one GPU it is the timed region itself.
        if self.world == 1:
            kernel_ms = ms_per_step
        else:
            reps = max(3, min(steps, 5))
            torch.cuda.synchronize()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record()
            for i in range(reps):
                wl.call_local(cb, sets[i % len(sets)], self.rank, self.world)
            k1.record()
            torch.cuda.synchronize()
            kernel_ms = k0.elapsed_time(k1) / reps
            self.timed_s += kernel_ms * reps * 1e-3
        local_flops = wl.local_flops(self.rank, self.world)
        achieved = local_flops / (kernel_ms * 1e-3) / 1e12 if local_flops > 0 else 0.0
        per_rank = self.gather({"kernel_ms": round(kernel_ms, 4), "tflops": round(achieved, 3)})

        ratio = self.max_over_ranks(wl.parity(cb, sets[0], self.rank, self.world, self.comm))
        rec = {"metric": wl.metric, "value": value, "unit": "TFLOP/s", "ms_per_step": ms_per_step, "steps": steps, "warmup": warmup,
               "scaling": wl.scaling, "gpu_launches": int(launches), "kernel": kernel, "clocks": clocks,
               "per_rank": per_rank, "parity_error_over_bound": ratio, "local_ms": kernel_ms, "achieved": achieved,
               "nl": wl.local_n(self.rank, self.world)}
        del sets
        torch.cuda.empty_cache()
        return rec


def roofline(cb, wl, rec, peak_cache, gemm_path=0):
    if wl.pipe not in peak_cache:
        peak_cache[wl.pipe] = cb.probe_peak(wl.pipe, 0.3)
    peak = peak_cache[wl.pipe]
    hbm_peak = None
    try:
        hbm_peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
    except Exception:
        pass
    min_bytes = wl.min_bytes(rec["nl"])
    out = {"bound": "tensor" if wl.pipe == "fp64" else "fma", "achieved": rec["achieved"], "peak": peak, "unit": "TFLOP/s",
           "frac": rec["achieved"] / peak if peak > 0 else None, "traffic": NCU_TRAFFIC_BYTES.get(wl.name),
           "peak_source": f"in-run {wl.pipe} issue-rate probe of this library (MEASURED_PEAKS.json has no {wl.pipe} figure); of measured",
           "nominal_peak": NOMINAL[wl.pipe], "frac_of_nominal": rec["achieved"] / NOMINAL[wl.pipe],
           "kernel_ms": rec["local_ms"], "algorithmic_bytes": int(min_bytes),
           "achieved_hbm_gbs": min_bytes / (rec["local_ms"] * 1e-3) / 1e9, "hbm_peak_gbs": hbm_peak}
    if gemm_path == 4 and wl.prec == "s":
        # Optional 3xTF32 variant: three TF32 tensor-core MMAs per product.  TF32 runs at half the BF16
        # rate, so the ceiling is the measured BF16 burst figure / 2 / 3.
        try:
            bf16 = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
            src = "MEASURED_PEAKS.json bf16_tflops / 2 (TF32 rate) / 3 (MMAs per product); of measured"
        except Exception:
            bf16, src = 1590.0, "fallback 1.59 PFLOP/s bf16 / 2 / 3; of fallback"
        out.update(bound="tensor", peak=bf16 / 6.0, frac=rec["achieved"] / (bf16 / 6.0), peak_source=src, fp32_ffma_peak=peak,
                   frac_of_fp32_ffma_peak=rec["achieved"] / peak if peak > 0 else None, traffic=NCU_TRAFFIC_BYTES_3XTF32.get(wl.name))
    return out


def run_e2e(run, wl, steps):
    """The same metric through the public call with HOST buffers: every step copies the inputs up from pinned host
    memory and the result back.  One GPU: the library's host-matrix entry point (copies and products pipelined inside
    the call).  Several GPUs: rank 0 uploads A, every rank uploads its own blocks of B (and C when beta != 0), the
    sharded call runs, every rank downloads its block of the result."""
    cb, torch = run.cb, run.torch
    host = wl.alloc(run.rank, run.world, run.device, host=True)
    single = run.world == 1
    dev_bufs = None if single else [torch.empty_like(h, device=run.device) for h in host]
    out_host = None if single else torch.empty_like(host[-1]).pin_memory()
    nbytes = [h.numel() * h.element_size() for h in host]
    # what has to travel up: A from rank 0 only (the others receive it over NVLink), B, and C only when it is read
    skip_out = wl.kind == "gemm" and wl.beta == 0
    up = [i for i in range(len(host)) if not (i == 0 and run.rank != 0) and not (i == len(host) - 1 and skip_out)]
    h2d, d2h = sum(nbytes[i] for i in up), nbytes[-1]

    def step(_):
        if single:
            return wl.call_host(cb, host)
        for i in up:
            dev_bufs[i].copy_(host[i], non_blocking=True)
        s = wl.call(cb, dev_bufs, run.rank, run.world, run.comm)
        out_host.copy_(dev_bufs[-1], non_blocking=True)
        return s

    ms, _, _ = run.timed(step, steps, 2)
    tot = run.gather((int(h2d), int(d2h)))
    return {"value": wl.flops(run.world) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": int(sum(t[0] for t in tot)), "d2h_bytes_per_step": int(sum(t[1] for t in tot)), "steps": steps,
            "api": ("clblasB200%s%sHost (pipelined copies and products)" % (wl.prec.upper(), "trsm" if wl.kind == "trsm" else "gemm"))
                   if single else "pinned copies + sharded device entry point on one stream per rank"}


def main():
    names = list(workloads().keys())
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="sgemm32768", choices=names + list(ALIASES))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="headline workload only")
    ap.add_argument("--gemm-path", type=int, default=0, choices=[0, 1, 4],
                    help="clblasB200SetGemmPath: 0 automatic, 1 alignment-free kernels, 4 SGEMM 3xTF32 on tcgen05")
    args = ap.parse_args()
    args.workload = ALIASES.get(args.workload, args.workload)
    wl = workloads()[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, wl, world)
        return
    args.warmup = max(args.warmup, 3)

    import clblas_b200 as cb          # raises ImportError when the CUDA library is not built
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        from clblas_b200 import partition
        comm = partition.get_comm()
    cb.check(cb.clblasSetup(), "clblasSetup")
    cb.set_gemm_path(args.gemm_path)
    sampler = ClockSampler(local_rank).start()
    time.sleep(0.25)
    run = Runner(args, cb, torch, dist, rank, world, local_rank, device, comm, sampler)
    peaks = {}

    # ---- headline ---------------------------------------------------------------------------------------
    rec = run.measure(wl, args.steps, args.warmup)
    line = dict(base_line(args, wl, world), value=rec["value"], ms_per_step=rec["ms_per_step"], clocks=rec["clocks"],
                gpu_launches=rec["gpu_launches"], kernel=rec["kernel"],
                pct_of_nominal_peak=100.0 * rec["value"] / (NOMINAL[wl.pipe] * world),
                roofline=roofline(cb, wl, rec, peaks, args.gemm_path), per_rank=rec["per_rank"])
    parity = {wl.name: rec["parity_error_over_bound"]}
    clocks_per_rank = run.gather(sampler.summary())
    if args.gemm_path == 4 and wl.prec == "s":
        line["metric"] = "SGEMM (3xTF32 on tcgen05) TFLOP/s"
        line["config"]["gemm_path"] = "3xTF32 tcgen05 (opt-in)"

    # ---- end to end ---------------------------------------------------------------------------------------
    line["e2e"] = None if args.no_e2e else run_e2e(run, wl, max(3, min(args.steps, 5)))
    torch.cuda.empty_cache()

    # ---- the other workloads, briefly ---------------------------------------------------------------------
    if not args.no_also and args.gemm_path == 0:
        also = {}
        plan = [("dgemm8192", 10), ("sgemm8192", 10), ("dtrsm8192", 5)]
        if world == 1:
            plan += [("sgemm1024", 200), ("sgemm_ragged", 20)]
        for name, steps in plan:
            if name == wl.name:
                continue
            w = workloads()[name]
            r = run.measure(w, steps, 3)
            rl = roofline(cb, w, r, peaks)
            also[name] = {"metric": r["metric"], "value": r["value"], "unit": "TFLOP/s", "ms_per_step": r["ms_per_step"], "steps": steps,
                          "warmup": 3, "scaling": r["scaling"], "config": w.config(world), "kernel": r["kernel"],
                          "gpu_launches": r["gpu_launches"],
                          "roofline": {"frac": rl["frac"], "frac_of_nominal": rl["frac_of_nominal"], "achieved": rl["achieved"],
                                       "peak": rl["peak"], "kernel_ms": rl["kernel_ms"], "traffic": rl["traffic"]},
                          "per_rank": r["per_rank"], "clocks": r["clocks"]}
            parity[name] = r["parity_error_over_bound"]
        line["also"] = also
    line["parity"] = parity
    line["parity_bound"] = "error / (4*K*u) for GEMM on |alpha||A||B|+|beta||C|, backward error / (4*M*u) for TRSM; sampled, worst over ranks; must be <= 1"
    line["timed_region_s_total"] = run.timed_s
    line["clocks_per_rank"] = clocks_per_rank
    line["device_fault_flag"] = cb.device_fault()
    sampler.stop()

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, cores, kind, text = cpu_reference_sample(wl)
        line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": text}
        line["cpu_blas"] = cpu_blas_sample(wl)
    bad = [k for k, v in parity.items() if not (v <= 1.0)]
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        from clblas_b200 import partition
        partition.release_comms()
        dist.destroy_process_group()
    if bad or line["device_fault_flag"]:
        print(f"bench.py: parity check failed for {bad}, device fault flag {line['device_fault_flag']}", file=sys.stderr)
        sys.exit(1)


if __name__ == "__main__":
    main()
