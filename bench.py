#!/usr/bin/env python
"""Benchmark of the level-3 hot path on B200, in the protocol of the reference's client
(src/client/client.cpp:497, :574-592: one untimed warm-up, then back-to-back enqueued calls timed
as a block; GFLOP/s = 2*M*N*K / t, src/client/clfunc_xgemm.hpp:95-98; TRSM M*(M+1)*N / t,
src/client/clfunc_xtrsm.hpp:70-80) with CUDA events in place of gettimeofday.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg1|cfg2|cfg3|cfg4|cfg5]
    python bench.py --impl reference ...     # the reference's own CPU code on the host cores

One step = one call of the workload through the clBLAS-shaped C ABI.  The default workload is
BASELINE config 2 (DGEMM column-major T/N, M=N=K=8192, normal(0,1), alpha=beta=1).  With N > 1
ranks (torchrun, one process per GPU) C and op(B) are split in column blocks, A is broadcast from
rank 0 over NCCL inside every step; cfg2 keeps 8192 columns per rank (weak scaling), cfg4/cfg5
split their fixed problem (strong scaling).  Rank 0 prints one JSON line.
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

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum), captured
# with ncu at the workload's full size (these two metrics take one pass; profiles/dram_traffic_full_size.md).
# None where no capture of that workload exists (cfg4 is 127 launches of different shapes; cfg5 runs 1.2 s).
NCU_TRAFFIC_BYTES = {
    "cfg1": int(12.63e6),                          # sgemm_ffma_tma N/N 1024^3 (operands L2 resident, C not written back yet)
    "cfg2": int(6.107e9 + 509.2e6 + 620.1e6 + 12.4e6),   # dgemm_mma_tma T/N 8192^3: main kernel (3996 tiles) + stream-K tail (100 tiles)
    "cfg3": int(94.89e6 + 18.84e6),                # sgemm_ffma_tma on the repacked operands of config 3
    "cfg4": None,
    "cfg5": None,
    "sgemm8192": int(3.257e9 + 263.6e6),           # sgemm_nt_16x8 N/T 8192^3
}
NCU_TRAFFIC_BYTES_3XTF32 = {"sgemm8192": int(2.70e9 + 256.35e6)}


# ------------------------------------------------------------------------------------------------
# workloads (column-major after normalisation; sizes are BASELINE.json's)
# ------------------------------------------------------------------------------------------------

class Workload:
    name = ""
    prec = "d"
    scaling = "weak"
    pipe = "fp64"

    def flops(self, world):            # whole-job flops per step
        raise NotImplementedError

    def min_bytes(self):               # algorithmic bytes of one rank's launch
        raise NotImplementedError


def _dt(prec):
    import torch
    return torch.float32 if prec == "s" else torch.float64


class GemmWorkload(Workload):
    def __init__(self, name, prec, order, transA, transB, M, N, K, alpha, beta, lda, ldb, ldc, offs=(0, 0, 0),
                 dist_kind="uniform", scaling="weak", sets=1, desc=""):
        self.name, self.prec, self.order, self.transA, self.transB = name, prec, order, transA, transB
        self.M, self.N, self.K, self.alpha, self.beta = M, N, K, alpha, beta
        self.lda, self.ldb, self.ldc, self.offs = lda, ldb, ldc, offs
        self.dist_kind, self.scaling, self.sets, self.desc = dist_kind, scaling, sets, desc
        self.pipe = "fp32" if prec == "s" else "fp64"

    def local_n(self, rank, world):
        if world == 1:
            return self.N
        if self.scaling == "weak":
            return self.N
        import clblas_b200 as cb
        b = cb.plan_shards(self.N, world, 128)
        return b[rank + 1] - b[rank]

    def flops(self, world):
        n_total = self.N * world if self.scaling == "weak" else self.N
        return 2.0 * self.M * n_total * self.K

    def min_bytes(self, n_local=None):
        n = self.N if n_local is None else n_local
        e = 4 if self.prec == "s" else 8
        return (self.M * self.K + self.K * n + self.M * n * (2 if self.beta != 0 else 1)) * e

    def alloc(self, rank, world, device, host=False):
        """Flat buffers for A (stored), B_local, C_local.  Row-major workloads are allocated in
        their own layout; the library does the operand swap."""
        import torch
        import clblas_b200 as cb
        dt = _dt(self.prec)
        nl = self.local_n(rank, world)

        def stored(trans, rows, cols):
            tra = (self.order == cb.clblasColumnMajor and trans == cb.clblasNoTrans) or \
                  (self.order == cb.clblasRowMajor and trans != cb.clblasNoTrans)
            return (rows, cols) if tra else (cols, rows)

        def length(trans, rows, cols, ld, off):
            inner, outer = stored(trans, rows, cols)
            return off + (outer - 1) * ld + inner

        la = length(self.transA, self.M, self.K, self.lda, self.offs[0])
        lb = length(self.transB, self.K, nl, self.ldb, self.offs[1])
        lc = length(cb.clblasNoTrans, self.M, nl, self.ldc, self.offs[2])
        gen = torch.Generator(device=device)
        gen.manual_seed(12345 + rank)
        out = []
        for n in (la, lb, lc):
            if self.dist_kind == "normal":
                t = torch.empty(n, dtype=dt, device=device).normal_(generator=gen)
            else:
                t = torch.empty(n, dtype=dt, device=device).uniform_(-1.0, 1.0, generator=gen)
            out.append(t.cpu().pin_memory() if host else t)
        return out

    def call(self, cb, bufs, rank, world):
        A, B, C = bufs
        nl = self.local_n(rank, world)
        fn = cb.clblasSgemm if self.prec == "s" else cb.clblasDgemm
        if world == 1:
            return fn(self.order, self.transA, self.transB, self.M, nl, self.K, self.alpha, A, self.offs[0], self.lda,
                      B, self.offs[1], self.ldb, self.beta, C, self.offs[2], self.ldc)
        from clblas_b200 import partition
        assert self.order == cb.clblasColumnMajor and self.offs == (0, 0, 0)
        return partition.gemm_column_sharded(self.prec, self.transA, self.transB, self.M, nl, self.K, self.alpha,
                                             A, self.lda, B, self.ldb, self.beta, C, self.ldc, root=0)

    def call_host(self, cb, bufs):
        """This rank's whole problem on pinned host matrices through the host-matrix entry point."""
        A, B, C = bufs
        fn = cb.clblasB200SgemmHost if self.prec == "s" else cb.clblasB200DgemmHost
        return fn(self.order, self.transA, self.transB, self.M, self.N, self.K, self.alpha, A, self.offs[0], self.lda,
                  B, self.offs[1], self.ldb, self.beta, C, self.offs[2], self.ldc)

    def config(self, world):
        return {"workload": f"{self.name}: {self.desc}", "M": self.M, "N": self.N * (world if self.scaling == "weak" else 1),
                "K": self.K, "alpha": self.alpha, "beta": self.beta, "lda": self.lda, "ldb": self.ldb, "ldc": self.ldc,
                "offsets": list(self.offs)}


class TrsmWorkload(Workload):
    name, prec, scaling, pipe = "cfg4", "d", "strong", "fp64"

    def __init__(self):
        self.M, self.N, self.alpha = 8192, 16384, 1.0
        self.desc = "DTRSM column-major Left/Lower/NoTrans/NonUnit, A 8192x8192, B 8192x16384"
        self.sets = 1

    def local_n(self, rank, world):
        import clblas_b200 as cb
        b = cb.plan_shards(self.N, world, 128)
        return b[rank + 1] - b[rank]

    def flops(self, world):
        return float(self.M) * (self.M + 1) * self.N

    def min_bytes(self, n_local=None):
        n = self.N if n_local is None else n_local
        return (self.M * (self.M + 1) // 2 + 2 * self.M * n) * 8

    def alloc(self, rank, world, device, host=False):
        import torch
        M, nl = self.M, self.local_n(rank, world)
        gen = torch.Generator(device=device)
        gen.manual_seed(12345 + rank)
        A = torch.empty(M * M, dtype=torch.float64, device=device).uniform_(-1.0, 1.0, generator=gen) / M
        Av = A.view(M, M)                                   # Av[j, i] = A(i, j) column-major
        Av.diagonal().uniform_(1.0, 2.0, generator=gen)
        # strictly upper part of A (i < j): garbage that must never be read
        iu = torch.triu_indices(M, M, offset=1, device=device)
        Av[iu[1], iu[0]] = float("nan")
        B = torch.empty(M * nl, dtype=torch.float64, device=device).normal_(generator=gen)
        if host:
            return [A.cpu().pin_memory(), B.cpu().pin_memory()]
        return [A, B]

    def call(self, cb, bufs, rank, world):
        A, B = bufs
        nl = self.local_n(rank, world)
        if world == 1:
            return cb.clblasDtrsm(cb.clblasColumnMajor, cb.clblasLeft, cb.clblasLower, cb.clblasNoTrans, cb.clblasNonUnit,
                                  self.M, nl, self.alpha, A, 0, self.M, B, 0, self.M)
        from clblas_b200 import partition
        return partition.trsm_rhs_sharded("d", cb.clblasLower, cb.clblasNoTrans, cb.clblasNonUnit, self.M, nl, self.alpha,
                                          A, self.M, B, self.M, root=0)

    def call_host(self, cb, bufs):
        A, B = bufs
        return cb.clblasB200DtrsmHost(cb.clblasColumnMajor, cb.clblasLeft, cb.clblasLower, cb.clblasNoTrans, cb.clblasNonUnit,
                                      self.M, self.N, self.alpha, A, 0, self.M, B, 0, self.M)

    def config(self, world):
        return {"workload": f"{self.name}: {self.desc}", "M": self.M, "N": self.N, "alpha": self.alpha,
                "lda": self.M, "ldb": self.M}


def workloads():
    import clblas_b200 as cb
    CM, RM, N_, T_ = cb.clblasColumnMajor, cb.clblasRowMajor, cb.clblasNoTrans, cb.clblasTrans
    return {
        "cfg1": GemmWorkload("cfg1", "s", CM, N_, N_, 1024, 1024, 1024, 1.5, 0.5, 1024, 1024, 1024, dist_kind="uniform",
                             sets=16, desc="SGEMM column-major N/N 1024^3, U[-1,1], alpha=1.5 beta=0.5"),
        "cfg2": GemmWorkload("cfg2", "d", CM, T_, N_, 8192, 8192, 8192, 1.0, 1.0, 8192, 8192, 8192, dist_kind="normal",
                             scaling="weak", desc="DGEMM column-major T/N 8192^3, normal(0,1), alpha=beta=1, tight ld"),
        "cfg3": GemmWorkload("cfg3", "s", RM, T_, N_, 4099, 3001, 1537, -2.0, 0.25, 4099 + 16, 3001 + 32, 3001 + 8,
                             offs=(7, 13, 5), sets=2,
                             desc="SGEMM row-major T/N M=4099 N=3001 K=1537, padded ld, offsets 7/13/5, alpha=-2 beta=0.25"),
        "cfg4": TrsmWorkload(),
        # the shape the reference publishes its own curves on (column-major N/T, m=n=k=ld, alpha=beta=1,
        # doc/performance/clBLAS_2.6.0/S9150/README.txt:21-35) at the size the FP32 target is stated for
        "sgemm8192": GemmWorkload("sgemm8192", "s", CM, N_, T_, 8192, 8192, 8192, 1.0, 1.0, 8192, 8192, 8192,
                                  desc="SGEMM column-major N/T 8192^3, U[-1,1], alpha=beta=1"),
        "cfg5": GemmWorkload("cfg5", "s", CM, N_, T_, 32768, 32768, 32768, 1.0, 0.0, 32768, 32768, 32768,
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

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smmax, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
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
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [c for c, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": max(smmax), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm)}


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

    if isinstance(wl, TrsmWorkload):
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
    n = 4096 if not isinstance(wl, TrsmWorkload) else 4096
    if isinstance(wl, TrsmWorkload):
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


def run_reference_arm(args, wl, world):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    for _ in range(max(1, args.warmup and 1)):
        cpu_reference_sample(wl, seconds_target=2.0)
    text = kind = None
    cores = 0
    per_step = max(2.0, min(20.0, 120.0 / max(args.steps, 1)))
    t_all = time.perf_counter()
    for _ in range(args.steps):
        v, cores, kind, text = cpu_reference_sample(wl, seconds_target=per_step)
        vals.append(v)
    wall = time.perf_counter() - t_all
    value = float(np.mean(vals))
    line = {"impl": "reference", "metric": metric_name(wl), "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3, "higher_is_better": True,
            "scaling": wl.scaling, "vs_baseline": None, "dtype": "f32" if wl.prec == "s" else "f64", "data": "synthetic",
            "config": wl.config(1), "gpu_launches": 0,
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": text},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def metric_name(wl):
    r = {"cfg1": "SGEMM", "cfg2": "DGEMM", "cfg3": "SGEMM", "cfg4": "DTRSM", "cfg5": "SGEMM", "sgemm8192": "SGEMM"}[wl.name]
    return f"{r} TFLOP/s"


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "sgemm8192"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--gemm-path", type=int, default=0, choices=[0, 1, 4],
                    help="clblasB200SetGemmPath: 0 automatic, 1 alignment-free kernels, 4 SGEMM 3xTF32 on tcgen05")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    import clblas_b200 as cb          # raises ImportError when the CUDA library is not built
    wl = workloads()[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, wl, world)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cb.check(cb.clblasSetup(), "clblasSetup")
    cb.set_gemm_path(args.gemm_path)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident run ---------------------------------------------------------------
    sets = [wl.alloc(rank, world, device) for _ in range(getattr(wl, "sets", 1))]
    set_bytes = sum(t.numel() * t.element_size() for t in sets[0])
    for i in range(args.warmup):
        cb.check(wl.call(cb, sets[i % len(sets)], rank, world), "warm-up call")
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = cb.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        st = wl.call(cb, sets[i % len(sets)], rank, world)
    e1.record()
    barrier()
    cb.check(st, "timed call")
    launches = cb.launch_count() - launches0
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    value = wl.flops(world) / (ms_per_step * 1e-3) / 1e12

    # ---- dominant kernel alone (local problem, no collective): roofline numerator ----------------
    nl = wl.local_n(rank, world)
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(3, min(args.steps, 10))
    single = workloads()[args.workload]
    single_world = 1
    if world > 1 and wl.scaling == "strong":
        single = None      # local shard differs from the 1-GPU problem: timed through the same sharded call
    torch.cuda.synchronize()
    k0.record()
    for i in range(reps):
        if single is not None:
            single.call(cb, sets[i % len(sets)], 0, 1)
        else:
            wl.call(cb, sets[i % len(sets)], rank, world)
    k1.record()
    torch.cuda.synchronize()
    kernel_ms = k0.elapsed_time(k1) / reps
    local_flops = (single.flops(1) if single is not None else wl.flops(world) / world)
    achieved = local_flops / (kernel_ms * 1e-3) / 1e12
    peak = cb.probe_peak(wl.pipe, 0.3)
    fault = cb.device_fault()

    # ---- end to end: pinned host buffers -> device -> call -> host, every step -------------------
    e2e = None
    if not args.no_e2e:
        host = wl.alloc(rank, world, device, host=True)
        dev_bufs = [torch.empty_like(h, device=device) for h in host]
        out_host = torch.empty_like(host[-1]).pin_memory()
        h2d = sum(h.numel() * h.element_size() for h in host)
        d2h = out_host.numel() * out_host.element_size()

        host_call = getattr(wl, "call_host", None) if (world == 1 or wl.scaling == "weak") else None

        def e2e_step():
            if host_call is not None:
                # the library's host-matrix entry point: uploads, products and downloads pipelined inside the call,
                # result written back into the pinned host C
                return host_call(cb, host)
            for h, d in zip(host, dev_bufs):
                d.copy_(h, non_blocking=True)
            s = wl.call(cb, dev_bufs, rank, world)
            out_host.copy_(dev_bufs[-1], non_blocking=True)
            return s

        for _ in range(2):
            e2e_step()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(3, min(args.steps, 5))
        t0.record()
        for _ in range(n_e2e):
            e2e_step()
        t1.record()
        barrier()
        ems = t0.elapsed_time(t1)
        if world > 1:
            t = torch.tensor([ems], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = float(t.item())
        e2e = {"value": wl.flops(world) / (ems / n_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": n_e2e,
               "api": ("clblasB200%s%sHost (pipelined copies and products)" % (getattr(wl, "prec", "d").upper(), "trsm" if wl.name == "cfg4" else "gemm"))
                      if host_call is not None
                      else "pinned copies + device entry point on one stream"}
        del host, dev_bufs, out_host

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    hbm_peak = None
    try:
        hbm_peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
    except Exception:
        pass
    min_bytes = wl.min_bytes(nl)
    traffic = NCU_TRAFFIC_BYTES.get(wl.name)
    line = {
        "metric": metric_name(wl), "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": wl.scaling,
        "vs_baseline": None, "dtype": "f32" if wl.prec == "s" else "f64", "data": "synthetic",
        "config": dict(wl.config(world), l2="inputs larger than L2" if set_bytes * len(sets) > 130e6 else "rotating buffer sets larger than L2",
                       buffer_sets=len(sets), parallelism=f"column blocks of C over {world} GPU(s), A broadcast over NCCL" if world > 1 else "1 GPU"),
        "clocks": clocks, "gpu_launches": int(launches), "kernel": cb.last_gemm_kernel(),
        "pct_of_nominal_peak": 100.0 * value / (NOMINAL[wl.pipe] * world),
        "e2e": e2e,
        "roofline": {"bound": "tensor" if wl.pipe == "fp64" else "fma", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak if peak > 0 else None, "traffic": traffic,
                     "peak_source": f"in-run {wl.pipe} issue-rate probe of this library (MEASURED_PEAKS.json has no {wl.pipe} figure); of measured",
                     "nominal_peak": NOMINAL[wl.pipe], "frac_of_nominal": achieved / NOMINAL[wl.pipe],
                     "kernel_ms": kernel_ms, "algorithmic_bytes": int(min_bytes),
                     "achieved_hbm_gbs": min_bytes / (kernel_ms * 1e-3) / 1e9, "hbm_peak_gbs": hbm_peak},
        "device_fault_flag": fault,
    }
    if args.gemm_path == 4 and wl.prec == "s":
        # Optional 3xTF32 variant: three TF32 tensor-core MMAs per product.  TF32 runs at half the BF16
        # rate, so the ceiling is the measured BF16 burst figure / 2 / 3.
        try:
            bf16 = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
            src = "MEASURED_PEAKS.json bf16_tflops / 2 (TF32 rate) / 3 (MMAs per product); of measured"
        except Exception:
            bf16, src = 1590.0, "fallback 1.59 PFLOP/s bf16 / 2 / 3; of fallback"
        r = line["roofline"]
        r.update(bound="tensor", peak=bf16 / 6.0, frac=achieved / (bf16 / 6.0), peak_source=src,
                 fp32_ffma_peak=peak, frac_of_fp32_ffma_peak=achieved / peak if peak > 0 else None,
                 traffic=NCU_TRAFFIC_BYTES_3XTF32.get(wl.name))
        line["metric"] = "SGEMM (3xTF32 on tcgen05) TFLOP/s"
        line["config"]["gemm_path"] = "3xTF32 tcgen05 (opt-in)"
    if world == 1 and not args.no_cpu_baseline:
        v, cores, kind, text = cpu_reference_sample(wl)
        line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": text}
        line["cpu_blas"] = cpu_blas_sample(wl)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
