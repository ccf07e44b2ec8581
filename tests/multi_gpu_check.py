"""Run under torchrun on N >= 2 GPUs (tests/test_multi_gpu.py launches it): the sharded C entry points
(clblasB200DgemmSharded / SgemmSharded / DtrsmSharded: NCCL broadcast in panels on a second stream, products and
solve behind events) against float64 numpy results computed on every rank from the same seeded inputs; then,
on rank 0 alone, clblasDgemm with two queues on two devices (stripes of N, peer copies)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import clblas_b200 as cb  # noqa: E402
from clblas_b200 import partition  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cb.check(cb.clblasSetup(), "clblasSetup")
    g = np.random.Generator(np.random.Philox(key=[4242, 0]))
    ok = True
    notes = []

    def flat(a):
        return np.asfortranarray(a).ravel(order="F").copy()

    # ---- GEMM, column blocks of C, integer inputs: exact.  All four transpositions, double and float; the
    # N/N double case twice in a row (the second call re-uses the communicator's events), an empty shard
    # (N = 100: only rank 0 owns columns) and K = 0 (C <- beta*C, nothing travels).
    shapes = [("d", 0, 0, 1024, 2048 + 128, 4096), ("d", 0, 0, 1024, 2048 + 128, 4096), ("d", 1, 0, 1536, 2176, 1024),
              ("s", 0, 1, 1152, 2176, 2048), ("s", 1, 1, 640, 1100, 512), ("d", 0, 1, 256, 100, 512), ("d", 0, 0, 256, 384, 0)]
    for prec, ta, tb, M, N, K in shapes:
        dt = np.float64 if prec == "d" else np.float32
        A = g.integers(-4, 5, (M, K)).astype(dt)
        B = g.integers(-4, 5, (K, N)).astype(dt)
        C = g.integers(-4, 5, (M, N)).astype(dt)
        b = partition.plan_columns(N, world)
        j0, j1 = b[rank], b[rank + 1]
        storedA = flat(A.T if ta else A)
        dA = torch.from_numpy(storedA if rank == 0 else np.zeros_like(storedA)).cuda() if K else torch.zeros(8, dtype=torch.from_numpy(storedA).dtype).cuda()
        Bl = B[:, j0:j1]
        dB = torch.from_numpy(flat(Bl.T if tb else Bl) if Bl.size else np.zeros(8, dt)).cuda()
        dC = torch.from_numpy(flat(C[:, j0:j1]) if j1 > j0 else np.zeros(8, dt)).cuda()
        lda = K if ta else M
        ldb = max(j1 - j0, 1) if tb else max(K, 1)
        st = partition.gemm_column_sharded(prec, ta, tb, M, j1 - j0, K, 2.0, dA, max(lda, 1), dB, ldb, -1.0, dC, M)
        torch.cuda.synchronize()
        good = st == cb.clblasSuccess
        if j1 > j0:
            got = dC.cpu().numpy().reshape(j1 - j0, M).T
            good &= bool(np.array_equal(got, 2.0 * A @ Bl - C[:, j0:j1]))
        if K:
            good &= bool(np.array_equal(dA.cpu().numpy(), storedA))          # every rank now holds A
        ok &= good
        notes.append(f"gemm {prec} ta={ta} tb={tb} {M}x{N}x{K}: {'ok' if good else 'FAILED'} ({cb.last_gemm_variant()})")

    # ---- TRSM, right-hand-side columns per rank, A broadcast in panels the solve waits for: every triangle /
    # transposition (ascending and descending panel order), unit diagonal once, alpha != 1, NaN outside the
    # triangle.  Order 4352 = 34 diagonal blocks, 3 panels (256, 1024, 3072 columns; mirrored when the substitution starts at the end).
    n, nrhs = 4096 + 256, 1024 + 128
    b = partition.plan_columns(nrhs, world)
    j0, j1 = b[rank], b[rank + 1]
    for uplo, trans, diag in ((cb.clblasLower, cb.clblasNoTrans, cb.clblasNonUnit), (cb.clblasUpper, cb.clblasNoTrans, cb.clblasNonUnit),
                              (cb.clblasLower, cb.clblasTrans, cb.clblasUnit), (cb.clblasUpper, cb.clblasTrans, cb.clblasNonUnit)):
        T = np.tril(g.uniform(-1, 1, (n, n)) / n, -1) + np.diag(g.uniform(1, 2, n))
        if diag == cb.clblasUnit:
            np.fill_diagonal(T, 1.0)
        T = T if uplo == cb.clblasLower else T.T.copy()
        stored = T.copy()
        stored[np.triu_indices(n, 1) if uplo == cb.clblasLower else np.tril_indices(n, -1)] = np.nan   # must not be read
        if diag == cb.clblasUnit:
            np.fill_diagonal(stored, np.nan)
        R = g.standard_normal((n, nrhs))
        dT = torch.from_numpy(flat(stored) if rank == 0 else np.zeros(n * n)).cuda()
        dR = torch.from_numpy(flat(R[:, j0:j1]) if j1 > j0 else np.zeros(8)).cuda()
        st = partition.trsm_rhs_sharded("d", uplo, trans, diag, n, j1 - j0, -2.0, dT, n, dR, n)
        torch.cuda.synchronize()
        ratio = 0.0
        good = st == cb.clblasSuccess
        if j1 > j0:
            X = dR.cpu().numpy().reshape(j1 - j0, n).T
            op = T.T if trans else T
            res = np.abs(-2.0 * R[:, j0:j1] - op @ X)
            den = np.abs(op) @ np.abs(X) + 2.0 * np.abs(R[:, j0:j1])
            ratio = float(np.max(res / den)) / (4 * n * 2.0 ** -53)
            good &= bool(np.all(np.isfinite(X))) and ratio <= 1.0
        ok &= good
        notes.append(f"trsm uplo={uplo} trans={trans} diag={diag}: backward error / bound = {ratio:.3f} {'ok' if good else 'FAILED'}")

    ok &= cb.device_fault() == 0
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()

    # ---- one process, two queues on two devices (rank 0 only; the other ranks are idle by now)
    if rank == 0 and torch.cuda.device_count() >= 2:
        M, N, K = 640, 1000, 384
        A = g.integers(-4, 5, (M, K)).astype(np.float64)
        B = g.integers(-4, 5, (K, N)).astype(np.float64)
        C = g.integers(-4, 5, (M, N)).astype(np.float64)
        dA, dB, dC = (torch.from_numpy(flat(x)).cuda() for x in (A, B, C))
        other = torch.device("cuda", 1 if local == 0 else 0)
        s0, s1 = torch.cuda.Stream(), torch.cuda.Stream(device=other)
        with torch.cuda.device(other):
            ev1 = torch.cuda.Event()
            ev1.record(s1)                  # gives the event its device; re-recorded by the call
        ev0 = torch.cuda.Event()
        ev0.record(s0)
        torch.cuda.synchronize()
        st = cb.clblasDgemm(cb.clblasColumnMajor, cb.clblasNoTrans, cb.clblasNoTrans, M, N, K, 3.0, dA, 0, M, dB, 0, K, 2.0, dC, 0, M,
                            queues=[s0, s1], events=[ev0, ev1])
        ev0.synchronize()
        ev1.synchronize()
        good = st == cb.clblasSuccess and bool(np.array_equal(dC.cpu().numpy().reshape(N, M).T, 3.0 * A @ B + 2.0 * C))
        notes.append(f"two queues on two devices: {'ok' if good else 'FAILED'}")
        if not good:
            flag.fill_(0)
    if rank == 0:
        for ln in notes:
            print(ln, flush=True)
        print("MULTI_GPU_CHECK", "OK" if flag.item() == 1 else "FAILED", flush=True)
    partition.release_comms()
    dist.destroy_process_group()
    return 0 if flag.item() == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
