"""The N > 1 host path on CPU: two gloo ranks run the partitioner's panel plan (clblasB200PanelPlan, the plan the
C entry points use), broadcast ordering, accumulation, an empty shard and K = 0 with CPU tensors.  The GEMM /
TRSM routine is injected here (the CPU oracle) only to make the rank logic observable without a GPU; on a GPU
box the same functions call clblasB200{S,D}gemmSharded / {S,D}trsmSharded."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from oracle import ColumnMajor, Left, Lower, NonUnit, NoTrans, Trans


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_gemm(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                 queues=None, wait=None, events=None):
    oracle.gemm(order, transA, transB, M, N, K, alpha, A.numpy(), offA, lda, B.numpy(), offB, ldb, beta, C.numpy(), offC, ldc)
    return 0


def _oracle_trsm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, queues=None, wait=None, events=None):
    oracle.trsm(order, side, uplo, transA, diag, M, N, alpha, A.numpy(), offA, lda, B.numpy(), offB, ldb)
    return 0


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from clblas_b200 import partition
        results = {}
        g = np.random.Generator(np.random.Philox(key=[777, 0]))
        for (M, N, K, ta, tb) in ((96, 300, 2100, NoTrans, Trans), (400, 300, 260, Trans, NoTrans), (96, 300, 1300, NoTrans, NoTrans),
                                  (300, 300, 70, Trans, Trans), (64, 100, 700, NoTrans, Trans), (64, 300, 0, NoTrans, NoTrans)):
            bounds = partition.plan_columns(N, world, 128)       # N = 100: rank 1 owns no column
            j0, j1 = bounds[rank], bounds[rank + 1]
            opA = g.integers(-8, 8, (M, K)).astype(np.float64)
            opB = g.integers(-8, 8, (K, N)).astype(np.float64)
            C0 = g.integers(-8, 8, (M, N)).astype(np.float64)
            lda = (M if ta == NoTrans else K) + 3
            A_full = oracle.pack(opA, ColumnMajor, ta, lda, 0, pad_value=0.0) if K else np.zeros(8)
            A = torch.from_numpy(A_full.copy() if rank == 0 else np.zeros_like(A_full))
            nl = j1 - j0
            ldb = (K if tb == NoTrans else max(nl, 1)) + 1
            B = torch.from_numpy(oracle.pack(opB[:, j0:j1], ColumnMajor, tb, ldb, 0, pad_value=0.0))
            C = torch.from_numpy(oracle.pack(C0[:, j0:j1], ColumnMajor, NoTrans, M + 2, 0, pad_value=0.0))
            st = partition.gemm_column_sharded("d", ta, tb, M, nl, K, 2.0, A, lda, B, ldb, 3.0, C, M + 2,
                                               root=0, gemm_fn=_oracle_gemm)
            got = oracle.view(C.numpy(), ColumnMajor, NoTrans, M, nl, M + 2, 0) if nl else np.zeros((M, 0))
            want = 2.0 * opA @ opB[:, j0:j1] + 3.0 * C0[:, j0:j1]
            results[f"gemm{ta}{tb}_{M}x{N}x{K}"] = (st, bool(np.array_equal(got, want)), bool(np.array_equal(A.numpy(), A_full)))

        n, nrhs = 64, 140
        bounds = partition.plan_columns(nrhs, world, 128)
        j0, j1 = bounds[rank], bounds[rank + 1]
        T = np.tril(g.uniform(-1, 1, (n, n)) / n, -1) + np.diag(g.uniform(1, 2, n))
        Bf = g.standard_normal((n, nrhs))
        A = torch.from_numpy(T.ravel(order="F").copy() if rank == 0 else np.zeros(n * n))
        Bl = torch.from_numpy(np.asfortranarray(Bf[:, j0:j1]).ravel(order="F").copy())
        st = partition.trsm_rhs_sharded("d", Lower, NoTrans, NonUnit, n, j1 - j0, 1.0, A, n, Bl, n, root=0, trsm_fn=_oracle_trsm)
        X = Bl.numpy().reshape(j1 - j0, n).T if j1 > j0 else np.zeros((n, 0))
        results["trsm"] = (st, bool(np.allclose(T @ X, Bf[:, j0:j1], atol=1e-10)), True)
        # several broadcast panels, both substitution directions (panels sent from the first or from the last column)
        from oracle import Upper
        for name, uplo in (("trsm_panels_lower", Lower), ("trsm_panels_upper", Upper)):
            n2 = 1300                  # three panels: 128, 512 and 660 columns
            T2 = np.tril(g.uniform(-1, 1, (n2, n2)) / n2) + np.diag(g.uniform(1, 2, n2))
            T2 = T2 if uplo == Lower else T2.T.copy()
            B2 = g.standard_normal((n2, nrhs))
            stored = T2.ravel(order="F").copy()
            A2 = torch.from_numpy(stored.copy() if rank == 0 else np.zeros(n2 * n2))
            Bl2 = torch.from_numpy(np.asfortranarray(B2[:, j0:j1]).ravel(order="F").copy())
            st = partition.trsm_rhs_sharded("d", uplo, NoTrans, NonUnit, n2, j1 - j0, -2.0, A2, n2, Bl2, n2, root=0,
                                            trsm_fn=_oracle_trsm)
            X2 = Bl2.numpy().reshape(j1 - j0, n2).T if j1 > j0 else np.zeros((n2, 0))
            results[name] = (st, bool(np.allclose(T2 @ X2, -2.0 * B2[:, j0:j1], atol=1e-9)), bool(np.array_equal(A2.numpy(), stored)))
        q.put((rank, results))
    finally:
        dist.destroy_process_group()


def test_two_rank_partition_over_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in out) == [0, 1]
    for rank, results in out:
        assert len(results) == 9
        for name, (st, ok, a_ok) in results.items():
            assert st == 0 and ok and a_ok, (rank, name, st, ok, a_ok)


def test_panel_plans_cover_all_columns_in_order():
    import clblas_b200 as cb
    from clblas_b200 import partition
    for ncols in (1, 100, 128, 1000, 4352, 8192, 32768):
        for min_cols in (128, 640):
            b = cb.panel_plan(ncols, min_cols, 12)
            assert b[0] == 0 and b[-1] == ncols and len(b) - 1 <= 12
            assert all(x < y for x, y in zip(b, b[1:])) and all(x % 128 == 0 for x in b[:-1])
            widths = [y - x for x, y in zip(b, b[1:])]
            assert widths[0] <= max(min_cols + 127, ncols // 32 + 128) or len(widths) == 1      # little is exposed
        for uplo in (cb.clblasLower, cb.clblasUpper):
            for trans in (cb.clblasNoTrans, cb.clblasTrans):
                plan = partition.trsm_panels(uplo, trans, ncols)
                cover = sorted(plan)
                assert cover[0][0] == 0 and cover[-1][1] == ncols and all(a[1] == b[0] for a, b in zip(cover, cover[1:]))
                assert all(c0 % 128 == 0 for c0, _ in plan)
                forward = (uplo == cb.clblasLower) != (trans != cb.clblasNoTrans)
                assert plan == (cover if forward else cover[::-1])       # first panel where the substitution starts
