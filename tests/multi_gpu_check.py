"""Run under torchrun on N >= 2 GPUs (tests/test_multi_gpu.py launches it): the partitioner's GEMM and TRSM
paths over NCCL against float64 numpy results computed on every rank from the same seeded inputs."""
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
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    cb.check(cb.clblasSetup(), "clblasSetup")
    g = np.random.Generator(np.random.Philox(key=[4242, 0]))
    ok = True

    # GEMM, column blocks of C, integer inputs: exact
    M, N, K = 1024, 2048 + 128, 4096
    A = g.integers(-4, 5, (M, K)).astype(np.float64)
    B = g.integers(-4, 5, (K, N)).astype(np.float64)
    C = g.integers(-4, 5, (M, N)).astype(np.float64)
    b = partition.plan_columns(N, world)
    j0, j1 = b[rank], b[rank + 1]
    dA = torch.from_numpy(A.ravel(order="F").copy() if rank == 0 else np.zeros(M * K)).cuda()
    dB = torch.from_numpy(np.asfortranarray(B[:, j0:j1]).ravel(order="F").copy()).cuda()
    dC = torch.from_numpy(np.asfortranarray(C[:, j0:j1]).ravel(order="F").copy()).cuda()
    st = partition.gemm_column_sharded("d", cb.clblasNoTrans, cb.clblasNoTrans, M, j1 - j0, K, 2.0, dA, M, dB, K, -1.0, dC, M)
    torch.cuda.synchronize()
    got = dC.cpu().numpy().reshape(j1 - j0, M).T
    ok &= st == cb.clblasSuccess and np.array_equal(got, 2.0 * A @ B[:, j0:j1] - C[:, j0:j1])

    # TRSM, right-hand-side columns per rank, pipelined column panels of A: both triangles, alpha != 1
    n, nrhs = 4096 + 256, 1024 + 128
    b = partition.plan_columns(nrhs, world)
    j0, j1 = b[rank], b[rank + 1]
    for uplo in (cb.clblasLower, cb.clblasUpper):
        T = np.tril(g.uniform(-1, 1, (n, n)) / n) + np.diag(g.uniform(1, 2, n))
        T = T if uplo == cb.clblasLower else T.T.copy()
        stored = T.copy()
        stored[np.triu_indices(n, 1) if uplo == cb.clblasLower else np.tril_indices(n, -1)] = np.nan   # must not be read
        R = g.standard_normal((n, nrhs))
        dT = torch.from_numpy(stored.ravel(order="F").copy() if rank == 0 else np.zeros(n * n)).cuda()
        dR = torch.from_numpy(np.asfortranarray(R[:, j0:j1]).ravel(order="F").copy()).cuda()
        panels = 4 if uplo == cb.clblasLower else 1          # the pipelined column panels and the one-piece broadcast
        st = partition.trsm_rhs_sharded("d", uplo, cb.clblasNoTrans, cb.clblasNonUnit, n, j1 - j0, -2.0, dT, n, dR, n, panels=panels)
        torch.cuda.synchronize()
        X = dR.cpu().numpy().reshape(j1 - j0, n).T
        res = np.abs(-2.0 * R[:, j0:j1] - T @ X)
        den = np.abs(T) @ np.abs(X) + 2.0 * np.abs(R[:, j0:j1])
        ratio = float(np.max(res / den)) / (4 * n * 2.0 ** -53) if X.size else 0.0
        ok &= st == cb.clblasSuccess and np.all(np.isfinite(X)) and ratio <= 1.0
        if rank == 0:
            print(f"trsm uplo={uplo}: backward error / bound = {ratio:.3f}", flush=True)

    ok &= cb.device_fault() == 0
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("MULTI_GPU_CHECK", "OK" if flag.item() == 1 else "FAILED", flush=True)
    dist.destroy_process_group()
    return 0 if flag.item() == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
