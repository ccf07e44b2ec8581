"""Single-box partitioner: one process per GPU, column-major problems sharded over the ranks.

The reference's only multi-device mechanism is "several command queues per call": its legacy
solver gives every queue one piece of the problem, split along N in pieces aligned to 128
(stripeDivision, src/library/blas/generic/solution_seq_make.c:764-866), and relies on all queues
sharing the OpenCL buffers.  GPUs of one box do not share buffers, so here

* GEMM: rank r owns the column block [b_r, b_{r+1}) of op(B) and of C (boundaries from
  clblasB200PlanShards); A lives on the root and is broadcast over NCCL in panels -- column
  blocks of A as stored, which are contiguous in memory.  For transA = N a panel is a K-slab and
  the panel products accumulate into C (beta only on the first panel, 1 afterwards -- the
  reference's own split-K accumulation, src/library/blas/specialCases/GemmSpecialCases.cpp:127-191);
  for transA = T a panel is a block of C's rows.  All broadcasts are issued up front on NCCL's
  stream; the GEMM on panel p is ordered after broadcast p only, so panel p+1 travels over NVLink
  while panel p is multiplied.
* TRSM (side = Left): rank r owns right-hand-side columns [b_r, b_{r+1}); A is broadcast once
  and every rank solves its block independently (no further exchange).

The GEMM / TRSM calls go through the C ABI (clblas_b200.clblasSgemm, ...).  `gemm_fn` / `trsm_fn`
exist so that the rank logic (panel plan, ordering, accumulation) can be exercised with CPU
tensors over gloo in the tests; the package itself has no CPU implementation to put there.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

import clblas_b200 as cb


def plan_columns(total: int, parts: int, align: int = 128) -> List[int]:
    return cb.plan_shards(total, parts, align)


def panel_plan(ncols: int, panels: int, align: int = 128) -> List[Tuple[int, int]]:
    """Column ranges [c0, c1) of the stored A, at most `panels` of them, aligned to `align`."""
    b = cb.plan_shards(ncols, max(1, panels), align)
    return [(b[i], b[i + 1]) for i in range(len(b) - 1) if b[i + 1] > b[i]]


def _default_gemm(prec: str) -> Callable:
    return cb.clblasSgemm if prec == "s" else cb.clblasDgemm


def _default_trsm(prec: str) -> Callable:
    return cb.clblasStrsm if prec == "s" else cb.clblasDtrsm


def gemm_column_sharded(prec: str, transA: int, transB: int, M: int, n_local: int, K: int, alpha: float,
                        A: torch.Tensor, lda: int, B_local: torch.Tensor, ldb: int, beta: float,
                        C_local: torch.Tensor, ldc: int, *, root: int = 0, panels: Optional[int] = None,
                        group: Optional[dist.ProcessGroup] = None, gemm_fn: Optional[Callable] = None) -> int:
    """Column-major C_local <- alpha*op(A)*op(B)_local + beta*C_local on every rank.

    A is a flat tensor holding the stored A (column-major, leading dimension lda) on the root and a
    receive buffer of the same size elsewhere; B_local / C_local hold this rank's column block
    (n_local columns) as flat column-major buffers.  Returns the first non-success clblasStatus.
    """
    gemm = gemm_fn or _default_gemm(prec)
    ta = transA != cb.clblasNoTrans
    tb = transB != cb.clblasNoTrans
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    a_cols = M if ta else K                     # columns of A as stored
    if panels is None:
        # K-slabs keep every tile of C in each launch, so many thin slabs cost nothing; row blocks of C
        # shrink the grid of each launch, so they stay large enough for several full waves of CTAs.
        panels = 8 if not ta else max(1, min(4, (M * max(n_local, 1)) // (128 * 128 * 148 * 6)))
    plan = panel_plan(a_cols, panels if world > 1 else 1)

    works = []
    if world > 1:
        for (c0, c1) in plan:
            end = min(c1 * lda, A.numel())
            works.append(dist.broadcast(A[c0 * lda:end], src=root, group=group, async_op=True))

    status = cb.clblasSuccess
    for idx, (c0, c1) in enumerate(plan):
        if works:
            works[idx].wait()                   # orders the compute stream after this panel's broadcast
        w = c1 - c0
        if n_local == 0:
            continue
        if not ta:
            # K-slab: C += alpha * A[:, c0:c1] * op(B)[c0:c1, :]
            offB = c0 * ldb if tb else c0
            st = gemm(cb.clblasColumnMajor, transA, transB, M, n_local, w, alpha, A, c0 * lda, lda,
                      B_local, offB, ldb, beta if idx == 0 else 1.0, C_local, 0, ldc)
        else:
            # row block of C: C[c0:c1, :] = alpha * A[:, c0:c1]^T * op(B) + beta * C[c0:c1, :]
            st = gemm(cb.clblasColumnMajor, transA, transB, w, n_local, K, alpha, A, c0 * lda, lda,
                      B_local, 0, ldb, beta, C_local, c0, ldc)
        if st != cb.clblasSuccess and status == cb.clblasSuccess:
            status = st
    return status


def trsm_rhs_sharded(prec: str, uplo: int, transA: int, diag: int, M: int, n_local: int, alpha: float,
                     A: torch.Tensor, lda: int, B_local: torch.Tensor, ldb: int, *, root: int = 0,
                     panels: Optional[int] = None, group: Optional[dist.ProcessGroup] = None,
                     trsm_fn: Optional[Callable] = None, gemm_fn: Optional[Callable] = None) -> int:
    """Column-major, side = Left: op(A) X_local = alpha B_local on every rank, B_local overwritten.

    panels > 1 with transA = N: A is broadcast in column panels in the order the substitution needs
    them (first to last for a lower triangle, last to first for an upper one), all broadcasts queued up
    front on NCCL's stream.  Step p waits for panel p only, solves its diagonal block and subtracts the
    panel times that solution from the rows still to be solved, so panel p+1 crosses NVLink meanwhile.
    Otherwise (the default, and always for a transposed A, whose panels would be strided row blocks of
    the stored matrix) A is broadcast in one piece and each rank makes one TRSM call on its columns.
    """
    trsm = trsm_fn or _default_trsm(prec)
    gemm = gemm_fn or _default_gemm(prec)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    lower = uplo == cb.clblasLower
    if panels is None:
        # Measured on 2 and 8 B200s (DTRSM 8192 x 16384): the one-piece broadcast of A costs a few per cent of
        # the solve over NVSwitch, while eight panels cost 10-15 % (eight diagonal-block inversions and
        # rank-1024 updates instead of the recursion's larger ones), so the pipeline is opt-in.
        panels = 1
    plan = panel_plan(M, panels) if transA == cb.clblasNoTrans else [(0, M)]
    if len(plan) == 1:
        if world > 1:
            dist.broadcast(A, src=root, group=group)
        if n_local == 0:
            return cb.clblasSuccess
        return trsm(cb.clblasColumnMajor, cb.clblasLeft, uplo, transA, diag, M, n_local, alpha, A, 0, lda, B_local, 0, ldb)

    order = plan if lower else plan[::-1]
    works = []
    if world > 1:
        for (c0, c1) in order:
            end = min(c1 * lda, A.numel())
            works.append(dist.broadcast(A[c0 * lda:end], src=root, group=group, async_op=True))
    status = cb.clblasSuccess
    for idx, (c0, c1) in enumerate(order):
        if works:
            works[idx].wait()                   # orders the compute stream after this panel's broadcast
        if n_local == 0:
            continue
        w = c1 - c0
        a_eff = alpha if idx == 0 else 1.0      # every row of B is scaled by alpha exactly once, at step 0
        st = trsm(cb.clblasColumnMajor, cb.clblasLeft, uplo, transA, diag, w, n_local, a_eff, A, c0 + c0 * lda, lda,
                  B_local, c0, ldb)
        if st == cb.clblasSuccess:
            # rows still to be solved: B_rest <- a_eff*B_rest - A[rest, c0:c1] * X_p
            r0, r1 = (c1, M) if lower else (0, c0)
            if r1 > r0:
                st = gemm(cb.clblasColumnMajor, cb.clblasNoTrans, cb.clblasNoTrans, r1 - r0, n_local, w, -1.0,
                          A, r0 + c0 * lda, lda, B_local, c0, ldb, a_eff, B_local, r0, ldb)
        if st != cb.clblasSuccess and status == cb.clblasSuccess:
            status = st
    return status
