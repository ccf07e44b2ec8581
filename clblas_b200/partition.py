"""Single-box partitioner, Python side: one process per GPU, column-major problems sharded over the ranks.

The work is done by the C ABI: ``clblasB200{S,D}gemmSharded`` / ``clblasB200{S,D}trsmSharded``
(csrc/sharded.cu) broadcast the shared operand over NCCL in column panels on a second stream and run
the panel products / the blocked solve behind cudaEvents.  This module adds what a torch.distributed
program needs around them:

* ``get_comm(group)``: the library communicator that matches a process group (created once per group;
  the group only carries the 128-byte id from rank 0 to the others);
* ``gemm_column_sharded`` / ``trsm_rhs_sharded``: the calls on torch tensors, column-major.

The reference's counterpart is its per-queue split of one call (stripes of N aligned to 128,
src/library/blas/generic/solution_seq_make.c:764-866; K-slab accumulation with beta -> 1,
src/library/blas/specialCases/GemmSpecialCases.cpp:127-191).

``gemm_fn`` / ``trsm_fn`` replace the C entry point by a per-panel routine and the NCCL broadcasts by
``torch.distributed`` ones, following the same panel plan (``clblasB200PanelPlan``) in the same order: that is
how the tests run the rank logic -- plan, ordering, accumulation, empty shards, K = 0 -- over gloo on CPU
tensors.  The package has no CPU implementation to put there; the tests inject their checker.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

import clblas_b200 as cb

_COMMS: Dict[object, int] = {}


def plan_columns(total: int, parts: int, align: int = 128) -> List[int]:
    return cb.plan_shards(total, parts, align)


def gemm_panels(prec: str, transA: int, M: int, n_local: int, K: int, sm_count: int = 148) -> List[Tuple[int, int]]:
    """Column ranges [c0, c1) of the stored A in the order they are broadcast: the plan of gemm_sharded_colmajor."""
    ta = transA != cb.clblasNoTrans
    cols = M if ta else K
    min_cols = 1024 if prec == "s" else 512
    if ta:
        min_cols = max(128, sm_count * 2 * 128 * 128 // max(n_local, 128))
    b = cb.panel_plan(cols, min_cols, 12)
    return [(b[i], b[i + 1]) for i in range(len(b) - 1)]


def trsm_panels(uplo: int, transA: int, n: int, right: bool = False) -> List[Tuple[int, int]]:
    """Column ranges of the stored triangular matrix in broadcast order: growing panels, first the small one where the
    substitution starts (the plan of trsm_sharded_colmajor)."""
    lower, trans = uplo == cb.clblasLower, transA != cb.clblasNoTrans
    ascending = ((lower != trans) != right)
    b = cb.panel_plan(n, 0 if ascending else 1, 10)
    plan = [(b[i], b[i + 1]) for i in range(len(b) - 1)]
    return plan if ascending else plan[::-1]


def get_comm(group: Optional[dist.ProcessGroup] = None) -> int:
    """The library communicator for a process group (collective on first use for that group)."""
    key = group if group is not None else "default"
    if key not in _COMMS:
        _COMMS[key] = cb.comm_from_process_group(group)
    return _COMMS[key]


def release_comms() -> None:
    for h in _COMMS.values():
        cb.comm_destroy(h)
    _COMMS.clear()


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def gemm_column_sharded(prec: str, transA: int, transB: int, M: int, n_local: int, K: int, alpha: float,
                        A: torch.Tensor, lda: int, B_local: torch.Tensor, ldb: int, beta: float,
                        C_local: torch.Tensor, ldc: int, *, root: int = 0,
                        group: Optional[dist.ProcessGroup] = None, gemm_fn: Optional[Callable] = None) -> int:
    """Column-major C_local <- alpha*op(A)*op(B)_local + beta*C_local on every rank.

    A is a flat tensor holding the stored A (leading dimension lda) on the root and a receive buffer of the
    same size elsewhere; B_local / C_local hold this rank's column block (n_local columns, possibly none).
    Returns the clblasStatus of the call.
    """
    if gemm_fn is None:
        fn = cb.clblasB200SgemmSharded if prec == "s" else cb.clblasB200DgemmSharded
        comm = get_comm(group) if _world(group) > 1 else None
        return fn(cb.clblasColumnMajor, transA, transB, M, n_local, K, alpha, A, 0, lda, B_local, 0, ldb, beta,
                  C_local, 0, ldc, comm, root)

    # ---- the same rank logic with an injected per-panel routine and torch.distributed broadcasts
    ta, tb = transA != cb.clblasNoTrans, transB != cb.clblasNoTrans
    a_rows, a_cols = (K, M) if ta else (M, K)
    if a_rows == 0 or a_cols == 0 or alpha == 0:
        # C <- beta*C; A is not referenced and nothing travels
        return gemm_fn(cb.clblasColumnMajor, transA, transB, M, n_local, K, alpha, A, 0, lda, B_local, 0, ldb, beta, C_local, 0, ldc) \
            if n_local else cb.clblasSuccess
    plan = gemm_panels(prec, transA, M, n_local, K)
    works = []
    if _world(group) > 1:
        for (c0, c1) in plan:
            end = (a_cols - 1) * lda + a_rows if c1 == a_cols else c1 * lda
            works.append(dist.broadcast(A[c0 * lda:end], src=root, group=group, async_op=True))
    status = cb.clblasSuccess
    for idx, (c0, c1) in enumerate(plan):
        if works:
            works[idx].wait()
        if n_local == 0:
            continue
        w = c1 - c0
        if not ta:      # K slab
            st = gemm_fn(cb.clblasColumnMajor, transA, transB, M, n_local, w, alpha, A, c0 * lda, lda,
                         B_local, c0 * ldb if tb else c0, ldb, beta if idx == 0 else 1.0, C_local, 0, ldc)
        else:           # rows [c0, c1) of C
            st = gemm_fn(cb.clblasColumnMajor, transA, transB, w, n_local, K, alpha, A, c0 * lda, lda,
                         B_local, 0, ldb, beta, C_local, c0, ldc)
        if st != cb.clblasSuccess and status == cb.clblasSuccess:
            status = st
    return status


def trsm_rhs_sharded(prec: str, uplo: int, transA: int, diag: int, M: int, n_local: int, alpha: float,
                     A: torch.Tensor, lda: int, B_local: torch.Tensor, ldb: int, *, root: int = 0,
                     group: Optional[dist.ProcessGroup] = None, trsm_fn: Optional[Callable] = None) -> int:
    """Column-major, side = Left: op(A) X_local = alpha B_local on every rank, B_local overwritten."""
    if trsm_fn is None:
        fn = cb.clblasB200StrsmSharded if prec == "s" else cb.clblasB200DtrsmSharded
        comm = get_comm(group) if _world(group) > 1 else None
        return fn(cb.clblasColumnMajor, cb.clblasLeft, uplo, transA, diag, M, n_local, alpha, A, 0, lda, B_local, 0, ldb,
                  comm, root)

    if M == 0:
        return cb.clblasSuccess
    if alpha != 0 and _world(group) > 1:
        works = []
        for (c0, c1) in trsm_panels(uplo, transA, M):
            end = (M - 1) * lda + M if c1 == M else c1 * lda
            works.append(dist.broadcast(A[c0 * lda:end], src=root, group=group, async_op=True))
        for w in works:       # on the GPU each step of the solve waits only for the panels it reads
            w.wait()
    if n_local == 0:
        return cb.clblasSuccess
    return trsm_fn(cb.clblasColumnMajor, cb.clblasLeft, uplo, transA, diag, M, n_local, alpha, A, 0, lda, B_local, 0, ldb)
