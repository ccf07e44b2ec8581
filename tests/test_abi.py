"""CPU-side checks of the drop-in boundary: the C-ABI library loads, exports every function that
include/clblas_b200.h declares, carries the reference's enum and status values, and rejects bad
arguments that can be detected before any CUDA work (no compute call is made here)."""
import ctypes
import os
import re

import pytest

import clblas_b200 as cb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "clblas_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^\s*(?:clblasStatus|clblasMem|void|unsigned long long|unsigned|double|const char\*|int)\s+(clblas\w+)\s*\(", text, flags=re.M)
    return sorted(set(names))


def test_header_symbols_exported():
    names = declared_functions()
    assert {"clblasSgemm", "clblasDgemm", "clblasStrsm", "clblasDtrsm", "clblasSetup", "clblasTeardown",
            "clblasGetVersion", "clblasB200PlanShards"} <= set(names)
    raw = ctypes.CDLL(cb.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in the header but not exported"
    assert set(names) == set(cb.EXPORTS)


def test_enum_and_status_values_match_reference_header():
    # src/clBLAS.h:78-113 (enums count from 0 in declaration order) and :123-155
    assert (cb.clblasRowMajor, cb.clblasColumnMajor) == (0, 1)
    assert (cb.clblasNoTrans, cb.clblasTrans, cb.clblasConjTrans) == (0, 1, 2)
    assert (cb.clblasUpper, cb.clblasLower) == (0, 1)
    assert (cb.clblasUnit, cb.clblasNonUnit) == (0, 1)
    assert (cb.clblasLeft, cb.clblasRight) == (0, 1)
    assert cb.clblasNotImplemented == -1024 and cb.clblasInsufficientMemVecY == -1007
    assert cb.clblasInvalidMatA == -1022 and cb.clblasInvalidDim == -1017 and cb.clblasInvalidLeadDimC == -1014
    text = open(HEADER).read()
    for name, val in cb.STATUS.items():
        assert re.search(rf"{name}\s*=\s*{val}\b", text), name


def test_version_is_reference_api_version():
    st, ver = cb.clblasGetVersion()
    assert st == cb.clblasSuccess and ver == (2, 12, 0)      # src/CMakeLists.txt:107-118


def test_null_buffers_rejected_before_any_device_work():
    """Check order of src/library/blas/xgemm.cc:685-706: memory objects first (A, then B, then C)."""
    args = (cb.clblasColumnMajor, cb.clblasNoTrans, cb.clblasNoTrans, 4, 4, 4, 1.0)
    q = [0]
    assert cb.clblasSgemm(*args, None, 0, 4, 8, 0, 4, 0.0, 8, 0, 4, queues=q) == cb.clblasInvalidMatA
    assert cb.clblasSgemm(*args, 8, 0, 4, None, 0, 4, 0.0, 8, 0, 4, queues=q) == cb.clblasInvalidMatB
    assert cb.clblasDgemm(*args, 8, 0, 4, 8, 0, 4, 0.0, None, 0, 4, queues=q) == cb.clblasInvalidMatC
    # M == 0 -> InvalidDim from the first size check (generic/common.c:601-603)
    assert cb.clblasDgemm(cb.clblasColumnMajor, 0, 0, 0, 4, 4, 1.0, 8, 0, 4, 8, 0, 4, 0.0, 8, 0, 4, queues=q) == cb.clblasInvalidDim
    # short leading dimension of A is found before anything is asked of the device
    assert cb.clblasSgemm(*args, 8, 0, 3, 8, 0, 4, 0.0, 8, 0, 4, queues=q) == cb.clblasInvalidLeadDimA


def test_trsm_queue_and_event_checks_come_first():
    """src/library/blas/xtrsm.cc:1623-1624: queues, then events, before anything else."""
    raw = cb.lib
    none_q = ctypes.POINTER(ctypes.c_void_p)()
    st = raw.clblasStrsm(1, 0, 0, 0, 1, 4, 4, 1.0, None, 0, 4, None, 0, 4, 0, none_q, 0, none_q, none_q)
    assert st == cb.clblasInvalidCommandQueue
    q = (ctypes.c_void_p * 1)(0)
    st = raw.clblasDtrsm(1, 0, 0, 0, 1, 4, 4, 1.0, None, 0, 4, None, 0, 4, 1, q, 2, none_q, none_q)
    assert st == cb.clblasInvalidEventWaitList


def test_plan_shards():
    """Column blocks aligned to 128 like the reference's DIVISION_ALIGNMENT
    (src/library/blas/generic/solution_seq_make.c:764), contiguous and complete."""
    assert cb.plan_shards(16384, 8) == [2048 * i for i in range(9)]
    assert cb.plan_shards(32768, 4) == [8192 * i for i in range(5)]
    b = cb.plan_shards(3001, 4, 128)
    assert b[0] == 0 and b[-1] == 3001 and all(x <= y for x, y in zip(b, b[1:]))
    assert all(x % 128 == 0 for x in b[:-1])
    assert cb.plan_shards(100, 8, 128) == [0] + [100] * 8       # fewer aligned pieces than devices
    assert cb.plan_shards(0, 2) == [0, 0, 0]
    for total in (1, 127, 128, 129, 4099, 100000):
        for parts in (1, 2, 3, 4, 8):
            b = cb.plan_shards(total, parts, 128)
            assert b[0] == 0 and b[-1] == total and len(b) == parts + 1
            assert all(0 <= y - x for x, y in zip(b, b[1:]))
