"""Helpers for the GPU parity tests: run one seeded case through the C-ABI on cuda:0."""
import numpy as np
import torch

import oracle
from oracle import NoTrans
from tests import cases


def dev(buf: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(buf).cuda()


def gemm_fn(cb, prec):
    return cb.clblasSgemm if prec == "s" else cb.clblasDgemm


def trsm_fn(cb, prec):
    return cb.clblasStrsm if prec == "s" else cb.clblasDtrsm


def run_gemm_gpu(cb, c, buffers=None):
    """Returns (status, C buffer after the call as numpy)."""
    A, B, C = buffers if buffers is not None else cases.gemm_buffers(c)
    dA, dB, dC = dev(A), dev(B), dev(C)
    st = gemm_fn(cb, c["prec"])(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], c["alpha"],
                                dA, c["offA"], c["lda"], dB, c["offB"], c["ldb"], c["beta"], dC, c["offC"], c["ldc"])
    torch.cuda.synchronize()
    return st, dC.cpu().numpy()


def run_gemm_oracle(c, buffers=None):
    A, B, C = buffers if buffers is not None else cases.gemm_buffers(c)
    C = C.copy()
    oracle.gemm(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"],
                B, c["offB"], c["ldb"], c["beta"], C, c["offC"], c["ldc"])
    return C


def run_trsm_gpu(cb, c, buffers=None):
    A, B = buffers if buffers is not None else cases.trsm_buffers(c)
    dA, dB = dev(A), dev(B)
    st = trsm_fn(cb, c["prec"])(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"],
                                dA, c["offA"], c["lda"], dB, c["offB"], c["ldb"])
    torch.cuda.synchronize()
    return st, dB.cpu().numpy()


def run_trsm_oracle(c, buffers=None):
    A, B = buffers if buffers is not None else cases.trsm_buffers(c)
    B = B.copy()
    oracle.trsm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A, c["offA"],
                c["lda"], B, c["offB"], c["ldb"])
    return B


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def outside_untouched(before, after, c, which="C"):
    """Every element of the flat buffer that is not part of the output matrix kept its bits."""
    if c["kind"] == "gemm":
        mask = oracle.outside_mask(before.size, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
    else:
        mask = oracle.outside_mask(before.size, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
    return np.array_equal(before[mask].view(np.uint8), after[mask].view(np.uint8))
