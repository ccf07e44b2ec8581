"""The native benchmark client (clblas_b200/client/client.cpp) with the reference client's options
(src/client/client.cpp:81-111): plain runs, --validate for gemm / trsm / trmm, --numQueues, --roundtrip, and -- on a
box with two GPUs -- the sharded --gpus run.  The client prints the reference's two result lines; a run passes when it
exits 0, prints them and, where asked, its validation line says PASS."""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLIENT = os.path.join(ROOT, "clblas_b200", "lib", "clblas_b200_client")


def _run(*args):
    r = subprocess.run([CLIENT, *map(str, args)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (args, r.stdout[-1000:], r.stderr[-1000:])
    assert re.search(r"BLAS kernel execution time < ns >: \d+", r.stdout), r.stdout
    m = re.search(r"BLAS kernel execution Gflops < .* >: ([0-9.]+)", r.stdout)
    assert m and float(m.group(1)) > 0, r.stdout
    return r.stdout


@pytest.mark.parametrize("args", [
    ("-f", "gemm", "-r", "s", "-m", 700, "-n", 650, "-k", 333, "--transposeB", 1, "-v", 1),
    ("-f", "gemm", "-r", "d", "-m", 512, "-n", 384, "-k", 640, "-o", 0, "--transposeA", 1, "-v", 1),
    ("-f", "trsm", "-r", "d", "-m", 600, "-n", 200, "--uplo", 1, "--diag", 1, "-v", 1),
    ("-f", "trsm", "-r", "s", "-m", 150, "-n", 420, "--side", 1, "--uplo", 0, "--transposeA", 1, "--diag", 1, "-o", 0, "-v", 1),
    ("-f", "trmm", "-r", "d", "-m", 300, "-n", 260, "--uplo", 1, "--diag", 1, "--alpha", 2, "-v", 1),
])
def test_validate(args):
    out = _run(*args, "-p", 2, "--apiCallCount", 2)
    assert "validation:" in out and "PASS" in out and "FAIL" not in out, out


def test_several_queues_and_roundtrip():
    _run("-f", "gemm", "-r", "d", "-m", 1025, "-n", 1025, "-k", 513, "--numQueues", 3, "-p", 2, "--apiCallCount", 2)
    _run("-f", "gemm", "-r", "s", "-m", 2048, "-n", 2048, "-k", 1024, "--roundtrip", "-p", 2, "--apiCallCount", 2)
    _run("-f", "trsm", "-r", "d", "-m", 1024, "-n", 2048, "--uplo", 1, "--diag", 1, "--roundtrip", "-p", 2, "--apiCallCount", 2)


def test_sharded_run_on_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    env_nvls = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for args in (("-f", "gemm", "-r", "s", "-m", 2048, "-n", 4096, "-k", 2048, "--transposeB", 1),
                 ("-f", "trsm", "-r", "d", "-m", 2048, "-n", 1024, "--uplo", 1, "--diag", 1)):
        r = subprocess.run([CLIENT, *map(str, args), "--gpus", "2", "-p", "2", "--apiCallCount", "2"], capture_output=True, text=True,
                           timeout=300, env=env_nvls)
        assert r.returncode == 0 and "2 GPUs" in r.stdout, (r.stdout[-1000:], r.stderr[-1000:])
