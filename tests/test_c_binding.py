"""The drop-in boundary from C: include/clblas_b200.h is valid C99, the library links from a plain C program, the
complex helper macros and constructors of the reference's clBLAS-complex.h are there, and an argument error is
reported through the return value before any device work (no GPU needed)."""
import os
import shutil
import subprocess

import pytest

import clblas_b200 as cb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_c99_program_compiles_links_and_runs(tmp_path):
    exe = str(tmp_path / "c_binding")
    libdir = os.path.dirname(cb.LIB_PATH)
    r = subprocess.run(["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
                        os.path.join(ROOT, "tests", "c_binding.c"), "-o", exe, "-L", libdir, "-lclblas_b200",
                        f"-Wl,-rpath,{libdir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    assert lines[0] == "0 2.12.0 1 4 8 16"          # status, version, CREAL / CIMAG, sizes of the complex types
    assert int(lines[1]) == cb.clblasInvalidMatA
