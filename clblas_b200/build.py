"""Builds libclblas_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python clblas_b200/build.py [--force]

Every .cu file under csrc/ is compiled to an object under build/ and linked into
lib/libclblas_b200.so; the native benchmark client (client/client.cpp) is linked against it.
Objects are rebuilt when their source or any header is newer.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libclblas_b200.so")
CLIENT_SRC = os.path.join(HERE, "client", "client.cpp")
CLIENT = os.path.join(LIBDIR, "clblas_b200_client")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-O3,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr",
]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src: str, obj: str) -> str:
    cmd = [NVCC, *NVCC_FLAGS, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    jobs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if force or _newer(obj, [src, *headers]):
            jobs.append((src, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for (src, _), log in zip(jobs, ex.map(lambda j: _compile(*j), jobs)):
                if verbose:
                    print(f"[build] {os.path.basename(src)}\n{log}", file=sys.stderr)
    objs = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in sources]
    # drop objects whose source was removed
    for o in glob.glob(os.path.join(OBJ, "*.o")):
        if o not in objs:
            os.remove(o)
    if force or jobs or _newer(LIB, objs):
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if os.path.exists(CLIENT_SRC) and (force or _newer(CLIENT, [CLIENT_SRC, LIB, *headers])):
        cmd = [NVCC, "-O2", "-std=c++17", "-o", CLIENT, CLIENT_SRC, "-L" + LIBDIR, "-lclblas_b200",
               "-Xlinker", "-rpath,$ORIGIN", "-Xcompiler", "-fopenmp"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"client build failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
