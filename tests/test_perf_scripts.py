"""Host logic of the performance scripts (counterparts of the reference's src/scripts/perf): size-list syntax of the
sweep driver and the side-by-side comparison of two tables in the reference's CSV schema."""
import importlib.util
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PERF = os.path.join(ROOT, "clblas_b200", "perf")


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(PERF, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_size_list_syntax():
    mp = _load("measure_performance")
    assert mp.expand("1024") == [1024]
    assert mp.expand("512-2048:512") == [512, 1024, 1536, 2048]
    assert mp.expand("15,2048-3000:500") == [15, 2048, 2548]
    assert mp.HEADER.split(",")[:3] == ["m", "n", "k"] and mp.HEADER.endswith("GFLOPS")


def test_compare_tables(tmp_path):
    a, b = tmp_path / "a.csv", tmp_path / "b.csv"
    a.write_text("m,n,k,label,GFLOPS\n1024,1024,1024,x,2000\n4096,4096,4096,x,8000\n")
    b.write_text("m,n,k,label,GFLOPS\n960,960,960,y,100\n4032,4032,4032,y,400\n")
    r = subprocess.run([sys.executable, os.path.join(PERF, "compare_performance.py"), str(a), str(b)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    rows = [ln.split() for ln in r.stdout.splitlines() if ln and not ln.startswith("#") and not ln.lstrip().startswith("m (A)")]
    assert rows == [["1024", "2000.0", "960", "100.0", "20.0"], ["4096", "8000.0", "4032", "400.0", "20.0"]]
    # the tables shipped with the library parse
    shipped = os.path.join(ROOT, "doc", "performance", "B200", "clblas_b200_dgemm_col_nt.csv")
    r = subprocess.run([sys.executable, os.path.join(PERF, "compare_performance.py"), shipped, shipped], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.count("\n") >= 16
