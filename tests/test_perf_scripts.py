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


def test_reference_arm_of_the_benchmark_maps_nothing_of_the_cuda_library():
    """`bench.py --impl reference` times the reference's CPU code only: the process must never import the CUDA package
    (or torch) and must print the same `config` object as the GPU arm builds for that workload."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import sys, json; sys.path.insert(0, %r); import bench\n"
        "bench.cpu_reference_sample = lambda wl, seconds_target=1.0, threads=None: (0.01, 4, 'port', 'stub sample')\n"
        "sys.argv = ['bench.py', '--impl', 'reference', '--steps', '2', '--warmup', '1']\n"
        "bench.main()\n"
        "maps = open('/proc/self/maps').read()\n"
        "print(json.dumps({'lib': 'libclblas_b200' in maps, 'pkg': 'clblas_b200' in sys.modules, 'torch': 'torch' in sys.modules}))\n" % root)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    line, flags = json.loads(lines[0]), json.loads(lines[1])
    assert flags == {"lib": False, "pkg": False, "torch": False}
    assert line["impl"] == "reference" and line["metric"] == "SGEMM TFLOP/s" and line["e2e"]["h2d_bytes_per_step"] == 0
    sys.path.insert(0, root)
    import bench
    assert line["config"] == bench.workloads()["sgemm32768"].config(1)
    assert line["cpu_baseline"]["kind"] in ("reference", "port")
