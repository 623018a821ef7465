"""The C++ host side: containers/dispatcher mirror (CPU), the GPU-B200 competitor behind the reference's
interface (GPU), and that the competitor header compiles against the reference's own headers."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "dphpc_b200"
SRC = PKG / "src"
OUT = ROOT / "tests" / "cpp" / "_build"
REFERENCE = Path(os.environ.get("SDDMM_REFERENCE_ROOT", str(ROOT.parent / "reference")))   # the reference checkout, beside this repository


def compile_cpp(name, sources, extra=()):
    OUT.mkdir(exist_ok=True)
    exe = OUT / name
    cmd = ["g++", "-O1", "-std=c++17", "-Wall", "-I", str(SRC), "-I", str(ROOT / "include"), "-I", str(ROOT / "tests" / "cpp"),
           "-o", str(exe), *map(str, sources), "-L", str(PKG), "-lsddmm_datasets", f"-Wl,-rpath,{PKG}", "-pthread", *extra]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-4000:]
    return exe


def test_host_staging_cpp():
    """Thread pool and copies of dphpc_b200/csrc/host_staging.cuh (host code only: compiled with g++ against the CUDA headers)."""
    cuda_inc = Path("/usr/local/cuda/include")
    if not (cuda_inc / "cuda_runtime.h").exists():
        pytest.skip("CUDA headers not found")
    exe = compile_cpp("host_staging_tests", [ROOT / "tests" / "cpp" / "host_staging_tests.cpp"],
                      extra=["-x", "c++", "-I", str(ROOT / "dphpc_b200" / "csrc"), "-I", str(cuda_inc), "-msse2"])
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-4000:]
    assert "0 failures" in res.stdout


def test_containers_and_dispatcher_cpp():
    exe = compile_cpp("container_tests", [ROOT / "tests" / "cpp" / "container_tests.cpp"])
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-4000:]
    assert "0 failures" in res.stdout


def test_benchmark_driver_builds():
    from dphpc_b200 import build

    exe = build.build_bench()
    assert exe.exists()
    res = subprocess.run([str(exe), "--bogus"], capture_output=True, text=True)
    assert res.returncode == 2 and "usage" in res.stderr


@pytest.mark.skipif(not (REFERENCE / "src" / "benchmark" / "competitor.hpp").exists(), reason="reference checkout absent")
def test_competitor_header_drops_into_the_reference_tree(tmp_path):
    # compile GPUB200 against the reference's OWN competitor.hpp / matrices (not this repository's mirror)
    tu = tmp_path / "dropin.cpp"
    tu.write_text('#include <cmath>\n#include "competitors/gpu/gpu_b200.hpp"\n#include "competitors/gpu/gpu_b200_multi.hpp"\n'
                  "int main() { Competitors::GPUB200 c; Competitors::GPUB200Multi m; SDDMM::Competitor<float> *p = &c, *q = &m;\n"
                  "             return p->is_gpu() && q->is_gpu() ? 0 : 1; }\n")
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-w", "-include", "cstdint", "-include", "cassert", "-I", str(REFERENCE / "src"),
           "-I", str(cuda_inc), "-I", str(ROOT / "include"), "-idirafter", str(SRC), str(tu)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-4000:]


@pytest.mark.gpu
def test_competitor_behind_the_reference_interface():
    oracle_c = ROOT / "oracle" / "sddmm_oracle.c"
    OUT.mkdir(exist_ok=True)
    obj = OUT / "sddmm_oracle.o"
    res = subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-c", "-o", str(obj), str(oracle_c)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    exe = compile_cpp("competitor_tests", [ROOT / "tests" / "cpp" / "competitor_tests.cpp", obj], extra=["-lsddmm_b200"])
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=900)
    lines = [ln for ln in res.stdout.splitlines() if not ln.startswith(("GPU-B200", "CPU-Basic"))]   # drop the CSV rows
    assert res.returncode == 0, "\n".join(lines[-60:]) + res.stderr[-2000:]
    assert "0 failures" in res.stdout


@pytest.mark.gpu
def test_benchmark_driver_reads_matrix_files(tmp_path):
    # sddmm_bench on a MatrixMarket file and on an edge list: CSV rows with correctness = 1 for both competitors
    import numpy as np
    from dphpc_b200 import build

    exe = build.build_bench()
    rng = np.random.default_rng(5)
    M, N, nnz = 300, 200, 4000
    flat = rng.choice(M * N, size=nnz, replace=False)
    mtx = tmp_path / "m.mtx"
    with open(mtx, "w") as f:
        f.write("%%MatrixMarket matrix coordinate real general\n% generated\n")
        f.write(f"{M} {N} {nnz}\n")
        for p in flat:
            f.write(f"{p // N + 1} {p % N + 1} {rng.uniform(0.1, 1.0):.6f}\n")
    edges = tmp_path / "e.txt"
    with open(edges, "w") as f:
        f.write("# edge list\n")
        for p in flat[:1500]:
            f.write(f"{p // N}\t{p % N}\n")
    for args in (["--mtx", str(mtx)], ["--edges", str(edges), "--rows", str(M), "--cols", str(N)]):
        res = subprocess.run([str(exe), *args, "-k", "32", "--num_runs", "2"], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
        rows = [ln.split(",") for ln in res.stdout.splitlines() if ln.startswith("GPU-B200")]
        header = next(ln.split(",") for ln in res.stdout.splitlines() if ln.startswith("competitor"))
        ci = header.index("correctness")
        assert len(rows) >= 2 and all(r[ci].strip() == "1" for r in rows), res.stdout[-2000:]


@pytest.mark.gpu
def test_competitor_under_the_reference_harness_unmodified():
    # oracle/_ref/ref_harness_bench = the reference's own Benchmark<float>, datasets and CPU-Basic (first competitor =
    # correctness baseline) compiled from its sources where they lie, with GPU-B200 registered beside it.  The binary is
    # built where the reference checkout is present and travels as a prebuilt file.
    exe = ROOT / "oracle" / "_ref" / "ref_harness_bench"
    if not exe.exists():
        pytest.skip("oracle/_ref/ref_harness_bench not built (reference checkout absent)")
    res = subprocess.run([str(exe), "2"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    rows = [ln.split(",") for ln in res.stdout.splitlines() if ln.count(",") >= 13]
    mine = [r for r in rows if r[0].startswith("GPU-B200")]
    datasets = {r[1] for r in mine}
    assert {"Dummy", "RandomWithDensity", "LatinHypercube"} <= datasets, res.stdout[-3000:]
    assert {r[2] for r in mine} == {"CSR", "COO"}
    wrong = [r[:3] for r in mine if r[11].strip() != "1"]
    assert not wrong, f"correctness = 0 under the reference's harness: {wrong}\n{res.stderr[-2000:]}"
    assert all(int(r[9]) > 0 for r in mine)   # the harness' own CUDA-event pair saw the compute phase
    assert "entry_device_kept=1" in res.stdout
