"""In-tree build of the native libraries (nvcc / g++ only, no CMake, no Torch).

    python -m dphpc_b200.build            # build whatever is out of date
    python -m dphpc_b200.build --force

Products (next to this file, git-ignored):
    libsddmm_b200.so      CUDA engine + C ABI (include/sddmm_b200.h), sm_100a only
    libsddmm_datasets.so  seeded synthetic inputs (include/sddmm_datasets.h), host only
    sddmm_bench           C++ benchmark driver built on the competitor interface
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"

ENGINE_LIB = PKG / "libsddmm_b200.so"
DATASETS_LIB = PKG / "libsddmm_datasets.so"
BENCH_BIN = PKG / "sddmm_bench"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
    "-Xptxas=-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA engine cannot be built")
    return exe


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, log_name: str) -> None:
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    (PKG / log_name).write_text(" ".join(map(str, cmd)) + "\n" + res.stdout)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd))}")


def engine_sources():
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h")))


def build_engine(force: bool = False) -> Path:
    srcs = engine_sources()
    if force or _newer(ENGINE_LIB, srcs):
        cu = sorted(CSRC.glob("*.cu"))
        cmd = [_nvcc(), *NVCC_FLAGS, "-shared", "-o", str(ENGINE_LIB), *map(str, cu), "-ldl"]
        _run(cmd, "build_engine.log")
    return ENGINE_LIB


def build_datasets(force: bool = False) -> Path:
    src = CSRC / "datasets.cpp"
    if force or _newer(DATASETS_LIB, [src, INCLUDE / "sddmm_datasets.h"]):
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-Wall", "-o", str(DATASETS_LIB), str(src)]
        _run(cmd, "build_datasets.log")
    return DATASETS_LIB


def build_bench(force: bool = False) -> Path:
    """The C++ driver: competitor interface + harness + synthetic datasets."""
    src_dir = PKG / "src"
    main = src_dir / "main.cpp"
    if not main.exists():
        return BENCH_BIN
    srcs = [p for p in src_dir.rglob("*") if p.suffix in (".cpp", ".hpp", ".h")]
    if force or _newer(BENCH_BIN, srcs + [ENGINE_LIB, DATASETS_LIB]):
        cmd = [
            "g++", "-O2", "-ffp-contract=off", "-std=c++17", "-Wall", "-I", str(src_dir), "-I", str(INCLUDE),
            "-o", str(BENCH_BIN), str(main),
            "-L", str(PKG), "-lsddmm_b200", "-lsddmm_datasets", f"-Wl,-rpath,{PKG}", "-Wl,-rpath,$ORIGIN", "-pthread",
        ]
        _run(cmd, "build_bench.log")
    return BENCH_BIN


def build_all(force: bool = False) -> None:
    build_engine(force)
    build_datasets(force)
    build_bench(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", ENGINE_LIB.name, DATASETS_LIB.name, BENCH_BIN.name if BENCH_BIN.exists() else "")
