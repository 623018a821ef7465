"""Build recipe for the CPU checkers (test infrastructure, never the product path).

    python oracle/build.py

  oracle/liboracle.so           gcc -O2 -ffp-contract=off oracle/sddmm_oracle.c
  oracle/_ref/libsddmm_ref.so   g++ -O2 on oracle/ref_shim.cpp against the UNMODIFIED reference
                                headers where they lie (-I<reference>/src); built only when the
                                reference checkout is present.  -O2 is the optimisation level of
                                the reference's Release build.  The two forced includes are needed
                                because src/matrices/CSR.hpp uses uint32_t/assert without
                                including <cstdint>/<cassert> under GCC 13, and the CUDA include
                                directory because CSR.hpp:13 includes <cuda_runtime.h>.
Outputs are git-ignored; oracle/_ref/ travels to the GPU box as a prebuilt binary.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ORACLE_LIB = HERE / "liboracle.so"
REF_DIR = HERE / "_ref"
REF_LIB = REF_DIR / "libsddmm_ref.so"
REF_HARNESS = REF_DIR / "ref_harness_bench"
# the reference checkout: SDDMM_REFERENCE_ROOT, else a directory "reference" beside this repository
REFERENCE_ROOT = Path(os.environ.get("SDDMM_REFERENCE_ROOT", str(HERE.parent.parent / "reference")))
CUDA_INCLUDE = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"


def _stale(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).exists() and Path(s).stat().st_mtime > t for s in sources)


def _run(cmd) -> None:
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("oracle build failed: " + " ".join(map(str, cmd)))


def build_oracle(force: bool = False) -> Path:
    src = HERE / "sddmm_oracle.c"
    if force or _stale(ORACLE_LIB, [src]):
        _run(["gcc", "-O2", "-ffp-contract=off", "-std=c11", "-fPIC", "-shared", "-Wall", "-o", str(ORACLE_LIB), str(src)])
    return ORACLE_LIB


def reference_present() -> bool:
    return (REFERENCE_ROOT / "src" / "competitors" / "cpu" / "cpu_basic.hpp").exists()


def build_ref(force: bool = False):
    """Compile the reference's CPU path from its own sources; returns None when they are absent."""
    if not reference_present():
        return REF_LIB if REF_LIB.exists() else None
    src = HERE / "ref_shim.cpp"
    if force or _stale(REF_LIB, [src]):
        REF_DIR.mkdir(exist_ok=True)
        _run([
            "g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-w",
            "-include", "cstdint", "-include", "cassert",
            "-I", str(REFERENCE_ROOT / "src"), "-I", str(CUDA_INCLUDE),
            "-o", str(REF_LIB), str(src),
        ])
    return REF_LIB


def build_ref_harness(force: bool = False):
    """The reference's unmodified Benchmark<T> + datasets + CPU-Basic, with this repository's GPU-B200 competitor
    registered next to it (oracle/ref_harness_main.cpp); links the CUDA runtime (the harness times with CUDA events)
    and the engine's C-ABI library.  Returns None when the reference, the CUDA runtime or the engine library is absent."""
    pkg = HERE.parent / "dphpc_b200"
    cuda_lib = CUDA_INCLUDE.parent / "lib64"
    if not reference_present() or not (pkg / "libsddmm_b200.so").exists() or not cuda_lib.exists():
        return REF_HARNESS if REF_HARNESS.exists() else None
    src = HERE / "ref_harness_main.cpp"
    deps = [src, pkg / "src" / "competitors" / "gpu" / "gpu_b200.hpp", HERE.parent / "include" / "sddmm_b200.h"]
    if force or _stale(REF_HARNESS, deps):
        REF_DIR.mkdir(exist_ok=True)
        _run([
            "g++", "-std=c++17", "-O2", "-w", "-include", "cstdint", "-include", "cassert",
            "-I", str(REFERENCE_ROOT / "src"), "-I", str(CUDA_INCLUDE), "-I", str(HERE.parent / "include"),
            "-idirafter", str(pkg / "src"),   # only gpu_b200.hpp comes from here: every other header is the reference's
            "-o", str(REF_HARNESS), str(src),
            "-L", str(pkg), "-lsddmm_b200", "-L", str(cuda_lib), "-lcudart",
            "-Wl,-rpath,$ORIGIN/../../dphpc_b200", f"-Wl,-rpath,{cuda_lib}", "-pthread",
        ])
    return REF_HARNESS


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
    print(build_ref_harness(force="--force" in sys.argv))
