#!/usr/bin/env python
"""SDDMM benchmark: P_ij = S_ij * (A_i . B_j) on seeded synthetic inputs, B200 engine vs host CPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C] [--k K] [--mode fp32|bf16|tf32|fp32_tc]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...      (N > 1: one rank per GPU)
    python bench.py --impl reference ...      (the reference's own CPU SDDMM on the host cores)

One step = one SDDMM over the whole sparse matrix.  For N > 1 the matrix is cut into
blocks, one per rank (dphpc_b200.partition.block_grid): nnz-balanced row ranges and, when B is
far larger than L2 and the rows are long enough, equal column ranges as well, so that each
rank gathers from a slice of B that stays in its L2.  A is row-sliced, B is broadcast once
over NCCL before the timed region, and no collective runs inside a step (strong scaling:
the total work is fixed).  Rank 0 prints one JSON line.

  value     GFLOP/s = 2*nnz*K / t with all operands resident in HBM; t = mean device time of a
            step (CUDA events on the engine's stream around its kernels), max over ranks;
            L2 is flushed between steps
  e2e       same metric through the host-buffer call sddmm_b200_pipeline_sddmm_csr (pinned host
            buffers: H2D of S, A, B + device-side plan, run, D2H of P.val, overlapped over row
            chunks), host wall clock, max over ranks; e2e.single_engine = the same through
            upload_csr -> run -> download on one engine; e2e.competitor = the C++ competitor
            GPUB200::init_csr + run_csr + cleanup_csr on the harness' pageable containers
  per_config  kernel-only figures of the other configurations and modes and of the K sweep
            (K = 64, 128, 256 in fp32 and bf16 storage), on the same kind of row shards, each
            with its own roofline fraction; max over ranks
  parity    every rank checks a sample of its shard's output against the CPU oracle outside
            the timed region
  roofline  algorithmic bytes of the dominant kernel / its mean device time, against the
            measured HBM copy bandwidth (MEASURED_PEAKS.json) or the 6650 GB/s fallback
  cpu_baseline  the reference's CPUBasic::run_csr (oracle/_ref, else the oracle port) on the host
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle"))   # the CPU checker: used by the cpu_baseline leg and the reference arm only

CONFIG_K = {1: 32, 2: 32, 3: 64, 4: 32, 5: 32}
CONFIG_NAME = {
    1: "config1 small-uniform 656^2 nnz 18,964",
    2: "config2 clustered 64x64 blocks 14,340^2 nnz 18.07M",
    3: "config3 banded 3x3 blocks 503,712^2 nnz 36.8M",
    4: "config4 power-law 2,601,977^2 nnz 36.2M",
    5: "config5 poisson-rows 1,453,908^2 nnz 37.5M",
}
DEFAULT_CONFIG = 5   # the largest K=32 configuration (configs[4]); it fits one GPU
FALLBACK_HBM_GBS = 6650.0
L2_FLUSH_BYTES = 512 << 20


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback 6650 GB/s (MEASURED_PEAKS.json absent)"


def tensor_peak():
    """Measured dense bf16 tensor throughput (TFLOP/s, burst) the tensor-path figure is compared with."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops)"
        except Exception:
            pass
    return 1590.0, "fallback 1590 TFLOP/s (MEASURED_PEAKS.json absent)"


def measured_traffic(kernel, workload_key):
    """DRAM bytes per launch from the committed ncu capture, if one covers this kernel and workload."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if not p.exists():
        return None
    try:
        return json.loads(p.read_text()).get(f"{kernel}:{workload_key}")
    except Exception:
        return None


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc = None
        self.path = Path(f"/tmp/sddmm_clocks_{os.getpid()}.csv")
        exe = shutil.which("nvidia-smi")
        if exe:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen([exe, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(gpu_index),
                                          "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            out["note"] = "nvidia-smi not found"
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.f.close()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.path.read_text().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); pw.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower() == "active":
                    reasons.add(n)
        self.path.unlink(missing_ok=True)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), power_w_max=float(max(pw)), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


def pinned_copy(lib, arr):
    """Copy a numpy array into pinned host memory from the engine library; returns (address, view)."""
    import ctypes as C
    p = C.c_void_p()
    if lib.sddmm_b200_host_alloc(C.byref(p), arr.nbytes):
        raise RuntimeError("pinned host allocation failed")
    buf = (C.c_char * max(arr.nbytes, 1)).from_address(p.value)
    view = np.frombuffer(buf, dtype=arr.dtype, count=arr.size)
    view[...] = arr.ravel()
    return p.value, view


def cpu_reference(M, N, K, row_ptr, col_idx, s_val, A, B, max_nnz, reps):
    """Time the reference's CPU SDDMM on a row-prefix sample of the workload: on all host threads (row ranges running
    concurrently, see CpuRowShards) and, for the record, on one thread (what the reference itself does)."""
    r_end = int(np.searchsorted(row_ptr, max_nnz, side="right") - 1) if row_ptr[M] > max_nnz else M
    r_end = max(1, min(M, r_end))
    out = {}
    for label, threads in (("all", host_threads()), ("one", 1)):
        shards = CpuRowShards(M, N, K, row_ptr, col_idx, s_val, A, B, r_end, threads)
        shards.step()   # warm-up
        t = float(np.median([shards.step() for _ in range(reps)]))
        out[label] = (shards.threads, shards.kind, shards.nnz, t)
        shards.close()
    threads, kind, nnz_s, t = out["all"]
    _, _, _, t1 = out["one"]
    return {"value": 2.0 * nnz_s * K / t / 1e9, "unit": "GFLOP/s", "cores": threads, "kind": kind,
            "sample": f"rows [0,{r_end}) of the workload = {nnz_s} nnz cut into {threads} nnz-balanced row ranges, each running "
                      f"CPUBasic::run_csr on its own host thread; median of {reps} runs, {t * 1e3:.1f} ms each",
            "single_thread": {"value": 2.0 * nnz_s * K / t1 / 1e9, "unit": "GFLOP/s", "ms": t1 * 1e3,
                              "what": "the same sample in one call of CPUBasic::run_csr (the reference has no threading)"},
            "host_cores_available": os.cpu_count()}, t, nnz_s


def host_threads():
    """Host threads the CPU legs may use (the cores this process is allowed to run on, at most 64)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(64, n))


class CpuRowShards:
    """The reference's CPU SDDMM on all host threads: the rows [0, r_end) are cut into nnz-balanced contiguous ranges
    (the way the GPU arm shards rows), every range is its own problem object of the UNMODIFIED reference code
    (CPUBasic::run_csr), and the ranges run concurrently, one host thread each (ctypes drops the GIL during the call).
    A step takes as long as its slowest range.  Falls back to the C restatement when the reference library is absent."""

    def __init__(self, M, N, K, row_ptr, col_idx, s_val, A, B, r_end, threads):
        import oracle_lib
        from dphpc_b200.partition import row_cuts
        self.ref = oracle_lib.Reference.try_load()
        self.kind = "reference" if self.ref is not None else "port"
        self.nnz = int(row_ptr[r_end])
        rp = np.ascontiguousarray(row_ptr[:r_end + 1])
        threads = max(1, min(threads, r_end))
        cuts = row_cuts(rp, threads) if threads > 1 else [0, r_end]
        self.parts = []
        self.ranges = []   # row range of every part
        orc = None if self.ref is not None else oracle_lib.Oracle()
        for a, b in zip(cuts[:-1], cuts[1:]):
            if b <= a:
                continue
            self.ranges.append((int(a), int(b)))
            lo, hi = int(rp[a]), int(rp[b])
            sub_rp = np.ascontiguousarray(rp[a:b + 1] - lo)
            ci, sv = np.ascontiguousarray(col_idx[lo:hi]), np.ascontiguousarray(s_val[lo:hi])
            Aa = np.ascontiguousarray(A[a:b])
            if self.ref is not None:
                run, _, destroy = self.ref.problem(b - a, N, K, sub_rp, ci, sv, Aa, B)
                self.parts.append((run, destroy))
            else:
                out = np.empty(hi - lo, np.float32)
                Bc = np.ascontiguousarray(B)
                self.parts.append(((lambda sub_rp=sub_rp, ci=ci, sv=sv, Aa=Aa, out=out, n=b - a:
                                    orc.sddmm_csr_rows(0, n, K, sub_rp, ci, sv, Aa, Bc, out)), (lambda: None)))
        self.threads = len(self.parts)
        from concurrent.futures import ThreadPoolExecutor
        self.pool = ThreadPoolExecutor(max_workers=self.threads)

    def step(self):
        """One pass over the sample on all threads; wall seconds."""
        t0 = time.perf_counter()
        list(self.pool.map(lambda p: p[0](), self.parts))
        return time.perf_counter() - t0

    def close(self):
        self.pool.shutdown()
        for _, destroy in self.parts:
            destroy()


def workload_config(cfg, K, mode, world, grid=None):
    part = (f"{world} nnz-balanced row range(s), B replicated" if grid is None or grid[1] == 1 else
            f"{grid[0]} nnz-balanced row range(s) x {grid[1]} equal column range(s): each rank one block with its rows of A and of B")
    return {"workload": f"{CONFIG_NAME[cfg]}, K={K}, A/B uniform [-1,1), seeded synthetic", "config_id": cfg, "k": K,
            "mode": mode, "partition": part, "l2": "flushed between steps (512 MiB write)"}


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    from dphpc_b200 import Dataset
    cfg, K = args.config, args.k or CONFIG_K[args.config]
    d = Dataset(cfg, K, args.scale)
    total = args.steps + args.warmup
    # bound each step so the whole run stays within a few minutes (CPUBasic does ~1-2 GFLOP/s)
    budget_nnz = int(max(2e5, min(d.nnz, 150.0 / max(total, 1) * 1.0e9 / (2 * K))))
    threads = host_threads()
    budget_nnz = min(d.nnz, budget_nnz * threads)   # the sample grows with the threads that share it
    r_end = int(np.searchsorted(d.row_ptr, budget_nnz, side="right") - 1) if d.nnz > budget_nnz else d.M
    r_end = max(1, min(d.M, r_end))
    shards = CpuRowShards(d.M, d.N, K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, r_end, threads)
    nnz_s = shards.nnz
    step, destroy = shards.step, shards.close
    for _ in range(args.warmup):
        step()
    ts = [step() for _ in range(args.steps)]
    destroy()
    tm = float(np.mean(ts))
    val = 2.0 * nnz_s * K / tm / 1e9
    from dphpc_b200.partition import block_grid
    ref_grid = block_grid(max(1, args.gpus), d.M, d.N, K, d.nnz, elem_bytes=2 if args.mode == "bf16" else 4)
    line = {
        "impl": "reference", "metric": "SDDMM GFLOP/s (2*nnz*K/t)", "value": val, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": tm * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, K, args.mode, max(1, args.gpus), ref_grid),   # the same workload description as the GPU arm prints
        "cpu_baseline": {"value": val, "unit": "GFLOP/s", "cores": shards.threads, "kind": shards.kind,
                         "sample": f"each step = CPUBasic::run_csr over rows [0,{r_end}) = {nnz_s} of {d.nnz} nnz, cut into "
                                   f"{shards.threads} nnz-balanced row ranges that run concurrently (one host thread each)",
                         "host_cores_available": os.cpu_count()},
        "e2e": {"value": val, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def kernel_only_stats(eng, steps, warmup, flush):
    """(median ms per step, {kernel: mean ms}) with L2 flushed before every step."""
    for _ in range(warmup):
        eng.run(); eng.sync()
    tot, per = [], {}
    for _ in range(steps):   # step time: no instrumentation between the kernels
        flush()
        eng.run(); eng.sync()
        tot.append(eng.last_run_ms())
    eng.set_kernel_timing(True)
    for _ in range(max(3, steps // 2)):   # per-kernel times: separate, instrumented steps
        flush()
        eng.run(); eng.sync()
        for name, ms in eng.kernel_times():
            per.setdefault(name, []).append(ms)
    eng.set_kernel_timing(False)
    return float(np.median(tot)), {k: float(np.mean(v)) for k, v in per.items()}


def shard_of(d, rank, world, mode="fp32"):
    """This rank's block of a dataset as a problem of its own (dphpc_b200.partition.block_shard): nnz-balanced row ranges
    (64-row aligned cuts keep the global tile grid) and, where B is far larger than L2 and the rows are long enough, equal
    column ranges as well, so that every device gathers from a slice of B that stays in its L2."""
    from dphpc_b200.partition import block_grid, block_shard
    grid = block_grid(world, d.M, d.N, d.K, d.nnz, elem_bytes=2 if mode == "bf16" else 4)
    return block_shard(d.row_ptr, d.col_idx, d.s_val, d.A, d.B, rank, grid, align=64 if d.M >= 64 * 8 * grid[0] else 1)


def dominant_kernel(kern, plan):
    """The kernel that owns most nonzeros (when two kernels overlap on the device, the event pair of the small residual
    kernel also spans its wait for a free SM, so time alone does not say which one dominates)."""
    if not kern:
        return None
    if len(kern) > 1:
        others = [k for k in kern if k != "sddmm_dense_tile_kernel"]
        return "sddmm_dense_tile_kernel" if 2 * plan["dense_nnz"] >= plan["nnz"] or not others else others[0]
    return next(iter(kern))


def roofline_block(eng, plan, kern, mode, K, cfg, world, peak, peak_src):
    dom = dominant_kernel(kern, plan)
    if not dom:
        return None
    dom_ms = float(kern[dom])
    alg = eng.algorithmic_bytes()
    if len(kern) > 1:   # split the compulsory bytes between the kernels by the nonzeros each one owns
        share = plan["dense_nnz"] / max(1, plan["nnz"])
        alg = alg * (share if "dense" in dom else 1.0 - share)
    ach = alg / (dom_ms * 1e-3) / 1e9
    eb = 2 if mode == "bf16" else 4
    out = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
           # the committed ncu capture is of the whole matrix on one GPU: no figure for a shard of it
           "traffic": measured_traffic(dom, f"config{cfg}_k{K}_{mode}") if world == 1 else None,
           "algorithmic_bytes_per_launch": int(alg), "launch_ms": dom_ms, "peak_source": peak_src, "kernels_ms": dict(kern),
           # what the same nonzeros would move if no gathered B row were ever reused (every nonzero fetches its own B row)
           "gather_model_bytes": int(eb * K * (plan["rows_nonempty"] + plan["nnz"]) + 12 * plan["nnz"] + 4 * (plan["rows"] + 1))}
    if "dense" in dom:
        # the dense contraction the tensor cores execute: 64x64xK' per tile (K' = 3K for the 3-term tf32 split)
        kp = 3 * K if mode == "fp32_tc" else K
        tpeak, tsrc = tensor_peak()
        tfl = 2.0 * 64 * 64 * kp * plan["dense_tiles"] / (dom_ms * 1e-3) / 1e12
        out["tensor"] = {"dense_tile_tflops": tfl, "peak_tflops": tpeak, "frac": tfl / tpeak, "peak_source": tsrc,
                         "note": "tensor throughput is not what bounds this path (8 B per nonzero of HBM traffic is)"}
    return out


def parity_sample(p, sh, K, mode, sample=200000, edge_rows=2000):
    """Outside the timed region: this rank's downloaded P block against the CPU oracle -- `sample` random nonzeros plus the
    first and last `edge_rows` rows of the block (the block is a problem of its own: local row_ptr, re-based columns, its
    rows of A and of B).  Returns (checked nonzeros, max |err| / (tol * |s| sum|ab|))."""
    import oracle_lib
    tol = 1e-5 if mode in ("fp32", "fp32_tc") else 1e-2
    orc = oracle_lib.Oracle()
    M, nnz = sh["M"], sh["nnz"]
    if nnz == 0:
        return 0, 0.0
    rp, col, val = np.ascontiguousarray(sh["rp"]), np.ascontiguousarray(sh["col"]), np.ascontiguousarray(sh["val"])
    A, B = np.ascontiguousarray(sh["A"]), np.ascontiguousarray(sh["B"])
    worst, checked = 0.0, 0
    for a, b in {(0, min(M, edge_rows)), (max(0, M - edge_rows), M)}:
        ja, jb = int(rp[a]), int(rp[b])
        if jb <= ja:
            continue
        ref = np.zeros(nnz, np.float32)
        orc.sddmm_csr_rows(a, b, K, rp, col, val, A, B, ref)
        rows = np.repeat(np.arange(a, b), np.diff(rp[a:b + 1]))
        bound = oracle_lib.abs_dot_bound(rows, col[ja:jb], val[ja:jb], A, B)
        err = np.abs(p[ja:jb].astype(np.float64) - ref[ja:jb])
        worst = max(worst, float(np.max(err / (tol * bound + 1e-30))))
        checked += jb - ja
    rng = np.random.default_rng(1234 + sh["r0"] + 7 * sh["c0"])
    idx = np.sort(rng.choice(nnz, min(sample, nnz), replace=False))
    rows = (np.searchsorted(rp, idx, side="right") - 1).astype(np.int64)
    want = oracle_lib.dot_f64(rows, col[idx], val[idx], A, B)
    bound = oracle_lib.abs_dot_bound(rows, col[idx], val[idx], A, B)
    err = np.abs(p[idx].astype(np.float64) - want)
    worst = max(worst, float(np.max(err / (max(tol, 2e-6) * bound + 1e-30))))
    if not np.isfinite(p).all():
        worst = float("inf")
    return checked + idx.size, worst


def competitor_e2e(cfg, K, mode, runs=3):
    """init_csr + run_csr + cleanup_csr of the C++ competitor on the harness' pageable std::vector containers: what a
    maintainer who registers GPUB200 in the reference's driver gets (total_ns column of the CSV)."""
    exe = ROOT / "dphpc_b200" / "sddmm_bench"
    if not exe.exists():
        return None
    try:
        res = subprocess.run([str(exe), "--config", str(cfg), "-k", str(K), "--num_runs", str(runs), "--mode", mode, "--no_cpu"],
                             capture_output=True, text=True, timeout=600)
        name = "GPU-B200" if mode == "fp32" else f"GPU-B200-{mode}"
        rows = [ln.split(",") for ln in res.stdout.splitlines() if ln.startswith(name + ",")]
        csr = [r for r in rows if r[2] == "CSR"]
        if res.returncode not in (0, 3) or not csr:
            return {"error": (res.stderr or res.stdout)[-300:]}
        tot = float(np.median([int(r[7]) for r in csr])) * 1e-9
        return {"value": 2.0 * int(csr[0][6]) * K / tot / 1e9, "unit": "GFLOP/s", "ms_per_step": tot * 1e3,
                "init_ms": float(np.median([int(r[8]) for r in csr])) * 1e-6, "comp_ms": float(np.median([int(r[9]) for r in csr])) * 1e-6,
                "cleanup_ms": float(np.median([int(r[10]) for r in csr])) * 1e-6,
                "what": f"sddmm_bench: Competitors::GPUB200 ({mode}) init_csr + run_csr + cleanup_csr on pageable host containers, "
                        f"median of {len(csr)} runs, one GPU"}
    except Exception as ex:   # report, never hide
        return {"error": str(ex)}


# kernel-only table: every configuration BASELINE.json names, every storage mode, and the K sweep of the last one
PER_CONFIG = [(2, 32, "fp32_tc"), (2, 32, "tf32"), (2, 32, "bf16"), (2, 32, "fp32"), (3, 64, "fp32"), (4, 32, "fp32"), (4, 32, "bf16"),
              (5, 32, "fp32"), (5, 32, "bf16"), (5, 64, "fp32"), (5, 64, "bf16"), (5, 128, "fp32"), (5, 128, "bf16"),
              (5, 256, "fp32"), (5, 256, "bf16")]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--config", type=int, default=DEFAULT_CONFIG, choices=[1, 2, 3, 4, 5])
    ap.add_argument("--k", type=int, default=0)
    ap.add_argument("--mode", default="fp32_tc", choices=["fp32", "bf16", "tf32", "fp32_tc"],
                    help="fp32_tc (default): fp32-grade results, dense tiles on tcgen05 where S has them; fp32: FMA everywhere")
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload (profiling captures only)")
    ap.add_argument("--no-extra", action="store_true", help="skip the per-config table, the parity sample and the CPU baseline")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "engine" and args.scale == 1.0 else args.warmup

    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch  # device buffers for the L2 flush and the NCCL broadcast only
    from dphpc_b200 import Dataset, Engine, Pipeline, load_engine_lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SDDMM engine has no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def max_over_ranks(x):
        if dist is None:
            return float(x)
        tt = torch.tensor([float(x)], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    def sum_over_ranks(x):
        if dist is None:
            return float(x)
        tt = torch.tensor([float(x)], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.SUM)
        return float(tt.item())

    cfg, K = args.config, args.k or CONFIG_K[args.config]
    d = Dataset(cfg, K, args.scale)
    sh = shard_of(d, rank, world, args.mode)
    rp_local, Mloc, Nloc, nnz_loc, grid = sh["rp"], sh["M"], sh["N"], sh["nnz"], sh["grid"]
    if Mloc < 1:
        raise SystemExit(f"rank {rank}: empty row range; use fewer GPUs for this workload")

    lib = load_engine_lib()
    eng = Engine(local, args.mode)
    # pinned host copies of this rank's shard (the buffers a host caller would own)
    h_rp, _ = pinned_copy(lib, rp_local)
    h_ci, _ = pinned_copy(lib, sh["col"])
    h_sv, _ = pinned_copy(lib, sh["val"])
    h_A, _ = pinned_copy(lib, sh["A"])
    h_B, _ = pinned_copy(lib, sh["B"])
    h_P, p_view = pinned_copy(lib, np.zeros(max(nnz_loc, 1), np.float32))

    # ---- resident operands: B broadcast once over NCCL (N > 1), then a device-to-device upload
    if world > 1:
        tB = torch.empty((d.N, K), dtype=torch.float32, device="cuda")
        if rank == 0:
            tB.copy_(torch.from_numpy(np.ascontiguousarray(d.B)))
        dist.broadcast(tB, src=0)
        t_rp = torch.from_numpy(rp_local).cuda()
        t_ci = torch.from_numpy(np.ascontiguousarray(sh["col"])).cuda()
        t_sv = torch.from_numpy(np.ascontiguousarray(sh["val"])).cuda()
        t_A = torch.from_numpy(np.ascontiguousarray(sh["A"])).cuda()
        torch.cuda.synchronize()
        # (a column block takes its rows of the broadcast B: a contiguous piece of it)
        eng.upload_csr_device(Mloc, Nloc, K, nnz_loc, t_rp.data_ptr(), t_ci.data_ptr(), t_sv.data_ptr(), t_A.data_ptr(),
                              tB.data_ptr() + 4 * K * sh["c0"])
        del t_rp, t_ci, t_sv, t_A, tB
    else:
        eng.upload_csr_raw(Mloc, Nloc, K, h_rp, h_ci, h_sv, h_A, h_B)
    eng.nnz = nnz_loc
    plan = eng.plan()

    flush_buf = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")

    def flush():
        flush_buf.fill_(1)
        torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ---------------------------------------------------------------
    for _ in range(args.warmup):
        eng.run(); eng.sync()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    wall0 = time.perf_counter()
    step_ms, kern = [], {}
    for _ in range(args.steps):   # the timed steps: no instrumentation between the kernels
        flush()
        eng.run(); eng.sync()
        step_ms.append(eng.last_run_ms())
    barrier()
    wall = time.perf_counter() - wall0
    # a few more steps with an event pair around every kernel, for the roofline of the dominant kernel (not part of `value`)
    eng.set_kernel_timing(True)
    for _ in range(max(3, min(args.steps, 10))):
        flush()
        eng.run(); eng.sync()
        for name, ms in eng.kernel_times():
            kern.setdefault(name, []).append(ms)
    eng.set_kernel_timing(False)
    kern = {k: float(np.mean(v)) for k, v in kern.items()}
    # keep the GPU busy a little longer so the clock sampler sees it under load even for short runs
    t_end = time.perf_counter() + (0.6 if rank == 0 else 0.0)
    while time.perf_counter() < t_end:
        eng.run(); eng.sync()
    clocks = sampler.stop() if sampler else None
    t_local = float(np.sum(step_ms))
    t_total = max_over_ranks(t_local)
    ms_per_step = t_total / args.steps
    # per-rank shard size and time (how well the nnz-balanced row cuts balance the device time)
    per_rank = None
    if dist is not None:
        mine = torch.tensor([float(nnz_loc), t_local / args.steps], dtype=torch.float64, device="cuda")
        allr = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)   # (every rank takes part; only rank 0 prints)
        nnzs = [int(t[0].item()) for t in allr]
        mss = [float(t[1].item()) for t in allr]
        per_rank = {"nnz": nnzs, "ms_per_step": mss, "nnz_imbalance_max_over_mean": max(nnzs) / max(1e-30, sum(nnzs) / world),
                    "time_imbalance_max_over_mean": max(mss) / max(1e-30, sum(mss) / world)}
    flops = 2.0 * d.nnz * K
    value = flops / (ms_per_step * 1e-3) / 1e9

    # ---- parity of what was just timed: this rank's P shard against the CPU oracle (outside the timed region) ----
    parity = None
    if not args.no_extra:
        checked, worst = 0, float("inf")
        try:
            eng.run()
            p_shard = eng.download()
            checked, worst = parity_sample(p_shard, sh, K, args.mode)
            del p_shard
        except Exception as ex:  # report, never hide (the collectives below still run on every rank)
            sys.stderr.write(f"rank {rank}: parity check failed to run: {ex}\n")
        worst_all = max_over_ranks(worst if np.isfinite(worst) else 1e30)
        checked_all = sum_over_ranks(checked)
        parity = {"checked_nnz": int(checked_all), "max_err_over_bound": worst_all, "ok": bool(worst_all <= 1.0), "ranks": world,
                  "what": "per rank: 200 000 sampled nonzeros of its shard against a float64 dot product, first and last 2 000 rows "
                          "against the CPU oracle; err / (tol |s| sum_k |a b|), tol 1e-5 (fp32 modes) or 1e-2 (tf32, bf16); max over ranks"}

    # ---- end to end through the host-buffer API ---------------------------------------------
    e2e = None
    if not args.no_e2e:
        n_e2e = max(3, min(args.steps, 10))

        def timed(step, warm):
            for _ in range(warm):
                step()
            barrier()
            ts = []
            for _ in range(n_e2e):
                t0 = time.perf_counter()
                step()
                ts.append(time.perf_counter() - t0)
            return max_over_ranks(float(np.mean(ts)))

        def e2e_step():
            eng.upload_csr_raw(Mloc, Nloc, K, h_rp, h_ci, h_sv, h_A, h_B)
            eng.run()
            eng.download_raw(h_P)
        t_e2e = timed(e2e_step, 2)

        # the same step when the pattern stays (iterative callers): only A, B and S.val travel up, the plan is kept
        def reuse_step():
            eng.update_raw(h_A, h_B, h_sv)
            eng.run()
            eng.download_raw(h_P)
        t_reuse = timed(reuse_step, 1)
        # the one-call form of the same sequence: row chunks whose upload, plan + run and download overlap on the full-duplex host link
        pipe = Pipeline(local, args.mode, chunks=4)
        t_pipe = timed(lambda: pipe.sddmm_csr_raw(Mloc, Nloc, K, h_rp, h_ci, h_sv, h_A, h_B, h_P), 2)
        pipe_chunks = pipe.last_chunks()
        # ... and when the pattern stays: only the numbers travel, chunk by chunk
        t_pipe_reuse = timed(lambda: pipe.update_csr_raw(h_sv, h_A, h_B, h_P), 1)
        pipe.close()
        h2d = 4 * (Mloc + 1) + 8 * nnz_loc + 4 * K * (Mloc + Nloc)
        e2e = {"value": flops / t_pipe / 1e9, "unit": "GFLOP/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(4 * nnz_loc),
               "ms_per_step": t_pipe * 1e3, "steps": n_e2e, "chunks": pipe_chunks,
               "what": "sddmm_b200_pipeline_sddmm_csr: pinned host S, A, B -> HBM, device-side validation + plan, run, P.val -> pinned host, "
                       "in nnz-balanced row chunks whose three phases overlap; per rank bytes",
               "single_engine": {"value": flops / t_e2e / 1e9, "unit": "GFLOP/s", "ms_per_step": t_e2e * 1e3,
                                 "what": "upload_csr + run + download on one engine, one phase after the other"},
               "pattern_reuse": {"value": flops / t_pipe_reuse / 1e9, "unit": "GFLOP/s", "ms_per_step": t_pipe_reuse * 1e3,
                                 "h2d_bytes_per_step": int(4 * nnz_loc + 4 * K * (Mloc + Nloc)), "d2h_bytes_per_step": int(4 * nnz_loc),
                                 "what": "sddmm_b200_pipeline_update_csr (pinned host A, B, S.val -> HBM; pattern and plans kept; run; "
                                         "P.val -> pinned host; row chunks overlapped)",
                                 "single_engine": {"value": flops / t_reuse / 1e9, "unit": "GFLOP/s", "ms_per_step": t_reuse * 1e3,
                                                   "what": "update_dense + update_values + run + download on one engine"}}}
        # the consumer on the device-resident result: Y = P B is computed on the GPU and only Y comes back (no P.val download)
        try:
            h_Y, _ = pinned_copy(lib, np.zeros((Mloc, K), np.float32))

            def fused_step():
                eng.upload_csr_raw(Mloc, Nloc, K, h_rp, h_ci, h_sv, h_A, h_B)
                eng.run()
                eng.spmm_raw(K, 0, h_Y)
            t_fused = timed(fused_step, 1)
            e2e["fused"] = {"value": flops / t_fused / 1e9, "unit": "GFLOP/s (SDDMM flops only)", "ms_per_step": t_fused * 1e3,
                            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(4 * Mloc * K), "spmm_kernel_ms": eng.last_spmm_ms(),
                            "what": "upload_csr + run + sddmm_b200_spmm(X = B): Y = P B on the device, Y (M x K floats) -> pinned host instead of "
                                    "P.val (nnz floats)"}
            lib.sddmm_b200_host_free(h_Y)
        except Exception as ex:  # report, never hide
            e2e["fused"] = {"error": str(ex)}
        if rank == 0 and world == 1 and args.scale == 1.0 and not args.no_extra:
            e2e["competitor"] = competitor_e2e(cfg, K, args.mode)
        eng.nnz = nnz_loc

    # ---- roofline of the dominant kernel (this rank's shard) -------------------------------------
    peak, peak_src = hbm_peak()
    roofline = roofline_block(eng, plan, kern, args.mode, K, cfg, world, peak, peak_src)

    line = None
    if rank == 0:
        line = {
            "metric": "SDDMM GFLOP/s (2*nnz*K/t)", "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"fp32": "f32", "fp32_tc": "f32 (tf32x3 on dense tiles)", "tf32": "tf32", "bf16": "bf16"}[args.mode],
            "data": "synthetic", "config": workload_config(cfg, K, args.mode, world, grid),
            "e2e": e2e, "gpu_launches": int(args.steps * (plan["n_kernels"] + max(0, plan.get("rowseg_passes", 1) - 1))), "roofline": roofline, "clocks": clocks,
            "wall_s_timed_region": wall, "per_rank": per_rank, "parity": parity,
            "plan": {k: plan[k] for k in ("nnz", "rows_nonempty", "cols_touched", "max_row_nnz", "rowtile_nnz", "rowtile_items",
                                          "rowtile_rows_per_stage", "rowtile_grid", "rowtile_smem_bytes", "dense_nnz", "dense_tiles",
                                          "rowgroup_nnz", "rowgroup_rows", "rowseg_nnz", "rowseg_units", "rowseg_panels", "rowseg_grid",
                                          "n_kernels")},
        }
        line["hbm_gb_per_s_algorithmic"] = eng.algorithmic_bytes() / (float(np.mean(step_ms)) * 1e-3) / 1e9

    # ---- CPU baseline (rank 0 at N = 1) ----------------------------------------------------------------
    if rank == 0 and world == 1 and not args.no_extra and args.scale == 1.0:
        base, _, _ = cpu_reference(d.M, d.N, K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, max_nnz=int(8e8 / K), reps=3)
        line["cpu_baseline"] = base

    # ---- every other configuration / mode and the K sweep, kernel only, on the same kind of row shards -----------------
    if not args.no_extra and args.scale == 1.0:
        per = {}
        cache = {}   # (config, K) -> dataset; generated once, shared by the modes
        for c, k_c, m in PER_CONFIG:
            key = f"config{c}_k{k_c}_{m}"
            ms_local, alg_local, nnz_c, plan_c, kern_c, e2 = 1e30, 0.0, 0, None, {}, None
            try:
                if (c, k_c) not in cache:
                    for dd_old in cache.values():
                        if dd_old is not d:
                            dd_old.close()
                    cache.clear()
                    cache[(c, k_c)] = d if (c, k_c) == (cfg, K) else Dataset(c, k_c, 1.0)
                dd = cache[(c, k_c)]
                nnz_c = int(dd.nnz)
                s2 = shard_of(dd, rank, world, m)
                if s2["M"] > 0 and s2["nnz"] > 0:
                    e2 = Engine(local, m)
                    e2.upload_csr(s2["M"], s2["N"], dd.K, s2["rp"], s2["col"], s2["val"], s2["A"], s2["B"])
                else:
                    ms_local = 0.0
            except Exception as ex:  # report, never hide (the collectives below still run on every rank)
                sys.stderr.write(f"rank {rank}: {key}: {ex}\n")
                if e2 is not None:
                    e2.close()
                e2, ms_local = None, 1e30
            # every rank has generated and uploaded before any rank times: a rank still generating its dataset on all host
            # cores would delay the launches of the ranks that already time (the event pair spans the launches of a step)
            barrier()
            try:
                if e2 is not None:
                    ms_local, kern_c = kernel_only_stats(e2, 10, 3, flush)
                    alg_local, plan_c = float(e2.algorithmic_bytes()), e2.plan()
            except Exception as ex:
                sys.stderr.write(f"rank {rank}: {key}: {ex}\n")
                ms_local = 1e30
            finally:
                if e2 is not None:
                    e2.close()
            barrier()
            ms = max_over_ranks(ms_local)
            alg = sum_over_ranks(alg_local)
            if rank == 0:
                if ms >= 1e29 or ms <= 0:
                    per[key] = {"error": "a rank failed (see stderr)"}
                else:
                    per[key] = {"ms": ms, "gflops": 2.0 * nnz_c * k_c / ms / 1e6, "gb_per_s": alg / ms / 1e6, "hbm_frac": alg / ms / 1e6 / (peak * world),
                                "kernels_ms_rank0": kern_c, "kernel": dominant_kernel(kern_c, plan_c) if plan_c else None,
                                "what": f"{world} block(s) (nnz-balanced row ranges, column ranges where B is far larger than L2), max over ranks; fraction = algorithmic bytes of all blocks / time / "
                                        f"({world} x HBM peak)"}
        for dd_old in cache.values():
            if dd_old is not d:
                dd_old.close()
        if rank == 0:
            line["per_config"] = per

    if rank == 0:
        print(json.dumps(line), flush=True)
    eng.close()
    for p in (h_rp, h_ci, h_sv, h_A, h_B, h_P):
        lib.sddmm_b200_host_free(p)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
