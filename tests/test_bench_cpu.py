"""CPU-side checks of bench.py: the reference arm's JSON line and the row-sharded CPU baseline (no GPU needed)."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def test_reference_arm_prints_the_contract_line():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--config", "1", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GFLOP/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["steps"] == 2 and line["warmup"] == 1
    assert line["config"]["config_id"] == 1 and line["config"]["mode"] == "fp32_tc"     # the GPU arm's default workload description
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_row_sharded_cpu_baseline_covers_every_nonzero_once(oracle):
    import bench

    rng = np.random.default_rng(3)
    M, N, K = 400, 300, 8
    lens = rng.integers(0, 30, M)
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(N, size=int(n), replace=False)) for n in lens]).astype(np.int32)
    sv = rng.random(len(ci), dtype=np.float32)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (N, K)).astype(np.float32)
    for threads in (1, 3, 8):
        shards = bench.CpuRowShards(M, N, K, rp, ci, sv, A, B, M, threads)
        try:
            assert shards.nnz == len(ci) and 1 <= shards.threads <= threads
            assert shards.ranges[0][0] == 0 and shards.ranges[-1][1] == M
            assert all(a[1] == b[0] for a, b in zip(shards.ranges[:-1], shards.ranges[1:]))   # contiguous, no overlap
            assert shards.step() > 0
        finally:
            shards.close()


def test_roofline_script_reads_the_driver_csv(tmp_path):
    # the corrected-constants roofline table over the benchmark driver's CSV schema (plot only where matplotlib exists)
    csv = tmp_path / "runs.csv"
    csv.write_text("competitor,dataset,mat_repr,M,N,K,NZ,total_ns,init_ns,comp_ns,cleanup_ns,correctness,num_thread_blocks,num_threads_per_block\n"
                   "GPU-B200,cfg,CSR,1000,1000,32,50000,900000,500000,100000,300000,1,10,256\n"
                   "GPU-B200,cfg,CSR,1000,1000,32,50000,900000,500000,300000,300000,1,10,256\n"
                   "GPU-B200,cfg,CSR,1000,1000,32,50000,900000,500000,200000,300000,0,10,256\n")
    res = subprocess.run([sys.executable, str(ROOT / "dphpc_b200" / "plots" / "plot_roofline.py"), str(csv), "--hbm-gbs", "1000",
                          "--out", str(tmp_path / "r.png")], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stderr[-2000:]
    rows = [ln.split(",") for ln in res.stdout.splitlines() if ln.startswith("GPU-B200")]
    assert len(rows) == 1
    flops, nbytes, secs = 2 * 32 * 50000 + 50000, 4 * 32 * 2000 + 12 * 50000 + 4 * 1001, 200000e-9   # median of the two correct runs
    assert abs(float(rows[0][4]) - flops / nbytes) < 1e-4 * flops / nbytes
    assert abs(float(rows[0][5]) - flops / secs) < 1e-4 * flops / secs
    assert abs(float(rows[0][7]) - (nbytes / secs) / 1e12) < 1e-4      # fraction of the 1000 GB/s roof
