#!/usr/bin/env python
"""Roofline of SDDMM runs on a B200 from the benchmark driver's CSV.

    dphpc_b200/sddmm_bench --config 5 > runs.csv
    python dphpc_b200/plots/plot_roofline.py runs.csv [--out roofline.png] [--hbm-gbs 6557] [--field comp_ns]

Reads the CSV schema the reference's driver and `sddmm_bench` both print
(competitor,dataset,mat_repr,M,N,K,NZ,total_ns,init_ns,comp_ns,cleanup_ns,correctness,...) and, per
(competitor, dataset, representation, K), prints operational intensity, achieved FLOP/s, achieved GB/s and the
fraction of the memory roof; with matplotlib installed it also draws the log-log roofline.

Same model as the reference's plots/plot_roofline.py with its constants put right:
  * unit prefixes: the reference writes 10e12 for "tera" and divides nanoseconds by 10e9 (plots/plot_roofline.py:19-20,
    :93) -- both a factor 10 off, which cancel in the achieved/peak ratio but put every point and both roofs a decade
    too high; here tera = 1e12 and ns -> s is 1e-9;
  * flops = 2 K NZ (+ NZ for the final scaling, as plots/plot_roofline.py:29);
  * bytes: the reference counts (M K + N K) 4 + 4 NZ -- dense operands plus S.val -- and leaves out col_idx, the
    P.val store and row_ptr (plots/plot_roofline.py:30); here bytes = e K (M + N) + 12 NZ + 4 (M + 1) with e = 4, or 2
    for the competitors whose name ends in -bf16 (bf16 storage of A and B);
  * roofs: the B200's measured copy bandwidth (MEASURED_PEAKS.json beside the repository root when present, else
    --hbm-gbs, else 6650 GB/s) and its fp32 FMA peak, 148 SMs x 128 lanes x 2 x 1.965 GHz = 74.4 TFLOP/s.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import pandas as pd

ROOT = Path(__file__).resolve().parent.parent.parent
FP32_PEAK_FLOPS = 148 * 128 * 2 * 1.965e9
FALLBACK_HBM_GBS = 6650.0


def hbm_bytes_per_s(arg):
    if arg:
        return float(arg) * 1e9, "--hbm-gbs"
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]) * 1e9, "measured copy bandwidth (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS * 1e9, "fallback 6650 GB/s"


def table(df: pd.DataFrame, field: str, percentile: float, beta: float) -> pd.DataFrame:
    df = df[df["correctness"].astype(int) == 1].copy() if "correctness" in df else df.copy()
    e = df["competitor"].astype(str).str.endswith("-bf16").map({True: 2, False: 4})
    df["flops"] = 2.0 * df["K"] * df["NZ"] + df["NZ"]
    df["bytes"] = e * df["K"] * (df["M"] + df["N"]) + 12.0 * df["NZ"] + 4.0 * (df["M"] + 1)
    df["seconds"] = df[field] * 1e-9
    g = df.groupby(["competitor", "dataset", "mat_repr", "K"], as_index=False).agg(
        seconds=("seconds", lambda s: s.quantile(percentile)), flops=("flops", "first"), bytes=("bytes", "first"))
    g["op_intensity"] = g["flops"] / g["bytes"]
    g["flops_per_s"] = g["flops"] / g["seconds"]
    g["gb_per_s"] = g["bytes"] / g["seconds"] / 1e9
    g["roof_flops_per_s"] = (g["op_intensity"] * beta).clip(upper=FP32_PEAK_FLOPS)
    g["frac_of_roof"] = g["flops_per_s"] / g["roof_flops_per_s"]
    return g


def draw(g: pd.DataFrame, beta: float, out: str, what: str) -> bool:
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        return False
    fig, ax = plt.subplots(figsize=(10, 8))
    ridge = FP32_PEAK_FLOPS / beta
    xs = [0.05, ridge, 500.0]
    ax.plot(xs, [beta * xs[0], FP32_PEAK_FLOPS, FP32_PEAK_FLOPS], color="black")
    ax.axvline(ridge, color="black", alpha=0.4, ls="--")
    for (comp, rep), part in g.groupby(["competitor", "mat_repr"]):
        ax.scatter(part["op_intensity"], part["flops_per_s"], s=60, label=f"{comp} - {rep}")
        for _, r in part.iterrows():
            ax.annotate(f"{r['dataset']} K={int(r['K'])}", (r["op_intensity"], r["flops_per_s"]), fontsize=7)
    ax.set_xscale("log"); ax.set_yscale("log")
    ax.set_xlabel("Operational intensity [flop / byte]"); ax.set_ylabel("Performance [flop / s]")
    ax.set_title(f"SDDMM roofline, NVIDIA B200 ({what}; fp32 FMA peak {FP32_PEAK_FLOPS / 1e12:.1f} TFLOP/s)")
    ax.legend(fontsize=8)
    fig.savefig(out, dpi=150, bbox_inches="tight")
    return True


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("csv")
    ap.add_argument("--out", default="roofline_b200.png")
    ap.add_argument("--field", default="comp_ns", choices=["total_ns", "init_ns", "comp_ns", "cleanup_ns"])
    ap.add_argument("--percentile", type=float, default=0.5)
    ap.add_argument("--hbm-gbs", default=None)
    args = ap.parse_args()
    beta, what = hbm_bytes_per_s(args.hbm_gbs)
    df = pd.read_csv(args.csv, comment="#")
    df = df[pd.to_numeric(df["NZ"], errors="coerce").notna()]   # (a concatenation of runs repeats the header line)
    for c in ("M", "N", "K", "NZ", "total_ns", "init_ns", "comp_ns", "cleanup_ns", "correctness"):
        df[c] = pd.to_numeric(df[c])
    g = table(df, args.field, args.percentile, beta)
    cols = ["competitor", "dataset", "mat_repr", "K", "op_intensity", "flops_per_s", "gb_per_s", "frac_of_roof"]
    print(f"# memory roof: {beta / 1e9:.1f} GB/s ({what}); compute roof: {FP32_PEAK_FLOPS / 1e12:.1f} TFLOP/s fp32")
    print(g[cols].to_csv(index=False, float_format="%.6g"), end="")
    if draw(g, beta, args.out, what):
        print(f"# wrote {args.out}")
    else:
        print("# matplotlib is not installed: table only")


if __name__ == "__main__":
    main()
