"""Generate tests/golden/sddmm_golden.json from the reference itself.

    python tests/golden/make_golden.py          (needs oracle/_ref, i.e. the reference checkout)

Every expected value in the fixture comes from the reference's own CPUBasic /
CSR / COO code (compiled unmodified by oracle/build.py into
oracle/_ref/libsddmm_ref.so).  Inputs of the tiny cases are the literals of the
reference's tests/matrix_test.cc:124-182 (sddmm_coo1..4) and of DummyDataset
(src/benchmark/dataset.hpp:183-204); the reference file holds no expected
values for them, they follow from running its CPU-Basic competitor.
Floats are stored as hex bit patterns so the comparison is bit exact.
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle"))

import oracle_lib  # noqa: E402
from dphpc_b200 import Dataset  # noqa: E402


def bits(a):
    return [int(x) for x in np.asarray(a, np.float32).view(np.uint32)]


TINY = {
    # name: (A, B, triplets (row, col, val), M, N)
    "sddmm_coo1": ([[1, 2], [3, 4]], [[-1, 2], [-3, 4]], [(0, 0, 1), (0, 1, 1), (1, 0, 1), (1, 1, 1)], 2, 2),
    "sddmm_coo2": ([[1, 2, 3], [4, 5, 6]], [[-1, -3, 5], [2, 4, -6]], [(0, 0, 1), (1, 0, 1), (1, 1, 1)], 2, 2),
    "sddmm_coo3": ([[1, 2, 3], [4, 5, 6]], [[-1, -3, 5]], [(0, 0, 1), (1, 0, -1)], 2, 2),
    "sddmm_coo4": ([[1, 2], [3, 4], [5, 6]], [[-1, -3], [2, 2], [3, 1]], [(0, 0, 1), (1, 0, -1), (2, 0, 1), (2, 2, 1)], 3, 3),
    "dummy_dataset": ([[1, 1], [1, 1]], [[1, 1], [1, 1]], [(0, 0, 1), (0, 1, 1), (1, 0, 1), (1, 1, 1)], 2, 2),
}


def main():
    ref = oracle_lib.Reference.try_load()
    if ref is None:
        raise SystemExit("oracle/_ref/libsddmm_ref.so missing: run `python oracle/build.py` with the reference present")
    out = {"tiny": {}, "random": {}, "configs": {}, "dispatch": {}}

    for name, (A, B, trip, M, N) in TINY.items():
        A = np.array(A, np.float32)
        B = np.array(B, np.float32)
        K = A.shape[1]
        r = np.array([t[0] for t in trip], np.int32)
        c = np.array([t[1] for t in trip], np.int32)
        v = np.array([t[2] for t in trip], np.float32)
        rp, ci, sv = ref.csr_from_triplets(M, N, r, c, v)
        cr, cc, cv = ref.coo_from_triplets(M, N, r, c, v)
        # B of sddmm_coo3 has one row although S is declared 2x2: only column 0 is referenced
        p_csr = ref.cpu_basic_csr(M, B.shape[0], K, rp, ci, sv, A, B)
        p_coo = ref.cpu_basic_coo(M, B.shape[0], K, cr, cc, cv, A, B)
        out["tiny"][name] = {
            "M": M, "N": N, "K": K, "A": A.tolist(), "B": B.tolist(),
            "triplets": [[int(a), int(b), float(x)] for a, b, x in trip],
            "row_ptr": rp.tolist(), "col_idx": ci.tolist(), "s_val": sv.tolist(),
            "coo_rows": cr.tolist(), "coo_cols": cc.tolist(),
            "p_csr": p_csr.tolist(), "p_coo": p_coo.tolist(),
        }

    # unsorted triplets with an empty row and K not a multiple of 4: full values, bit exact
    rng = np.random.default_rng(20231004)
    for name, (M, N, K, n) in {"rand_37x29_k5": (37, 29, 5, 300), "rand_64x48_k32": (64, 48, 32, 700),
                               "rand_50x70_k33": (50, 70, 33, 500)}.items():
        cells = rng.choice(M * N, size=n, replace=False)
        r, c = (cells // N).astype(np.int32), (cells % N).astype(np.int32)
        keep = r != 3  # row 3 stays empty
        r, c = r[keep], c[keep]
        v = rng.random(r.size, dtype=np.float32)
        A = (rng.random((M, K), dtype=np.float32) * 2 - 1).astype(np.float32)
        B = (rng.random((N, K), dtype=np.float32) * 2 - 1).astype(np.float32)
        rp, ci, sv = ref.csr_from_triplets(M, N, r, c, v)
        p = ref.cpu_basic_csr(M, N, K, rp, ci, sv, A, B)
        out["random"][name] = {
            "M": M, "N": N, "K": K, "trip_rows": r.tolist(), "trip_cols": c.tolist(), "trip_vals_bits": bits(v),
            "A_bits": bits(A.ravel()), "B_bits": bits(B.ravel()),
            "row_ptr": rp.tolist(), "col_idx": ci.tolist(), "s_val_bits": bits(sv), "p_bits": bits(p),
        }

    # the five synthetic configurations at a CPU-sized scale: digest of the inputs and of the reference's output
    for cfg, scale, K in ((1, 1.0, 32), (2, 0.05, 32), (3, 0.004, 64), (4, 0.002, 32), (5, 0.003, 32), (5, 0.002, 128)):
        d = Dataset(cfg, K, scale)
        p = ref.cpu_basic_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        key = f"config{cfg}_scale{scale}_k{K}"
        out["configs"][key] = {
            "config": cfg, "scale": scale, "K": K, "seed": d.seed, "M": d.M, "N": d.N, "nnz": d.nnz,
            "pattern_sha256": hashlib.sha256(d.row_ptr.tobytes() + d.col_idx.tobytes()).hexdigest(),
            "inputs_sha256": hashlib.sha256(d.s_val.tobytes() + d.A.tobytes() + d.B.tobytes()).hexdigest(),
            "p_sha256": hashlib.sha256(p.tobytes()).hexdigest(),
            "p_head_bits": bits(p[:8]),
            "p_sum_f64": float(p.astype(np.float64).sum()),
        }
        d.close()

    # dispatcher: literals of tests/matrix_test.cc:354-425, 460-477 re-derived by the reference code
    def diag(n):
        return np.arange(n + 1, dtype=np.int32), np.arange(n, dtype=np.int32)

    cases = {
        "more_threads_than_rows": (2, 2, [0, 2, 4], [0, 1, 0, 1], 4, False),
        "equal_threads": (2, 2, [0, 2, 4], [0, 1, 0, 1], 2, False),
        "less_threads": (4, 2, [0, 1, 2, 3, 4], [0, 0, 1, 1], 2, False),
        "empty_rows": (4, 2, [0, 0, 1, 1, 1], [0], 2, False),
        "tensor_diag64": (64, 64, diag(64)[0].tolist(), diag(64)[1].tolist(), 4, True),
        "diag_1500_half": (1500, 1500, diag(1500)[0].tolist(), diag(1500)[1].tolist(), 750, False),
    }
    for name, (M, N, rp, ci, parts, tensor) in cases.items():
        s = ref.dispatch(M, N, np.array(rp, np.int32), np.array(ci, np.int32), parts, tensor)
        out["dispatch"][name] = {"M": M, "N": N, "row_ptr": rp if M <= 64 else "diag", "col_idx": ci if M <= 64 else "diag",
                                 "parts": parts, "tensor": tensor, "start_idx": s.tolist() if M <= 64 else "2*i",
                                 "start_idx_sha256": hashlib.sha256(s.astype(np.int32).tobytes()).hexdigest()}

    (HERE / "sddmm_golden.json").write_text(json.dumps(out, indent=0, separators=(",", ":")))
    print("wrote", HERE / "sddmm_golden.json", (HERE / "sddmm_golden.json").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
