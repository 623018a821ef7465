"""Parity of the CUDA engine (through the C ABI) against the CPU oracle.  Needs a B200.

Bar: pattern untouched (the engine returns values in the order of the uploaded col_idx), values within
  |p - p_ref| <= tol * |s_ij| * sum_k |a_ik b_jk|
with tol = 1e-5 for the fp32 modes and 1e-2 for tf32 / bf16 -- "rel 1e-5 / 1e-2" made robust to the
cancellation that A, B in [-1, 1) produce.  p_ref is the oracle restating the reference's CPUBasic.
"""
import json
from pathlib import Path

import numpy as np
import pytest

import oracle_lib
from dphpc_b200 import Dataset, Engine, Pipeline, SddmmError

pytestmark = pytest.mark.gpu

GOLD = json.loads((Path(__file__).parent / "golden" / "sddmm_golden.json").read_text())
TOL = {"fp32": 1e-5, "fp32_tc": 1e-5, "tf32": 1e-2, "bf16": 1e-2}
MODES = ["fp32", "bf16", "tf32", "fp32_tc"]


@pytest.fixture(scope="module")
def engines():
    es = {m: Engine(0, m) for m in MODES}
    yield es
    for e in es.values():
        e.close()


def check(engine, mode, oracle, M, N, K, rp, ci, sv, A, B, coo=False, what=""):
    rp, ci = np.ascontiguousarray(rp, np.int32), np.ascontiguousarray(ci, np.int32)
    sv = np.ascontiguousarray(sv, np.float32)
    A, B = np.ascontiguousarray(A, np.float32), np.ascontiguousarray(B, np.float32)
    rows = oracle.coo_rows(M, rp)
    if coo:
        p = engine.sddmm_coo(M, N, K, rows, ci, sv, A, B)
    else:
        p = engine.sddmm_csr(M, N, K, rp, ci, sv, A, B)
    p_ref = oracle.sddmm_csr(M, K, rp, ci, sv, A, B)
    bound = oracle_lib.abs_dot_bound(rows, ci, sv, A, B)
    oracle_lib.assert_values_close(p, p_ref, bound, TOL[mode], what or f"{mode} {M}x{N} K={K}")
    return p


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", sorted(GOLD["tiny"]))
def test_tiny_golden_cases(engines, oracle, mode, name):
    # sddmm_coo1..4 and DummyDataset: K = 2 or 3 -> scalar path; bf16 storage cannot take K % 4 != 0
    g = GOLD["tiny"][name]
    A, B = np.array(g["A"], np.float32), np.array(g["B"], np.float32)
    e = engines[mode]
    if mode == "bf16":
        with pytest.raises(SddmmError) as ei:
            e.sddmm_csr(g["M"], B.shape[0], g["K"], g["row_ptr"], g["col_idx"], g["s_val"], A, B)
        assert ei.value.code == 6
        return
    p = e.sddmm_csr(g["M"], B.shape[0], g["K"], g["row_ptr"], g["col_idx"], g["s_val"], A, B)
    assert p.tolist() == g["p_csr"]  # small integers: exact in every summation order
    p = e.sddmm_coo(g["M"], B.shape[0], g["K"], g["coo_rows"], g["coo_cols"], g["s_val"], A, B)
    assert p.tolist() == g["p_coo"]


@pytest.mark.parametrize("mode", ["fp32", "fp32_tc"])
@pytest.mark.parametrize("name", sorted(GOLD["random"]))
def test_random_golden_cases(engines, oracle, mode, name):
    g = GOLD["random"][name]
    f = lambda b: np.array(b, np.uint32).view(np.float32)  # noqa: E731
    A, B = f(g["A_bits"]).reshape(g["M"], g["K"]), f(g["B_bits"]).reshape(g["N"], g["K"])
    p = check(engines[mode], mode, oracle, g["M"], g["N"], g["K"], g["row_ptr"], g["col_idx"], f(g["s_val_bits"]), A, B)
    # and directly against the reference's stored output
    rows = oracle.coo_rows(g["M"], np.array(g["row_ptr"], np.int32))
    bound = oracle_lib.abs_dot_bound(rows, np.array(g["col_idx"]), f(g["s_val_bits"]), A, B)
    oracle_lib.assert_values_close(p, f(g["p_bits"]), bound, 1e-5, name)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("cfg,scale,K", [(1, 1.0, 32), (2, 0.05, 32), (2, 0.12, 32), (3, 0.004, 64), (4, 0.002, 32),
                                         (4, 0.02, 32), (5, 0.003, 32), (5, 0.002, 128), (5, 0.002, 64), (5, 0.001, 256)])
def test_synthetic_configs_small(engines, oracle, mode, cfg, scale, K):
    d = Dataset(cfg, K, scale)
    check(engines[mode], mode, oracle, d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, what=f"{mode} cfg{cfg} K={K}")
    check(engines[mode], mode, oracle, d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, coo=True,
          what=f"{mode} cfg{cfg} K={K} coo")


def test_config2_unaligned_blocks(engines, oracle):
    # 64x64 blocks at arbitrary offsets: the tile detector anchors its tiles on the blocks, not on the 64-grid
    d = Dataset(2, 32, 0.1, variant=1)
    for mode in ("fp32", "fp32_tc", "tf32", "bf16"):
        check(engines[mode], mode, oracle, d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, what=f"{mode} unaligned")
        plan = engines[mode].plan()
        if mode != "fp32":
            assert plan["dense_nnz"] >= 0.6 * d.nnz, f"{mode}: only {plan['dense_nnz']} of {d.nnz} nonzeros on the tensor path"
            assert plan["dense_nnz"] + plan["rowseg_nnz"] + plan["rowtile_nnz"] == d.nnz
        check(engines[mode], mode, oracle, d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, coo=True, what=f"{mode} unaligned coo")
    # the grid-only detection on the same input catches far less, and gives the same values
    with Engine(0, "fp32_tc") as e:
        e.set_knob("offset_tiles", 0)
        q = check(e, "fp32_tc", oracle, d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, what="grid tiles only")
        assert e.plan()["dense_nnz"] < engines["fp32_tc"].plan()["dense_nnz"]
    d.close()


def test_overlapping_dense_blocks_have_one_owner_per_nonzero(engines, oracle):
    # two dense 64x64 blocks that overlap in rows and columns, a third stacked right below the first, one at the matrix
    # corner (its window reaches past the last row and column): every nonzero is computed exactly once
    rng = np.random.default_rng(21)
    M = N = 400
    dense = np.zeros((M, N), bool)
    for r0, c0 in ((10, 20), (40, 50), (74, 20), (350, 350), (200, 100), (200, 164)):
        dense[r0:r0 + 64, c0:c0 + 64] |= rng.random((min(64, M - r0), min(64, N - c0))) < 0.8
    dense |= rng.random((M, N)) < 0.01      # thin background
    rows, cols = np.nonzero(dense)
    rp = np.concatenate([[0], np.cumsum(np.bincount(rows, minlength=M))]).astype(np.int32)
    ci = cols.astype(np.int32)
    sv = rng.uniform(-1, 1, ci.size).astype(np.float32)
    A = rng.uniform(-1, 1, (M, 64)).astype(np.float32)
    B = rng.uniform(-1, 1, (N, 64)).astype(np.float32)
    for mode in ("fp32_tc", "tf32", "bf16"):
        e = Engine(0, mode)
        e.set_knob("offset_tiles", 1)
        p = check(e, mode, oracle, M, N, 64, rp, ci, sv, A, B, what=f"overlapping blocks {mode}")
        plan = e.plan()
        assert plan["dense_tiles"] >= 4 and plan["dense_nnz"] + plan["rowseg_nnz"] + plan["rowtile_nnz"] == ci.size
        # the same input with the residual on the row-tile kernel (flag: no row segments)
        e2 = Engine(0, mode, flags=4)
        e2.set_knob("offset_tiles", 1)
        q = check(e2, mode, oracle, M, N, 64, rp, ci, sv, A, B, what=f"overlapping blocks {mode}, row-tile residual")
        assert e2.plan()["rowseg_units"] == 0 and [n for n, _ in e2.kernel_times()][-1] == "sddmm_rowtile_kernel"
        e2.close()
        e.run()
        assert np.array_equal(e.download(), p)   # same plan, same owners: bit-identical on a second run
        e.close()


@pytest.mark.parametrize("K", [1, 2, 3, 4, 8, 12, 20, 31, 32, 33, 36, 64, 96, 100, 128, 160, 256, 260])
def test_any_k(engines, oracle, K):
    # the reference's kernels need K % 8 == 0 or K % 32 == 0 (src/competitors/gpu/gpu_basic.cu:77-80,
    # gpu_shared.cu:98-101); the engine takes any K >= 1
    d = Dataset(uniform=(301, 257, 6000), K=K, seed=K)
    check(engines["fp32"], "fp32", oracle, d.M, d.N, K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    if K % 8 == 0 and K <= 256:
        check(engines["bf16"], "bf16", oracle, d.M, d.N, K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)


@pytest.mark.parametrize("M,N,K,density", [(500, 500, 32, 0.3), (250, 250, 32, 0.7), (10000, 10000, 32, 0.001)])
def test_reference_random_suite(engines, oracle, M, N, K, density):
    # sddmm_random_coo / _dense_coo / _sparse_coo / sddmm_csr_coo (tests/matrix_test.cc:184-246)
    d = Dataset(uniform=(M, N, int(M * N * density)), K=K, seed=M)
    for mode in MODES:
        p_csr = check(engines[mode], mode, oracle, M, N, K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        p_coo = check(engines[mode], mode, oracle, M, N, K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, coo=True)
        assert np.array_equal(p_csr, p_coo)  # COO(P_csr) == P_coo, bit for bit


def test_edge_shapes(engines, oracle):
    e = engines["fp32"]
    rng = np.random.default_rng(5)

    def dense(m, k):
        return (rng.random((m, k), dtype=np.float32) * 2 - 1).astype(np.float32)

    # a single 50 000-nnz row next to empty rows; M = 1; N = 1; fully dense 66x66; diagonal; non-square
    N = 60000
    cols = np.sort(rng.choice(N, 50000, replace=False)).astype(np.int32)
    rp = np.array([0, 0, 50000, 50000, 50000], np.int32)
    check(e, "fp32", oracle, 4, N, 32, rp, cols, rng.random(50000, dtype=np.float32), dense(4, 32), dense(N, 32), what="one long row")
    check(e, "fp32", oracle, 1, 7, 8, [0, 3], [0, 2, 6], [1, 2, 3], dense(1, 8), dense(7, 8), what="M=1")
    check(e, "fp32", oracle, 5, 1, 4, [0, 1, 1, 2, 3, 3], [0, 0, 0], [1, 2, 3], dense(5, 4), dense(1, 4), what="N=1")
    rp = (np.arange(67) * 66).astype(np.int32)
    ci = np.tile(np.arange(66, dtype=np.int32), 66)
    for mode in MODES:
        check(engines[mode], mode, oracle, 66, 66, 32, rp, ci, rng.random(66 * 66, dtype=np.float32), dense(66, 32), dense(66, 32),
              what=f"{mode} dense 66x66")
    n = 3000
    check(e, "fp32", oracle, n, n, 32, np.arange(n + 1), rng.permutation(n), rng.random(n, dtype=np.float32), dense(n, 32),
          dense(n, 32), what="latin")
    d = Dataset(uniform=(4562 // 4, 5761 // 4, 40000), K=32, seed=9)
    check(e, "fp32", oracle, d.M, d.N, 32, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, what="non-square")
    # trailing empty rows and an empty first row
    check(e, "fp32", oracle, 6, 9, 16, [0, 0, 2, 2, 5, 5, 5], [1, 8, 0, 3, 4], [1, 1, 1, 1, 1], dense(6, 16), dense(9, 16), what="empty rows")


def test_empty_matrix(engines):
    e = engines["fp32"]
    p = e.sddmm_csr(3, 3, 4, [0, 0, 0, 0], np.zeros(0, np.int32), np.zeros(0, np.float32), np.ones((3, 4)), np.ones((3, 4)))
    assert p.size == 0
    assert e.plan()["n_kernels"] == 0


def test_stale_output_is_overwritten(engines, oracle):
    # the reference's test helper reuses one P object that still holds S's values (tests/matrix_test.cc:66-67)
    d = Dataset(1, 32, 1.0)
    e = engines["fp32"]
    e.upload_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    out = np.full(d.nnz, 123.0, np.float32)
    e.run()
    e.download(out)
    assert np.array_equal(out, e.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B))


def test_bad_inputs_are_rejected(engines):
    e = engines["fp32"]
    A = np.ones((3, 4), np.float32)
    with pytest.raises(SddmmError) as ei:
        e.sddmm_csr(3, 3, 4, [0, 2, 1, 3], [0, 1, 2], [1, 1, 1], A, A)  # row_ptr decreases
    assert ei.value.code == 2
    with pytest.raises(SddmmError) as ei:
        e.sddmm_csr(3, 3, 4, [0, 1, 2, 3], [0, 3, 2], [1, 1, 1], A, A)  # column out of range
    assert ei.value.code == 2
    with pytest.raises(SddmmError) as ei:
        e.sddmm_coo(3, 3, 4, [1, 0, 2], [0, 1, 2], [1, 1, 1], A, A)  # COO rows not sorted
    assert ei.value.code == 2
    with pytest.raises(SddmmError) as ei:
        e.upload_csr(3, 3, 0, [0, 1, 2, 3], [0, 1, 2], [1, 1, 1], np.zeros((3, 0)), np.zeros((3, 0)))
    assert ei.value.code == 1
    # the engine is still usable afterwards
    assert e.sddmm_csr(3, 3, 4, [0, 1, 2, 3], [0, 1, 2], [1, 1, 1], A, A).tolist() == [4.0, 4.0, 4.0]
    fresh = Engine(0, "fp32")
    with pytest.raises(SddmmError) as ei:
        fresh.run()
    assert ei.value.code == 5
    fresh.close()


def test_plan_reports_histogram_and_counts(engines):
    d = Dataset(4, 32, 0.01)
    e = engines["fp32"]
    e.upload_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    p = e.plan()
    lens = np.diff(d.row_ptr)
    assert p["rows_nonempty"] == int((lens > 0).sum())
    assert p["cols_touched"] == np.unique(d.col_idx).size
    assert p["max_row_nnz"] == int(lens.max())
    hist = np.zeros(20, np.int64)
    for L in lens:
        hist[min(19, int(L).bit_length())] += 1
    assert p["row_len_hist"] == hist.tolist()
    assert p["cols_sorted"] == 1
    assert e.flops() == 2 * d.nnz * d.K
    assert e.algorithmic_bytes() == 4 * d.K * (p["rows_nonempty"] + p["cols_touched"]) + 12 * d.nnz + 4 * (d.M + 1)


def test_unsorted_columns_inside_rows(engines, oracle):
    # not something the reference's containers produce, but nothing in the math needs sorted columns
    d = Dataset(uniform=(200, 300, 5000), K=32, seed=2)
    ci = d.col_idx.copy()
    rng = np.random.default_rng(0)
    for i in range(d.M):
        a, b = d.row_ptr[i], d.row_ptr[i + 1]
        ci[a:b] = rng.permutation(ci[a:b])
    for mode in ("fp32", "fp32_tc"):
        engines[mode].upload_csr(d.M, d.N, d.K, d.row_ptr, ci, d.s_val, d.A, d.B)
        assert engines[mode].plan()["cols_sorted"] == 0
        check(engines[mode], mode, oracle, d.M, d.N, d.K, d.row_ptr, ci, d.s_val, d.A, d.B, what="unsorted")


def test_update_values_and_dense_keep_the_plan(engines, oracle):
    d = Dataset(5, 32, 0.003)
    e = engines["fp32"]
    p1 = e.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    e.update_values(d.s_val * 2)
    e.run()
    assert np.array_equal(e.download(), p1 * 2)  # scaling by 2 is exact: linearity in S
    e.update_dense(A=d.A * 0.5)
    e.run()
    assert np.array_equal(e.download(), p1)


# ---- full BASELINE sizes: EVERY nonzero against the oracle, plus size-independent properties --------------------------
def full_compare(p, d, oracle, tol, what):
    """All nonzeros of a full-size result against the CPU oracle (row ranges on a thread pool)."""
    ref = oracle_lib.sddmm_csr_all_rows(oracle, d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    bound = oracle_lib.abs_dot_bound_all_rows(oracle, d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    oracle_lib.assert_values_close(p, ref, bound, tol, what)
    return ref, bound


@pytest.mark.parametrize("cfg,K,mode", [(2, 32, "fp32"), (2, 32, "fp32_tc"), (2, 32, "tf32"), (2, 32, "bf16"), (3, 64, "fp32"),
                                        (4, 32, "fp32"), (4, 32, "bf16"), (5, 32, "fp32"), (5, 32, "bf16"), (2, 64, "fp32_tc"),
                                        (3, 32, "fp32_tc"), (5, 128, "bf16"), (5, 64, "fp32"), (5, 128, "fp32")])
def test_full_size_all_nonzeros(engines, oracle, cfg, K, mode):
    d = Dataset(cfg, K, 1.0)
    e = engines[mode]
    p = e.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    # (a) every nonzero against the oracle
    full_compare(p, d, oracle, TOL[mode], f"cfg{cfg} K={K} {mode} full size")
    # (b) 200 000 random nonzeros against a float64 dot product
    rng = np.random.default_rng(cfg)
    idx = np.sort(rng.choice(d.nnz, 200000, replace=False))
    rows = (np.searchsorted(d.row_ptr, idx, side="right") - 1).astype(np.int64)
    want = oracle_lib.dot_f64(rows, d.col_idx[idx], d.s_val[idx], d.A, d.B)
    bound = oracle_lib.abs_dot_bound(rows, d.col_idx[idx], d.s_val[idx], d.A, d.B)
    oracle_lib.assert_values_close(p[idx], want, bound, max(TOL[mode], 2e-6 * 1), f"cfg{cfg} sampled")
    # (c) linearity in S (exact: doubling is exact in fp32) and determinism
    e.update_values(d.s_val * 2)
    e.run()
    assert np.array_equal(e.download(), p * 2)
    e.update_values(d.s_val)
    e.run()
    assert np.array_equal(e.download(), p)
    # (d) COO upload gives the same bits
    if cfg in (2, 5):
        assert np.array_equal(e.sddmm_coo(d.M, d.N, d.K, d.row_idx(), d.col_idx, d.s_val, d.A, d.B), p)
    d.close()


@pytest.mark.parametrize("mode", ["fp32_tc", "tf32", "bf16", "fp32"])
def test_full_size_config2_randomly_placed_blocks(engines, oracle, mode):
    # configs[1] as BASELINE words it: 64x64 blocks at arbitrary (not grid-aligned) offsets
    d = Dataset(2, 32, 1.0, variant=1)
    p = engines[mode].sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    full_compare(p, d, oracle, TOL[mode], f"cfg2 unaligned blocks {mode} full size")
    d.close()


def test_golden_and_config1_against_the_reference_itself(engines, ref, oracle):
    # where the reference's own CPU path is at hand (oracle/_ref: its headers compiled unmodified) the GPU result is
    # compared with IT, not only with the restatement
    f = lambda b: np.array(b, np.uint32).view(np.float32)  # noqa: E731
    for name in sorted(GOLD["random"]):
        g = GOLD["random"][name]
        A, B = f(g["A_bits"]).reshape(g["M"], g["K"]), f(g["B_bits"]).reshape(g["N"], g["K"])
        rp, ci, sv = np.array(g["row_ptr"], np.int32), np.array(g["col_idx"], np.int32), f(g["s_val_bits"])
        want = ref.cpu_basic_csr(g["M"], g["N"], g["K"], rp, ci, sv, A, B)
        bound = oracle_lib.abs_dot_bound(oracle.coo_rows(g["M"], rp), ci, sv, A, B)
        for mode in ("fp32", "fp32_tc"):
            oracle_lib.assert_values_close(engines[mode].sddmm_csr(g["M"], g["N"], g["K"], rp, ci, sv, A, B), want, bound, 1e-5, name)
    for cfg, scale, K in ((1, 1.0, 32), (2, 0.05, 32), (4, 0.002, 32), (5, 0.003, 64)):
        d = Dataset(cfg, K, scale)
        want = ref.cpu_basic_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        want_coo = ref.cpu_basic_coo(d.M, d.N, d.K, d.row_idx(), d.col_idx, d.s_val, d.A, d.B)
        bound = oracle_lib.abs_dot_bound(oracle.coo_rows(d.M, d.row_ptr), d.col_idx, d.s_val, d.A, d.B)
        for mode in MODES:
            oracle_lib.assert_values_close(engines[mode].sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B), want, bound,
                                           TOL[mode], f"cfg{cfg} {mode} vs reference CSR")
            oracle_lib.assert_values_close(engines[mode].sddmm_coo(d.M, d.N, d.K, d.row_idx(), d.col_idx, d.s_val, d.A, d.B), want_coo,
                                           bound, TOL[mode], f"cfg{cfg} {mode} vs reference COO")
        d.close()


# ---- the row-segment kernel and its column panels -------------------------------------------------------------
@pytest.mark.parametrize("cfg,scale,K,mode,panels", [(5, 0.01, 32, "fp32", 1), (5, 0.01, 32, "fp32", 3), (5, 0.01, 64, "fp32", 4),
                                                      (4, 0.01, 32, "fp32", 2), (4, 0.01, 32, "bf16", 5), (5, 0.005, 128, "bf16", 2),
                                                      (5, 0.004, 256, "fp32", 3), (5, 0.01, 36, "fp32", 2), (2, 0.1, 32, "fp32", 7),
                                                      (1, 1.0, 32, "fp32", 64)])
def test_row_segments_and_column_panels(oracle, cfg, scale, K, mode, panels):
    # rows cut into segments of at most 8 nonzeros; with column panels the segment list is ordered panel-major
    d = Dataset(cfg, K, scale)
    e = Engine(0, mode)
    try:
        e.set_knob("rowseg", 1)
        e.set_knob("panels", panels)
        p = check(e, mode, oracle, d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, what=f"row segments cfg{cfg} K={K} {mode} P={panels}")
        plan = e.plan()
        assert [n for n, _ in e.kernel_times()] == ["sddmm_rowseg_kernel"]
        assert plan["rowseg_nnz"] == d.nnz and plan["rowseg_panels"] == panels and plan["rowtile_nnz"] == 0
        lens = np.diff(d.row_ptr).astype(np.int64)
        if panels == 1:
            assert plan["rowseg_units"] == int(((lens + 7) // 8).sum())
        else:
            assert int(((lens + 7) // 8).sum()) <= plan["rowseg_units"] <= d.nnz // 8 + min(d.nnz, d.M * panels)
        p_coo = check(e, mode, oracle, d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B, coo=True, what="row segments coo")
        assert np.array_equal(p, p_coo)
        # the same input through the A-row-tile kernel
        e2 = Engine(0, mode, flags=4)
        q = e2.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        assert [n for n, _ in e2.kernel_times()] == ["sddmm_rowtile_kernel"] and e2.plan()["rowseg_units"] == 0
        e2.close()
        bound = oracle_lib.abs_dot_bound(oracle.coo_rows(d.M, d.row_ptr), d.col_idx, d.s_val, d.A, d.B)
        oracle_lib.assert_values_close(q, p, bound, 2 * TOL[mode], "row-segment kernel vs row-tile kernel")
    finally:
        e.close()
        d.close()


def test_row_segments_edge_shapes(oracle):
    rng = np.random.default_rng(12)
    e = Engine(0, "fp32")
    e.set_knob("rowseg", 1)
    e.set_knob("panels", 3)

    def dense(m, k):
        return rng.uniform(-1, 1, (m, k)).astype(np.float32)

    try:
        # one 50 000-nnz row between empty rows; rows of exactly 8, 9, 1 nonzeros; a single column
        N = 60000
        cols = np.sort(rng.choice(N, 50000, replace=False)).astype(np.int32)
        check(e, "fp32", oracle, 4, N, 32, [0, 0, 50000, 50000, 50000], cols, rng.random(50000, dtype=np.float32), dense(4, 32), dense(N, 32),
              what="segments: one long row")
        lens = [8, 9, 1, 0, 16, 7, 0, 0, 33]
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        ci = np.concatenate([np.sort(rng.choice(100, n, replace=False)) for n in lens]).astype(np.int32)
        check(e, "fp32", oracle, len(lens), 100, 20, rp, ci, rng.random(ci.size, dtype=np.float32), dense(len(lens), 20), dense(100, 20),
              what="segments: ragged rows")
        assert e.plan()["rowseg_panels"] == 3
        check(e, "fp32", oracle, 5, 1, 4, [0, 1, 1, 2, 3, 3], [0, 0, 0], [1, 2, 3], dense(5, 4), dense(1, 4), what="segments: N=1")
        # unsorted columns inside rows: a panel run would not be contiguous, so the list is built without panels
        d = Dataset(uniform=(200, 300, 5000), K=32, seed=2)
        ci = d.col_idx.copy()
        for i in range(d.M):
            a, b = d.row_ptr[i], d.row_ptr[i + 1]
            ci[a:b] = rng.permutation(ci[a:b])
        check(e, "fp32", oracle, d.M, d.N, d.K, d.row_ptr, ci, d.s_val, d.A, d.B, what="segments: unsorted columns")
        assert e.plan()["rowseg_panels"] == 1 and e.plan()["rowseg_units"] > 0
        # K the chunked kernels cannot take falls to the scalar kernel whatever the knob says
        check(e, "fp32", oracle, d.M, d.N, 3, d.row_ptr, d.col_idx, d.s_val, dense(d.M, 3), dense(d.N, 3), what="segments: K=3")
        assert e.plan()["rowseg_units"] == 0
    finally:
        e.close()


def test_two_engines_on_one_device_keep_their_launch_limits(oracle):
    # the dynamic shared memory limit of a kernel belongs to the device, not to an engine: an engine whose rows are short
    # (small stage) must not leave another engine, whose plan needs a large stage, with a limit below its launch
    long_rows = Dataset(uniform=(600, 4000, 600 * 400), K=32, seed=3)      # mean row length 400 -> few rows per stage
    short_rows = Dataset(uniform=(60000, 4000, 60000 * 4), K=32, seed=4)   # mean row length 4 -> 256 rows per stage
    a, b = Engine(0, "fp32", flags=4), Engine(0, "fp32", flags=4)          # (flags=4: the row-tile kernel)
    try:
        b.upload_csr(short_rows.M, short_rows.N, 32, short_rows.row_ptr, short_rows.col_idx, short_rows.s_val, short_rows.A, short_rows.B)
        a.upload_csr(long_rows.M, long_rows.N, 32, long_rows.row_ptr, long_rows.col_idx, long_rows.s_val, long_rows.A, long_rows.B)
        assert b.plan()["rowtile_smem_bytes"] > a.plan()["rowtile_smem_bytes"]
        for eng, d in ((b, short_rows), (a, long_rows), (b, short_rows)):
            eng.run()
            p = eng.download()
            want = oracle.sddmm_csr(d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
            bound = oracle_lib.abs_dot_bound(oracle.coo_rows(d.M, d.row_ptr), d.col_idx, d.s_val, d.A, d.B)
            oracle_lib.assert_values_close(p, want, bound, 1e-5, "two engines on one device")
    finally:
        a.close()
        b.close()
    # chunked call whose first half has short rows and whose second half has long ones, then the pattern replayed
    rp = np.concatenate([short_rows.row_ptr, long_rows.row_ptr[1:] + short_rows.row_ptr[-1]]).astype(np.int32)
    ci = np.concatenate([short_rows.col_idx, long_rows.col_idx])
    sv = np.concatenate([short_rows.s_val, long_rows.s_val])
    A = np.concatenate([short_rows.A, long_rows.A])
    B = short_rows.B
    M = rp.size - 1
    want = oracle.sddmm_csr(M, 32, rp, ci, sv, A, B)
    bound = oracle_lib.abs_dot_bound(oracle.coo_rows(M, rp), ci, sv, A, B)
    with Pipeline(0, "fp32", flags=4, chunks=2, min_chunk_bytes=1 << 20) as pl:
        p = pl.sddmm_csr(M, 4000, 32, rp, ci, sv, A, B)
        assert pl.last_chunks() == 2
        oracle_lib.assert_values_close(p, want, bound, 1e-5, "chunked call, short then long rows")
        out = np.zeros(ci.size, np.float32)
        pl.update_csr_raw(sv, A, B, out)
        oracle_lib.assert_values_close(out, want, bound, 1e-5, "chunked call replayed")


def _blocked_pattern(rng, n_block_rows, G, N, blocks_per_row, break_every=0):
    """CSR pattern of G x G dense blocks: the G rows of a block row share one column list.
    break_every > 0 drops the last entry of the last row of every break_every-th block row, so that group does not match."""
    rp, ci = [0], []
    for b in range(n_block_rows):
        bc = np.sort(rng.choice(N // G, size=min(blocks_per_row, N // G), replace=False))
        cols = (bc[:, None] * G + np.arange(G)[None, :]).ravel()
        for t in range(G):
            c = cols[:-1] if (break_every and b % break_every == 0 and t == G - 1) else cols
            ci.extend(c.tolist())
            rp.append(len(ci))
    return np.array(rp, np.int32), np.array(ci, np.int32)


@pytest.mark.parametrize("G,K,extra_rows,break_every,lead_rows", [(3, 64, 0, 0, 0), (3, 32, 2, 5, 1), (2, 32, 1, 0, 1), (4, 64, 3, 7, 0),
                                                                  (4, 32, 0, 3, 3), (3, 64, 1, 0, 2)])
def test_row_groups_share_the_gather(engines, oracle, G, K, extra_rows, break_every, lead_rows):
    # rows with identical column lists (block rows of G x G blocks) take the row-group kernel; the result is the same.
    # lead_rows: rows in front of the first block row (a row shard cut in the middle of a block row)
    rng = np.random.default_rng(100 * G + K + extra_rows + 7 * lead_rows)
    N = 1200
    rp, ci = _blocked_pattern(rng, 150, G, N, 20, break_every)
    for _ in range(lead_rows):
        lead = np.sort(rng.choice(N, size=23, replace=False)).astype(np.int32)
        ci = np.concatenate([lead, ci])
        rp = np.concatenate([[0], rp + len(lead)]).astype(np.int32)
    blocked_nnz = int(rp[lead_rows + 150 * G] - rp[lead_rows])
    for _ in range(extra_rows):   # ragged tail: rows that belong to no complete group
        extra = np.sort(rng.choice(N, size=17, replace=False)).astype(np.int32)
        ci = np.concatenate([ci, extra])
        rp = np.concatenate([rp, [len(ci)]]).astype(np.int32)
    M = len(rp) - 1
    sv = rng.random(len(ci), dtype=np.float32)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (N, K)).astype(np.float32)
    for mode in ("fp32", "fp32_tc"):
        p = check(engines[mode], mode, oracle, M, N, K, rp, ci, sv, A, B, what=f"row groups G={G} K={K} {mode}")
        plan = engines[mode].plan()
        assert plan["rowgroup_rows"] == G and plan["n_kernels"] == 1 and plan["rowtile_nnz"] == 0
        # the group's column list cut into shared segments of 8 columns: one unit serves all G rows
        assert [n for n, _ in engines[mode].kernel_times()] == ["sddmm_rowseg_group_kernel"]
        lens = np.diff(rp).astype(np.int64)
        assert plan["rowseg_units"] <= int(((lens + 7) // 8).sum())
        if not break_every:
            assert plan["rowgroup_nnz"] == blocked_nnz
            assert plan["rowseg_units"] == int(((lens + 7) // 8).sum()) - (G - 1) * 150 * ((int(lens[lead_rows]) + 7) // 8)
        else:
            assert 0 < plan["rowgroup_nnz"] < blocked_nnz
    # the same groups through the warp-per-group kernel (knob "group_units" = 0)
    with Engine(0, "fp32") as e0:
        e0.set_knob("group_units", 0)
        q0 = e0.sddmm_csr(M, N, K, rp, ci, sv, A, B)
        assert [n for n, _ in e0.kernel_times()] == ["sddmm_rowgroup_kernel"] and e0.plan()["rowgroup_rows"] == G
        bound0 = oracle_lib.abs_dot_bound(oracle.coo_rows(M, rp), ci, sv, A, B)
        oracle_lib.assert_values_close(q0, p, bound0, 2e-5, "row-group kernel vs shared segments")
    # the same input with the path switched off goes through the row-tile kernel and agrees
    e = Engine(0, "fp32", flags=2)
    try:
        q = e.sddmm_csr(M, N, K, rp, ci, sv, A, B)
        assert e.plan()["rowgroup_rows"] == 0
        bound = oracle_lib.abs_dot_bound(oracle.coo_rows(M, rp), ci, sv, A, B)
        oracle_lib.assert_values_close(q, p, bound, 2e-5, "row-group kernel vs row-tile kernel")
    finally:
        e.close()


def test_row_groups_not_taken_without_structure(engines):
    # uniformly random rows: no aligned group matches, the general kernel runs
    d = Dataset(5, 32, 0.002)
    e = engines["fp32"]
    e.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    assert e.plan()["rowgroup_rows"] == 0 and e.plan()["rowseg_nnz"] + e.plan()["rowtile_nnz"] == d.nnz


def test_kernel_timing_is_opt_in():
    # kernel names are always reported; an event pair around every kernel is recorded only on request
    d = Dataset(2, 32, 0.12)
    e = Engine(0, "fp32_tc")
    try:
        e.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        names = [n for n, _ in e.kernel_times()]
        assert names == ["sddmm_dense_tile_kernel", "sddmm_rowseg_kernel"]   # the tiles, and what they left as row segments
        assert all(ms == -1.0 for _, ms in e.kernel_times())
        e.set_kernel_timing(True)
        e.run(); e.sync()
        assert [n for n, _ in e.kernel_times()] == names and all(ms > 0 for _, ms in e.kernel_times())
        assert e.last_run_ms() > 0
        e.set_kernel_timing(False)
        e.run(); e.sync()
        assert all(ms == -1.0 for _, ms in e.kernel_times()) and e.last_run_ms() > 0
    finally:
        e.close()


@pytest.mark.parametrize("cfg,scale,K,mode,chunks", [(2, 0.3, 32, "fp32_tc", 4), (2, 0.3, 32, "fp32", 3), (2, 0.25, 32, "tf32", 8),
                                                      (3, 0.02, 64, "fp32", 4), (5, 0.02, 32, "fp32", 5), (5, 0.01, 128, "bf16", 2)])
def test_pipeline_matches_oracle_and_engine(engines, oracle, cfg, scale, K, mode, chunks):
    # chunked host-to-host call: same values as one engine (same kernels per nonzero), pattern order kept across the cuts
    d = Dataset(cfg, K, scale)
    with Pipeline(0, mode, chunks=chunks, min_chunk_bytes=1 << 20) as pl:
        p = pl.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        assert 1 < pl.last_chunks() <= chunks
        p_again = pl.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)   # the object is reusable
        p_coo = pl.sddmm_coo(d.M, d.N, d.K, oracle.coo_rows(d.M, d.row_ptr), d.col_idx, d.s_val, d.A, d.B)
        assert 1 < pl.last_chunks() <= chunks
        # same pattern, new numbers: only S.val, A, B travel, the plans stay
        rng = np.random.default_rng(11)
        sv2 = rng.uniform(-1, 1, d.s_val.size).astype(np.float32)
        A2, B2 = rng.uniform(-1, 1, (d.M, K)).astype(np.float32), rng.uniform(-1, 1, (d.N, K)).astype(np.float32)
        p2 = np.full(d.s_val.size, np.nan, np.float32)
        pl.update_csr_raw(sv2, A2, B2, p2)
    p_ref = oracle.sddmm_csr(d.M, K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    rows = oracle.coo_rows(d.M, d.row_ptr)
    bound = oracle_lib.abs_dot_bound(rows, d.col_idx, d.s_val, d.A, d.B)
    np.testing.assert_array_equal(p, p_again)   # (overlapping tiles included: their shared nonzeros have a deterministic owner)
    oracle_lib.assert_values_close(p, p_ref, bound, TOL[mode], f"pipeline {mode} cfg{cfg}")
    oracle_lib.assert_values_close(p_coo, p_ref, bound, TOL[mode], f"pipeline coo {mode} cfg{cfg}")   # (its cuts may differ by a row)
    p_one = engines[mode].sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    oracle_lib.assert_values_close(p, p_one, bound, 2 * TOL[mode], f"pipeline vs one engine {mode} cfg{cfg}")
    p2_ref = oracle.sddmm_csr(d.M, K, d.row_ptr, d.col_idx, sv2, A2, B2)
    oracle_lib.assert_values_close(p2, p2_ref, oracle_lib.abs_dot_bound(rows, d.col_idx, sv2, A2, B2), TOL[mode], f"pipeline update {mode} cfg{cfg}")


def test_pipeline_edges(oracle):
    rng = np.random.default_rng(7)
    with Pipeline(0, "fp32", chunks=4, min_chunk_bytes=4 << 20) as pl:
        with pytest.raises(SddmmError) as ei:   # no pattern yet
            pl.update_csr_raw(np.ones(3, np.float32), np.ones((3, 4), np.float32), np.ones((3, 4), np.float32), np.zeros(3, np.float32))
        assert ei.value.code == 5
        # small input: one range; golden-sized case exact
        A = np.ones((3, 4), np.float32)
        assert pl.sddmm_csr(3, 3, 4, [0, 1, 2, 3], [0, 1, 2], [1, 1, 1], A, A).tolist() == [4.0, 4.0, 4.0]
        assert pl.last_chunks() == 1
        # no nonzeros at all
        assert pl.sddmm_csr(3, 3, 4, [0, 0, 0, 0], [], [], A, A).size == 0
        # all nonzeros in few rows between long runs of empty rows: some ranges hold no rows or no nonzeros
        M, N, K = 40, 300000, 32
        lens = np.zeros(M, np.int64)
        lens[[5, 6, 30]] = [200000, 150000, 100000]
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        ci = np.concatenate([np.sort(rng.choice(N, n, replace=False)) for n in lens if n]).astype(np.int32)
        sv = rng.uniform(-1, 1, ci.size).astype(np.float32)
        A, B = rng.uniform(-1, 1, (M, K)).astype(np.float32), rng.uniform(-1, 1, (N, K)).astype(np.float32)
        p = pl.sddmm_csr(M, N, K, rp, ci, sv, A, B)
        assert pl.last_chunks() == 4
        p_ref = oracle.sddmm_csr(M, K, rp, ci, sv, A, B)
        bound = oracle_lib.abs_dot_bound(oracle.coo_rows(M, rp), ci, sv, A, B)
        oracle_lib.assert_values_close(p, p_ref, bound, 1e-5, "pipeline ragged")
        # errors name the status of the engine; the object stays usable
        bad = rp.copy()
        bad[7] = bad[6] - 5
        with pytest.raises(SddmmError) as ei:
            pl.sddmm_csr(M, N, K, bad, ci, sv, A, B)
        assert ei.value.code == 2
        ci_bad = ci.copy()
        ci_bad[-1] = N
        with pytest.raises(SddmmError) as ei:
            pl.sddmm_csr(M, N, K, rp, ci_bad, sv, A, B)
        assert ei.value.code == 2
        rows = oracle.coo_rows(M, rp)
        oracle_lib.assert_values_close(pl.sddmm_coo(M, N, K, rows, ci, sv, A, B), p_ref, bound, 1e-5, "pipeline ragged coo")
        rows_bad = rows.copy()
        rows_bad[250000], rows_bad[250001] = rows_bad[-1], rows_bad[0]   # unsorted inside a chunk
        with pytest.raises(SddmmError) as ei:
            pl.sddmm_coo(M, N, K, rows_bad, ci, sv, A, B)
        assert ei.value.code == 2
        rows_bad = rows.copy()
        rows_bad[-1] = M
        with pytest.raises(SddmmError) as ei:
            pl.sddmm_coo(M, N, K, rows_bad, ci, sv, A, B)
        assert ei.value.code == 2
        with pytest.raises(SddmmError) as ei:   # the failed call left no usable pattern
            pl.update_csr_raw(sv, A, B, np.zeros(ci.size, np.float32))
        assert ei.value.code == 5
        np.testing.assert_array_equal(pl.sddmm_csr(M, N, K, rp, ci, sv, A, B), p)
        p_up = np.zeros(ci.size, np.float32)
        pl.update_csr_raw(sv, 2 * A, B, p_up)   # ranges without rows or nonzeros are skipped here too
        oracle_lib.assert_values_close(p_up, 2 * p_ref, 2 * bound, 1e-5, "pipeline ragged update")
    with pytest.raises(SddmmError):
        Pipeline(0, "fp32", chunks=0)


# ---- the consumer of P on the device: Y = P X ------------------------------------------------------------------
@pytest.mark.parametrize("cfg,scale,K,mode,K2", [(5, 0.01, 32, "fp32", 32), (4, 0.01, 32, "fp32", 64), (2, 0.1, 32, "fp32_tc", 32),
                                                  (3, 0.01, 64, "fp32", 16), (5, 0.005, 64, "bf16", 36), (1, 1.0, 32, "fp32", 256)])
def test_consumer_spmm_on_the_device_resident_result(engines, oracle, cfg, scale, K, mode, K2):
    import scipy.sparse as sp

    d = Dataset(cfg, K, scale)
    e = engines[mode]
    p = e.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    rng = np.random.default_rng(K2)
    X = rng.uniform(-1, 1, (d.N, K2)).astype(np.float32)
    Y = e.spmm(X)
    assert Y.shape == (d.M, K2) and np.isfinite(Y).all()
    # (a) the consumer alone: against a float64 product with the P the engine itself computed
    P64 = sp.csr_matrix((p.astype(np.float64), d.col_idx, d.row_ptr), shape=(d.M, d.N))
    want = P64 @ X.astype(np.float64)
    bound = abs(P64) @ np.abs(X.astype(np.float64))
    assert (np.abs(Y - want) <= 3e-5 * bound + 1e-30).all(), f"consumer off by up to {np.max(np.abs(Y - want) / (bound + 1e-30)):.2e} of the bound"
    # (b) the chain SDDMM -> SpMM against the CPU oracle's chain
    p_ref = oracle.sddmm_csr(d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    y_ref = oracle.spmm_csr(d.M, K2, d.row_ptr, d.col_idx, p_ref, X)
    rows = oracle.coo_rows(d.M, d.row_ptr)
    pb = oracle_lib.abs_dot_bound(rows, d.col_idx, d.s_val, d.A, d.B)            # scale of each P entry
    chain_bound = sp.csr_matrix((pb, d.col_idx, d.row_ptr), shape=(d.M, d.N)) @ np.abs(X.astype(np.float64))
    tol = 4 * TOL[mode]
    assert (np.abs(Y - y_ref) <= tol * chain_bound + 1e-30).all(), "SDDMM -> SpMM chain differs from the oracle's"
    # a second call (other K2) reuses the unit list; the result of the first call is reproducible to rounding
    Y2 = e.spmm(X[:, :8].copy())
    assert (np.abs(Y2 - want[:, :8]) <= 3e-5 * bound[:, :8] + 1e-30).all()
    if d.M == d.N or True:   # X = None: the engine's own copy of B is the right-hand side (nothing is uploaded)
        Bq = d.B.astype(np.float32)
        if mode == "bf16":   # the engine holds the bf16-rounded B
            Bq = (Bq.view(np.uint32) + 0x7FFF + ((Bq.view(np.uint32) >> 16) & 1) & 0xFFFF0000).astype(np.uint32).view(np.float32)
        YB = e.spmm(None)
        wantB = P64 @ Bq.astype(np.float64)
        boundB = abs(P64) @ np.abs(Bq.astype(np.float64))
        assert YB.shape == (d.M, d.K) and (np.abs(YB - wantB) <= 3e-5 * boundB + 1e-30).all()
    assert e.last_spmm_ms() > 0
    d.close()


def test_consumer_rejects_what_it_cannot_take(engines):
    e = engines["fp32"]
    A = np.ones((3, 4), np.float32)
    e.sddmm_csr(3, 3, 4, [0, 1, 2, 3], [0, 1, 2], [1, 1, 1], A, A)
    assert e.spmm(np.ones((3, 4), np.float32)).tolist() == [[4.0] * 4] * 3
    for bad in (3, 6, 260):
        with pytest.raises(SddmmError) as ei:
            e.spmm(np.ones((3, bad), np.float32))
        assert ei.value.code == 6
    fresh = Engine(0, "fp32")
    with pytest.raises(SddmmError) as ei:
        fresh.spmm(np.ones((3, 4), np.float32), rows=3)
    assert ei.value.code == 5
    fresh.close()


def test_bounded_wait_runs_out_and_is_reported(oracle):
    # the failure path of every device-side wait, exercised without a fault: a one-thread kernel waits a bounded number of
    # times on a barrier nothing completes, records the time-out and returns; sync reports it; the next run is clean again
    d = Dataset(1, 32, 1.0)
    with Engine(0, "fp32") as e:
        p = e.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        assert e.lib.sddmm_b200_selftest_wait_timeout(e.h, 64) == 8            # SDDMM_B200_ERR_DEVICE_WAIT
        assert b"wait" in e.lib.sddmm_b200_last_error(e.h)
        assert e.lib.sddmm_b200_selftest_wait_timeout(e.h, 0) == 1             # bad argument
        e.run()                                                                  # clears the error word
        assert np.array_equal(e.download(), p)
    fresh = Engine(0, "fp32")
    assert fresh.lib.sddmm_b200_selftest_wait_timeout(fresh.h, 64) == 5         # before any upload: call order
    fresh.close()
@pytest.mark.gpu
def test_coo_row_slices_keep_the_global_row_numbers(oracle):
    """Row shards of one COO matrix (sddmm_b200_coo_cuts + sddmm_b200_upload_coo_rows): each engine gets its slice of the
    caller's arrays as they are, the device subtracts the slice's first row; together the slices give the whole result."""
    from dphpc_b200.partition import coo_cuts
    d = Dataset(5, 32, 0.02)
    rows = d.row_idx()
    want = oracle.sddmm_csr(d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    bound = oracle_lib.abs_dot_bound(rows, d.col_idx, d.s_val, d.A, d.B)
    cuts, offs = coo_cuts(rows, d.M, 3, align=64)
    got = np.empty(d.nnz, np.float32)
    for g in range(3):
        r0, r1, j0, j1 = int(cuts[g]), int(cuts[g + 1]), int(offs[g]), int(offs[g + 1])
        with Engine(0, "fp32") as e:
            e.upload_coo_rows(r1 - r0, d.N, d.K, r0, rows[j0:j1], d.col_idx[j0:j1], d.s_val[j0:j1], d.A[r0:r1], d.B)
            e.run(); e.sync()
            got[j0:j1] = e.download()
    oracle_lib.assert_values_close(got, want, bound, 1e-5, "COO row slices")
    with Engine(0, "fp32") as e:   # a slice that holds a row of its neighbour is refused, not misread
        r0, r1, j0, j1 = int(cuts[1]), int(cuts[2]), int(offs[1]), int(offs[2])
        with pytest.raises(SddmmError) as err:
            e.upload_coo_rows(r1 - r0, d.N, d.K, r0, rows[j0 - 1:j1], d.col_idx[j0 - 1:j1], d.s_val[j0 - 1:j1], d.A[r0:r1], d.B)
        assert err.value.code == 2   # SDDMM_B200_ERR_INDEX
    d.close()


@pytest.mark.gpu
@pytest.mark.parametrize("K", [32, 64, 96])
@pytest.mark.parametrize("variant", [0, 1])
def test_fp32_grade_dense_tiles_three_slot_operands(oracle, K, variant):
    """fp32-grade mode on dense tiles with the operands going through three shared-memory slots and two accumulators in
    tensor memory (the default for K >= 64) against the one-buffer form: both within the fp32 bar of the oracle, for one,
    two and three 32-column pieces of K, tiles on the grid and at arbitrary offsets (overlapping tiles: own masks)."""
    d = Dataset(2, K, 0.15, variant=variant)
    want = oracle.sddmm_csr(d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    bound = oracle_lib.abs_dot_bound(oracle.coo_rows(d.M, d.row_ptr), d.col_idx, d.s_val, d.A, d.B)
    for split3 in (1, 0):
        with Engine(0, "fp32_tc") as e:
            e.set_knob("dense_split3", split3)
            p = e.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
            plan = e.plan()
            assert plan["dense_tiles"] > 0 and plan["dense_nnz"] > 0.9 * d.nnz
        oracle_lib.assert_values_close(p, want, bound, 1e-5, f"fp32_tc K={K} variant {variant} split3={split3}")
    d.close()


@pytest.mark.gpu
@pytest.mark.parametrize("K,panels", [(128, 1), (192, 2), (256, 3)])
@pytest.mark.parametrize("mode", ["fp32", "fp32_tc"])
def test_k_in_slices_of_64_columns(oracle, K, panels, mode):
    """Large K on the row-segment path: one launch per 64-column slice of K over the same segment list, every later slice
    adding to P.val (what the planner does when B is far larger than L2); forced here on a small input, with and without
    column panels, and run twice (the first slice of a run must overwrite what the previous run left)."""
    d = Dataset(5, K, 0.01)
    want = oracle.sddmm_csr(d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    bound = oracle_lib.abs_dot_bound(oracle.coo_rows(d.M, d.row_ptr), d.col_idx, d.s_val, d.A, d.B)
    with Engine(0, mode) as e:
        e.set_knob("k_slices", 1)
        e.set_knob("panels", panels)
        e.upload_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        plan = e.plan()
        assert plan["rowseg_passes"] == K // 64 and plan["rowseg_panels"] == panels
        for _ in range(2):
            e.run(); e.sync()
            oracle_lib.assert_values_close(e.download(), want, bound, 1e-5, f"{mode} K={K} in {K // 64} slices, {panels} panels")
    with Engine(0, mode) as e:   # and the whole rows at once agree with it
        e.set_knob("k_slices", 0)
        p1 = e.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        assert e.plan()["rowseg_passes"] == 1
    oracle_lib.assert_values_close(p1, want, bound, 1e-5, f"{mode} K={K} whole rows")
    d.close()


@pytest.mark.gpu
def test_k_slices_beside_dense_tiles(oracle):
    """K in slices on what the dense tiles leave: the residual row segments run once per slice on the side stream and add to
    their own nonzeros only, the tensor-core kernel writes the rest (fp32-grade mode, K = 128, blocks at arbitrary offsets)."""
    d = Dataset(2, 128, 0.1, variant=1)
    want = oracle.sddmm_csr(d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    bound = oracle_lib.abs_dot_bound(oracle.coo_rows(d.M, d.row_ptr), d.col_idx, d.s_val, d.A, d.B)
    with Engine(0, "fp32_tc") as e:
        e.set_knob("k_slices", 1)
        e.upload_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        plan = e.plan()
        assert plan["dense_tiles"] > 0 and 0 < plan["dense_nnz"] < d.nnz
        for _ in range(2):
            e.run(); e.sync()
            oracle_lib.assert_values_close(e.download(), want, bound, 1e-5, "fp32_tc K=128: dense tiles + sliced residual")
    d.close()


@pytest.mark.gpu
@pytest.mark.parametrize("cfg,scale", [(4, 0.02), (5, 0.01)])
@pytest.mark.parametrize("panels,threshold", [(2, 16), (3, 8), (4, 64)])
def test_column_panels_for_the_long_rows_only(oracle, cfg, scale, panels, threshold):
    """Power-law row lengths: the rows of at least `threshold` nonzeros are cut into column panels, the shorter rows follow
    whole as one more entry of the panel-major segment list (what the planner does on the full-size power-law
    configuration, where B is far larger than L2; forced here on small inputs, also on one whose rows are all alike)."""
    d = Dataset(cfg, 32, scale)
    want = oracle.sddmm_csr(d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    bound = oracle_lib.abs_dot_bound(oracle.coo_rows(d.M, d.row_ptr), d.col_idx, d.s_val, d.A, d.B)
    with Engine(0, "fp32") as e:
        e.set_knob("panels", panels)
        e.set_knob("long_rows", threshold)
        p = e.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        plan = e.plan()
        assert plan["rowseg_panels"] == panels + 1 and plan["rowseg_nnz"] == d.nnz
        e.update_values(d.s_val * 2.0)   # the per-unit copies of S follow the new values
        e.run(); e.sync()
        p2 = e.download()
    oracle_lib.assert_values_close(p, want, bound, 1e-5, f"cfg{cfg}: {panels} panels for rows >= {threshold}")
    oracle_lib.assert_values_close(p2, 2.0 * want, 2.0 * bound, 1e-5, f"cfg{cfg}: the same after update_values")
    d.close()


@pytest.mark.gpu
def test_full_size_chunked_call_on_power_law_rows(engines, oracle):
    """The chunked host-to-host call on the full-size power-law configuration: every row range plans for itself (column
    panels for its long rows only) and the whole result still equals the one-engine result bit for bit and the oracle within
    the fp32 bar, the COO form included."""
    d = Dataset(4, 32, 1.0)
    with Pipeline(0, "fp32", chunks=4) as pl:
        p = pl.sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
        assert pl.last_chunks() == 4
        p_coo = pl.sddmm_coo(d.M, d.N, d.K, d.row_idx(), d.col_idx, d.s_val, d.A, d.B)
    full_compare(p, d, oracle, TOL["fp32"], "chunked call, power-law rows, full size")
    p_one = engines["fp32"].sddmm_csr(d.M, d.N, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    assert engines["fp32"].plan()["rowseg_panels"] > 1   # (the long-row panels are in use on the whole matrix)
    np.testing.assert_array_equal(p, p_one)
    np.testing.assert_array_equal(p_coo, p_one)
    d.close()


