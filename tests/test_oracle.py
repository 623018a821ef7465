"""The CPU oracle (oracle/sddmm_oracle.c) pinned against the reference.

Three anchors: (1) literals from the reference's own tests (tests/matrix_test.cc
dispatcher vectors :354-425, :460-477; DummyDataset's expected 2.0s,
src/benchmark/dataset.hpp:183-204); (2) the committed fixture generated from the
reference's code (tests/golden/make_golden.py); (3) the reference's headers
compiled here (oracle/_ref), bit for bit, when present.
"""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

from dphpc_b200 import Dataset

GOLD = json.loads((Path(__file__).parent / "golden" / "sddmm_golden.json").read_text())


def f32_from_bits(b):
    return np.array(b, dtype=np.uint32).view(np.float32)


# ---- (1) literals of the reference's tests ------------------------------------------------
def test_dummy_dataset_known_answer(oracle):
    A = np.ones((2, 2), np.float32)
    rp, ci, sv = oracle.csr_from_triplets(2, [0, 0, 1, 1], [0, 1, 0, 1], [1, 1, 1, 1])
    p = oracle.sddmm_csr(2, 2, rp, ci, sv, A, A)
    assert p.tolist() == [2.0, 2.0, 2.0, 2.0]


@pytest.mark.parametrize("rows,cols,M,parts,stride,expected", [
    ([0, 1, 0, 1], [0, 0, 1, 1], 2, 4, 1, [0, 1, 2, 2, 2]),   # dispatcher_more_threads_than_rows
    ([0, 1, 0, 1], [0, 0, 1, 1], 2, 2, 1, [0, 1, 2]),         # dispatcher_equal_num_threads_than_rows
    ([0, 1, 2, 3], [0, 0, 1, 1], 4, 2, 1, [0, 2, 4]),         # dispatcher_less_threads_than_rows
    ([1], [0], 4, 2, 1, [0, 4, 4]),                           # dispatcher_empty_rows
])
def test_dispatcher_literals(oracle, rows, cols, M, parts, stride, expected):
    rp, _, _ = oracle.csr_from_triplets(M, rows, cols, np.ones(len(rows), np.float32))
    assert oracle.dispatch(M, rp, parts, stride).tolist() == expected


def test_dispatcher_large_regular_input(oracle):
    n = 150000  # tests/matrix_test.cc:406-425
    rp = np.arange(n + 1, dtype=np.int32)
    got = oracle.dispatch(n, rp, n // 2)
    assert np.array_equal(got, 2 * np.arange(n // 2 + 1, dtype=np.int32))


def test_dispatcher_tensor_stride16(oracle):
    rp = np.arange(65, dtype=np.int32)  # test_dispatch_tensor, :460-477
    assert oracle.dispatch(64, rp, 4, 16).tolist() == [0, 16, 32, 48, 64]


def test_representation_conversion(oracle):
    # BasicTest.RepresentationConversion / BiggerConversion (:93-122): CSR(COO) == CSR, COO(CSR) == COO,
    # unsorted triplets come out sorted
    rng = np.random.default_rng(7)
    for i in range(100, 1501, 175):
        rows, cols, n = 2 * i, i, i
        cells = rng.choice(rows * cols, size=n, replace=False)
        r, c = (cells // cols).astype(np.int32), (cells % cols).astype(np.int32)
        v = rng.random(n, dtype=np.float32) + 0.5
        rp, ci, sv = oracle.csr_from_triplets(rows, r, c, v)
        cr, cc, cv = oracle.sort_unique(r, c, v)
        assert np.array_equal(oracle.coo_rows(rows, rp), cr) and np.array_equal(ci, cc) and np.array_equal(sv, cv)
        order = np.lexsort((c, r))
        assert np.array_equal(cr, r[order]) and np.array_equal(cc, c[order])


def test_unique_rule_keeps_zero_valued_duplicates(oracle):
    # Triplet operator== ANDs the values as booleans (src/matrices/triplet.h:11-14)
    r, c, v = oracle.sort_unique([0, 0, 0, 0], [1, 1, 2, 2], [1.0, 2.0, 0.0, 3.0])
    assert c.tolist() == [1, 2, 2] and v.tolist() == [1.0, 0.0, 3.0]


# ---- (2) committed fixture --------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(GOLD["tiny"]))
def test_tiny_cases_against_fixture(oracle, name):
    g = GOLD["tiny"][name]
    A, B = np.array(g["A"], np.float32), np.array(g["B"], np.float32)
    t = g["triplets"]
    rp, ci, sv = oracle.csr_from_triplets(g["M"], [x[0] for x in t], [x[1] for x in t], [x[2] for x in t])
    assert rp.tolist() == g["row_ptr"] and ci.tolist() == g["col_idx"] and sv.tolist() == g["s_val"]
    assert oracle.sddmm_csr(g["M"], g["K"], rp, ci, sv, A, B).tolist() == g["p_csr"]
    assert oracle.sddmm_coo(g["K"], g["coo_rows"], g["coo_cols"], sv, A, B).tolist() == g["p_coo"]


@pytest.mark.parametrize("name", sorted(GOLD["random"]))
def test_random_cases_bit_exact_against_fixture(oracle, name):
    g = GOLD["random"][name]
    A, B = f32_from_bits(g["A_bits"]), f32_from_bits(g["B_bits"])
    rp, ci, sv = oracle.csr_from_triplets(g["M"], g["trip_rows"], g["trip_cols"], f32_from_bits(g["trip_vals_bits"]))
    assert rp.tolist() == g["row_ptr"] and ci.tolist() == g["col_idx"]
    assert np.array_equal(sv.view(np.uint32), np.array(g["s_val_bits"], np.uint32))
    p = oracle.sddmm_csr(g["M"], g["K"], rp, ci, sv, A, B)
    assert np.array_equal(p.view(np.uint32), np.array(g["p_bits"], np.uint32))


@pytest.mark.parametrize("key", sorted(GOLD["configs"]))
def test_config_digests_against_fixture(oracle, key):
    g = GOLD["configs"][key]
    d = Dataset(g["config"], g["K"], g["scale"])
    assert (d.M, d.N, d.nnz, d.seed) == (g["M"], g["N"], g["nnz"], g["seed"])
    assert hashlib.sha256(d.row_ptr.tobytes() + d.col_idx.tobytes()).hexdigest() == g["pattern_sha256"]
    assert hashlib.sha256(d.s_val.tobytes() + d.A.tobytes() + d.B.tobytes()).hexdigest() == g["inputs_sha256"]
    p = oracle.sddmm_csr(d.M, d.K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    assert hashlib.sha256(p.tobytes()).hexdigest() == g["p_sha256"]
    assert np.array_equal(p[:8].view(np.uint32), np.array(g["p_head_bits"], np.uint32))
    # CSR and COO forms of the oracle agree bit for bit (sddmm_csr_coo, tests/matrix_test.cc:229-246)
    assert np.array_equal(p, oracle.sddmm_coo(d.K, oracle.coo_rows(d.M, d.row_ptr), d.col_idx, d.s_val, d.A, d.B))


@pytest.mark.parametrize("name", sorted(GOLD["dispatch"]))
def test_dispatch_against_fixture(oracle, name):
    g = GOLD["dispatch"][name]
    rp = np.arange(g["M"] + 1, dtype=np.int32) if g["row_ptr"] == "diag" else np.array(g["row_ptr"], np.int32)
    s = oracle.dispatch(g["M"], rp, g["parts"], 16 if g["tensor"] else 1)
    assert hashlib.sha256(s.astype(np.int32).tobytes()).hexdigest() == g["start_idx_sha256"]


# ---- (3) the reference compiled here ------------------------------------------------------------
@pytest.mark.parametrize("M,N,K,density", [(500, 500, 32, 0.3), (250, 250, 32, 0.7), (3000, 3000, 32, 0.001),
                                           (97, 131, 7, 0.2), (4562 // 8, 5761 // 8, 64, 0.02)])
def test_oracle_equals_reference_bitwise(oracle, ref, M, N, K, density):
    # shapes of sddmm_random_coo / _dense_coo / _sparse_coo (tests/matrix_test.cc:184-227), scaled for time
    d = Dataset(uniform=(M, N, int(M * N * density)), K=K, seed=M * 31 + K)
    rows = d.row_idx()
    p_ref = ref.cpu_basic_csr(M, N, K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B)
    assert np.array_equal(p_ref, oracle.sddmm_csr(M, K, d.row_ptr, d.col_idx, d.s_val, d.A, d.B))
    assert np.array_equal(ref.cpu_basic_coo(M, N, K, rows, d.col_idx, d.s_val, d.A, d.B),
                          oracle.sddmm_coo(K, rows, d.col_idx, d.s_val, d.A, d.B))
    # generator output is already what the reference's constructors would build from the same triplets
    rp, ci, sv = ref.csr_from_triplets(M, N, rows[::-1], d.col_idx[::-1], d.s_val[::-1])
    assert np.array_equal(rp, d.row_ptr) and np.array_equal(ci, d.col_idx) and np.array_equal(sv, d.s_val)
    orp, oci, osv = oracle.csr_from_triplets(M, rows[::-1], d.col_idx[::-1], d.s_val[::-1])
    assert np.array_equal(orp, rp) and np.array_equal(oci, ci) and np.array_equal(osv, sv)


@pytest.mark.parametrize("parts", [1, 3, 64, 1000])
def test_dispatch_equals_reference(oracle, ref, parts):
    d = Dataset(4, 4, 0.001)  # power-law row lengths
    assert np.array_equal(ref.dispatch(d.M, d.N, d.row_ptr, d.col_idx, parts), oracle.dispatch(d.M, d.row_ptr, parts))


def test_equality_rule_matches_reference(oracle, ref):
    d = Dataset(uniform=(40, 40, 300), K=4, seed=3)
    base = np.abs(d.s_val) + 0.5
    for scale in (1.0, 1.0005, 1.002, 0.9985):
        lhs = (base * scale).astype(np.float32)
        assert ref.csr_equal(d.M, d.N, d.row_ptr, d.col_idx, lhs, base) == oracle.values_equal_reference_rule(lhs, base)
