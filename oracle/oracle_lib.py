"""ctypes access to the CPU checkers under oracle/ (tests, smoke and bench baselines only)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_LIB = ROOT / "oracle" / "liboracle.so"
REF_LIB = ROOT / "oracle" / "_ref" / "libsddmm_ref.so"

_vp = C.c_void_p


def _p(a):
    return _vp(a.ctypes.data)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    """oracle/sddmm_oracle.c: restatement of CPUBasic, CSR/COO construction and the dispatcher."""

    def __init__(self):
        self.lib = C.CDLL(str(ORACLE_LIB))
        L = self.lib
        L.oracle_sddmm_csr.argtypes = [C.c_int32, C.c_int32] + [_vp] * 6
        L.oracle_sddmm_csr.restype = None
        L.oracle_sddmm_coo.argtypes = [C.c_int64, C.c_int32] + [_vp] * 6
        L.oracle_sddmm_coo.restype = None
        L.oracle_sddmm_csr_rows.argtypes = [C.c_int32, C.c_int32, C.c_int32] + [_vp] * 6
        L.oracle_sddmm_csr_rows.restype = None
        L.oracle_spmm_csr_rows.argtypes = [C.c_int32, C.c_int32, C.c_int32] + [_vp] * 5
        L.oracle_spmm_csr_rows.restype = None
        L.oracle_sort_unique_triplets.argtypes = [C.c_int64] + [_vp] * 6
        L.oracle_sort_unique_triplets.restype = C.c_int64
        L.oracle_coo_rows_to_row_ptr.argtypes = [C.c_int32, C.c_int64, _vp, _vp]
        L.oracle_coo_rows_to_row_ptr.restype = None
        L.oracle_row_ptr_to_coo_rows.argtypes = [C.c_int32, _vp, _vp]
        L.oracle_row_ptr_to_coo_rows.restype = None
        L.oracle_dispatch.argtypes = [C.c_int32, _vp, C.c_int32, C.c_int32, _vp]
        L.oracle_dispatch.restype = C.c_int64
        L.oracle_values_equal_reference_rule.argtypes = [C.c_int64, _vp, _vp]
        L.oracle_values_equal_reference_rule.restype = C.c_int

    def sddmm_csr(self, M, K, row_ptr, col_idx, s_val, A, B):
        row_ptr, col_idx, s_val, A, B = _i32(row_ptr), _i32(col_idx), _f32(s_val), _f32(A), _f32(B)
        out = np.empty(int(row_ptr[M]), dtype=np.float32)
        self.lib.oracle_sddmm_csr(M, K, _p(row_ptr), _p(col_idx), _p(s_val), _p(A), _p(B), _p(out))
        return out

    def sddmm_csr_rows(self, r0, r1, K, row_ptr, col_idx, s_val, A, B, out):
        self.lib.oracle_sddmm_csr_rows(r0, r1, K, _p(row_ptr), _p(col_idx), _p(s_val), _p(A), _p(B), _p(out))

    def spmm_csr(self, M, K2, row_ptr, col_idx, p_val, X):
        """Y = P X, the consumer of the SDDMM result (plain CSR loop, fp32)."""
        row_ptr, col_idx, p_val, X = _i32(row_ptr), _i32(col_idx), _f32(p_val), _f32(X)
        Y = np.empty((M, K2), dtype=np.float32)
        self.lib.oracle_spmm_csr_rows(0, M, K2, _p(row_ptr), _p(col_idx), _p(p_val), _p(X), _p(Y))
        return Y

    def sddmm_coo(self, K, row_idx, col_idx, s_val, A, B):
        row_idx, col_idx, s_val, A, B = _i32(row_idx), _i32(col_idx), _f32(s_val), _f32(A), _f32(B)
        out = np.empty(row_idx.size, dtype=np.float32)
        self.lib.oracle_sddmm_coo(row_idx.size, K, _p(row_idx), _p(col_idx), _p(s_val), _p(A), _p(B), _p(out))
        return out

    def sort_unique(self, rows, cols, vals):
        rows, cols, vals = _i32(rows), _i32(cols), _f32(vals)
        n = rows.size
        orow, ocol, oval = np.empty(n, np.int32), np.empty(n, np.int32), np.empty(n, np.float32)
        m = self.lib.oracle_sort_unique_triplets(n, _p(rows), _p(cols), _p(vals), _p(orow), _p(ocol), _p(oval))
        return orow[:m].copy(), ocol[:m].copy(), oval[:m].copy()

    def csr_from_triplets(self, M, rows, cols, vals):
        r, c, v = self.sort_unique(rows, cols, vals)
        rp = np.empty(M + 1, np.int32)
        self.lib.oracle_coo_rows_to_row_ptr(M, r.size, _p(r), _p(rp))
        return rp, c, v

    def coo_rows(self, M, row_ptr):
        row_ptr = _i32(row_ptr)
        out = np.empty(int(row_ptr[M]), np.int32)
        self.lib.oracle_row_ptr_to_coo_rows(M, _p(row_ptr), _p(out))
        return out

    def dispatch(self, M, row_ptr, parts, stride=1):
        row_ptr = _i32(row_ptr)
        out = np.empty(max(parts, M // stride + 1) + 2, np.int32)
        n = self.lib.oracle_dispatch(M, _p(row_ptr), parts, stride, _p(out))
        return out[:n].copy()

    def values_equal_reference_rule(self, lhs, rhs) -> bool:
        lhs, rhs = _f32(lhs), _f32(rhs)
        return bool(self.lib.oracle_values_equal_reference_rule(lhs.size, _p(lhs), _p(rhs)))


class Reference:
    """oracle/_ref: the reference's own headers compiled unmodified (oracle/ref_shim.cpp)."""

    @staticmethod
    def try_load():
        if not REF_LIB.exists():
            return None
        try:
            return Reference()
        except OSError:
            return None

    def __init__(self):
        self.lib = C.CDLL(str(REF_LIB))
        L = self.lib
        L.ref_csr_from_triplets.argtypes = [C.c_int32, C.c_int32, C.c_int64] + [_vp] * 6
        L.ref_csr_from_triplets.restype = C.c_int64
        L.ref_coo_from_triplets.argtypes = [C.c_int32, C.c_int32, C.c_int64] + [_vp] * 6
        L.ref_coo_from_triplets.restype = C.c_int64
        L.ref_cpu_basic_csr.argtypes = [C.c_int32, C.c_int32, C.c_int32] + [_vp] * 6
        L.ref_cpu_basic_csr.restype = C.c_int64
        L.ref_cpu_basic_coo.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int64] + [_vp] * 6
        L.ref_cpu_basic_coo.restype = C.c_int64
        L.ref_dispatch.argtypes = [C.c_int32, C.c_int32, _vp, _vp, C.c_int32, C.c_int32, _vp, C.c_int64]
        L.ref_dispatch.restype = C.c_int64
        L.ref_csr_equal.argtypes = [C.c_int32, C.c_int32] + [_vp] * 4
        L.ref_csr_equal.restype = C.c_int
        L.ref_problem_create.argtypes = [C.c_int32, C.c_int32, C.c_int32] + [_vp] * 5
        L.ref_problem_create.restype = _vp
        L.ref_problem_run.argtypes = [_vp]
        L.ref_problem_run.restype = C.c_int64
        L.ref_problem_result.argtypes = [_vp, _vp]
        L.ref_problem_result.restype = None
        L.ref_problem_destroy.argtypes = [_vp]
        L.ref_problem_destroy.restype = None

    def problem(self, M, N, K, row_ptr, col_idx, s_val, A, B):
        """Build the reference's objects once; returns (run() -> ns, result() -> P.val, destroy())."""
        row_ptr, col_idx, s_val, A, B = _i32(row_ptr), _i32(col_idx), _f32(s_val), _f32(A), _f32(B)
        h = self.lib.ref_problem_create(M, N, K, _p(row_ptr), _p(col_idx), _p(s_val), _p(A), _p(B))
        if not h:
            raise ValueError("the reference's CSR constructor dropped entries")
        nnz = int(row_ptr[M])

        def result():
            out = np.empty(nnz, np.float32)
            self.lib.ref_problem_result(h, _p(out))
            return out

        return (lambda: int(self.lib.ref_problem_run(h))), result, (lambda: self.lib.ref_problem_destroy(h))

    def csr_from_triplets(self, M, N, rows, cols, vals):
        rows, cols, vals = _i32(rows), _i32(cols), _f32(vals)
        n = rows.size
        rp, c, v = np.empty(M + 1, np.int32), np.empty(n, np.int32), np.empty(n, np.float32)
        m = self.lib.ref_csr_from_triplets(M, N, n, _p(rows), _p(cols), _p(vals), _p(rp), _p(c), _p(v))
        return rp, c[:m].copy(), v[:m].copy()

    def coo_from_triplets(self, M, N, rows, cols, vals):
        rows, cols, vals = _i32(rows), _i32(cols), _f32(vals)
        n = rows.size
        r, c, v = np.empty(n, np.int32), np.empty(n, np.int32), np.empty(n, np.float32)
        m = self.lib.ref_coo_from_triplets(M, N, n, _p(rows), _p(cols), _p(vals), _p(r), _p(c), _p(v))
        return r[:m].copy(), c[:m].copy(), v[:m].copy()

    def cpu_basic_csr(self, M, N, K, row_ptr, col_idx, s_val, A, B, return_ns=False):
        row_ptr, col_idx, s_val, A, B = _i32(row_ptr), _i32(col_idx), _f32(s_val), _f32(A), _f32(B)
        out = np.empty(int(row_ptr[M]), np.float32)
        ns = self.lib.ref_cpu_basic_csr(M, N, K, _p(row_ptr), _p(col_idx), _p(s_val), _p(A), _p(B), _p(out))
        if ns < 0:
            raise ValueError("the reference's CSR constructor dropped entries (duplicate positions in the input)")
        return (out, ns) if return_ns else out

    def cpu_basic_coo(self, M, N, K, row_idx, col_idx, s_val, A, B):
        row_idx, col_idx, s_val, A, B = _i32(row_idx), _i32(col_idx), _f32(s_val), _f32(A), _f32(B)
        out = np.empty(row_idx.size, np.float32)
        ns = self.lib.ref_cpu_basic_coo(M, N, K, row_idx.size, _p(row_idx), _p(col_idx), _p(s_val), _p(A), _p(B), _p(out))
        if ns < 0:
            raise ValueError("the reference's COO constructor dropped entries")
        return out

    def dispatch(self, M, N, row_ptr, col_idx, parts, tensor=False):
        row_ptr, col_idx = _i32(row_ptr), _i32(col_idx)
        cap = max(parts, M) + 8
        out = np.empty(cap, np.int32)
        n = self.lib.ref_dispatch(M, N, _p(row_ptr), _p(col_idx), parts, 1 if tensor else 0, _p(out), cap)
        return out[:n].copy()

    def csr_equal(self, M, N, row_ptr, col_idx, lhs, rhs) -> bool:
        row_ptr, col_idx, lhs, rhs = _i32(row_ptr), _i32(col_idx), _f32(lhs), _f32(rhs)
        return bool(self.lib.ref_csr_equal(M, N, _p(row_ptr), _p(col_idx), _p(lhs), _p(rhs)))


def abs_dot_bound(row_idx, col_idx, s_val, A, B, chunk=1 << 20):
    """|s_ij| * sum_k |a_ik * b_jk| per nonzero, float64: the scale relative error is measured against."""
    A64, B64 = np.abs(np.asarray(A, np.float64)), np.abs(np.asarray(B, np.float64))
    out = np.empty(len(col_idx), np.float64)
    for a in range(0, len(col_idx), chunk):
        b = min(len(col_idx), a + chunk)
        out[a:b] = np.einsum("ik,ik->i", A64[row_idx[a:b]], B64[col_idx[a:b]]) * np.abs(s_val[a:b].astype(np.float64))
    return out


def dot_f64(row_idx, col_idx, s_val, A, B, chunk=1 << 20):
    A64, B64 = np.asarray(A, np.float64), np.asarray(B, np.float64)
    out = np.empty(len(col_idx), np.float64)
    for a in range(0, len(col_idx), chunk):
        b = min(len(col_idx), a + chunk)
        out[a:b] = np.einsum("ik,ik->i", A64[row_idx[a:b]], B64[col_idx[a:b]]) * s_val[a:b].astype(np.float64)
    return out


def assert_values_close(p, p_ref, bound, tol, what=""):
    """|p - p_ref| <= tol * |s| * sum_k|a b|  (relative error made robust to cancellation), plus exact zeros."""
    p = np.asarray(p, np.float64)
    p_ref = np.asarray(p_ref, np.float64)
    assert p.shape == p_ref.shape, f"{what}: shape {p.shape} vs {p_ref.shape}"
    assert np.isfinite(p).all(), f"{what}: non-finite output"
    err = np.abs(p - p_ref)
    lim = tol * bound + 1e-30
    bad = err > lim
    if bad.any():
        i = int(np.argmax(err / np.maximum(lim, 1e-300)))
        raise AssertionError(f"{what}: {int(bad.sum())} of {p.size} values off; worst at {i}: got {p[i]!r} want {p_ref[i]!r} "
                             f"err {err[i]:.3e} limit {lim[i]:.3e}")


def host_threads(limit=32):
    import os
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(limit, n))


def sddmm_csr_all_rows(oracle, M, K, row_ptr, col_idx, s_val, A, B, threads=None):
    """The oracle over EVERY row, the rows cut into nnz-balanced ranges that run on a thread pool (each range is one
    call of the same C loop; ctypes releases the GIL).  Bit-identical to one call over all rows."""
    from concurrent.futures import ThreadPoolExecutor

    row_ptr, col_idx, s_val, A, B = _i32(row_ptr), _i32(col_idx), _f32(s_val), _f32(A), _f32(B)
    nnz = int(row_ptr[M])
    out = np.empty(nnz, np.float32)
    threads = threads or host_threads()
    cuts = np.unique(np.concatenate([[0], np.searchsorted(row_ptr, np.arange(1, threads) * (nnz / threads)), [M]]).astype(np.int64))
    with ThreadPoolExecutor(max_workers=threads) as pool:
        list(pool.map(lambda ab: oracle.sddmm_csr_rows(int(ab[0]), int(ab[1]), K, row_ptr, col_idx, s_val, A, B, out),
                      zip(cuts[:-1], cuts[1:])))
    return out


def abs_dot_bound_all_rows(oracle, M, K, row_ptr, col_idx, s_val, A, B, threads=None):
    """|s_ij| * sum_k |a_ik b_jk| for every nonzero of a CSR matrix: the oracle's own loop on the absolute values
    (fp32 accumulation of non-negative terms: relative error ~K * 2^-24, widened by the factor below)."""
    b = sddmm_csr_all_rows(oracle, M, K, row_ptr, col_idx, np.abs(_f32(s_val)), np.abs(_f32(A)), np.abs(_f32(B)), threads)
    return b.astype(np.float64) * (1.0 + 1e-4)


def abs_dot_bound_rows(row_ptr, col_idx, s_val, A, B, threads=None, chunk=1 << 19):
    """abs_dot_bound for a whole CSR matrix (row indices expanded chunk by chunk, chunks on a thread pool)."""
    from concurrent.futures import ThreadPoolExecutor

    row_ptr = np.asarray(row_ptr, np.int64)
    nnz = int(row_ptr[-1])
    A32, B32 = np.abs(np.asarray(A, np.float32)), np.abs(np.asarray(B, np.float32))
    out = np.empty(nnz, np.float64)

    def work(a):
        b = min(nnz, a + chunk)
        rows = np.searchsorted(row_ptr, np.arange(a, b), side="right") - 1
        prod = np.einsum("ik,ik->i", A32[rows].astype(np.float64), B32[col_idx[a:b]].astype(np.float64))
        out[a:b] = prod * np.abs(np.asarray(s_val[a:b], np.float64))

    with ThreadPoolExecutor(max_workers=threads or host_threads()) as pool:
        list(pool.map(work, range(0, nnz, chunk)))
    return out
