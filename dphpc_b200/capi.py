"""ctypes bindings of the two C-ABI libraries.

`Engine` wraps include/sddmm_b200.h (the CUDA SDDMM engine), `Dataset` wraps
include/sddmm_datasets.h (seeded synthetic inputs).  Nothing here computes: a
missing or unloadable CUDA library raises, there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

PKG = Path(__file__).resolve().parent
import os

ENGINE_LIB = Path(os.environ.get("SDDMM_B200_LIB", PKG / "libsddmm_b200.so"))  # override: A/B-test another build
DATASETS_LIB = PKG / "libsddmm_datasets.so"

FP32, TF32, BF16, FP32_TC = 0, 1, 2, 3
MODES = {"fp32": FP32, "tf32": TF32, "bf16": BF16, "fp32_tc": FP32_TC}
FLAG_NO_DENSE_TILES = 1
FLAG_NO_ROW_GROUPS = 2
FLAG_NO_ROW_SEGMENTS = 4
HIST_BINS = 20

STATUS = {
    0: "ok", 1: "bad argument", 2: "bad index", 3: "out of memory", 4: "cuda error", 5: "call order",
    6: "unsupported", 7: "communicator", 8: "device wait ran out",
}

# every symbol include/sddmm_b200.h declares
ENGINE_SYMBOLS = [
    "sddmm_b200_create", "sddmm_b200_destroy", "sddmm_b200_upload_csr", "sddmm_b200_upload_coo",
    "sddmm_b200_upload_csr_device", "sddmm_b200_update_dense", "sddmm_b200_update_values", "sddmm_b200_run",
    "sddmm_b200_sync", "sddmm_b200_download", "sddmm_b200_p_device", "sddmm_b200_last_run_ms", "sddmm_b200_last_kernel_ms",
    "sddmm_b200_get_plan", "sddmm_b200_algorithmic_bytes", "sddmm_b200_flops", "sddmm_b200_last_error",
    "sddmm_b200_stream", "sddmm_b200_device_count", "sddmm_b200_version", "sddmm_b200_host_alloc",
    "sddmm_b200_host_free", "sddmm_b200_sddmm_csr_prealloc", "sddmm_b200_set_kernel_timing",
    "sddmm_b200_pipeline_create", "sddmm_b200_pipeline_destroy", "sddmm_b200_pipeline_sddmm_csr",
    "sddmm_b200_pipeline_last_chunks", "sddmm_b200_pipeline_last_error", "sddmm_b200_pipeline_set_min_chunk_bytes",
    "sddmm_b200_pipeline_update_csr", "sddmm_b200_pipeline_sddmm_coo", "sddmm_b200_set_knob",
    "sddmm_b200_spmm", "sddmm_b200_last_spmm_ms", "sddmm_b200_row_cuts", "sddmm_b200_coo_cuts", "sddmm_b200_upload_coo_rows", "sddmm_b200_stage_b",
    "sddmm_b200_selftest_wait_timeout",
]
DATASET_SYMBOLS = [
    "sddmm_dataset_create", "sddmm_dataset_create_uniform", "sddmm_dataset_destroy", "sddmm_dataset_dims",
    "sddmm_dataset_name", "sddmm_dataset_row_ptr", "sddmm_dataset_col_idx", "sddmm_dataset_s_val",
    "sddmm_dataset_A", "sddmm_dataset_B",
]


class PlanInfo(C.Structure):
    _fields_ = [
        ("rows", C.c_int64), ("cols", C.c_int64), ("k", C.c_int64), ("nnz", C.c_int64),
        ("rows_nonempty", C.c_int64), ("cols_touched", C.c_int64), ("max_row_nnz", C.c_int64),
        ("row_len_hist", C.c_int64 * HIST_BINS),
        ("cols_sorted", C.c_int32), ("mode", C.c_int32),
        ("rowtile_nnz", C.c_int64),
        ("rowtile_items", C.c_int32), ("rowtile_item_nnz", C.c_int32), ("rowtile_rows_per_stage", C.c_int32),
        ("rowtile_grid", C.c_int32), ("rowtile_block", C.c_int32), ("rowtile_smem_bytes", C.c_int32),
        ("dense_nnz", C.c_int64),
        ("dense_tiles", C.c_int32), ("dense_tile_rows", C.c_int32), ("dense_tile_cols", C.c_int32),
        ("dense_grid", C.c_int32), ("dense_block", C.c_int32), ("dense_smem_bytes", C.c_int32),
        ("rowgroup_nnz", C.c_int64),
        ("rowgroup_groups", C.c_int32),
        ("rowgroup_rows", C.c_int32),
        ("rowgroup_grid", C.c_int32),
        ("n_kernels", C.c_int32), ("n_devices", C.c_int32),
        ("rowseg_nnz", C.c_int64),
        ("rowseg_units", C.c_int32), ("rowseg_panels", C.c_int32), ("rowseg_grid", C.c_int32), ("rowseg_passes", C.c_int32),
    ]

    def as_dict(self) -> dict:
        out = {}
        for name, _ in self._fields_:
            v = getattr(self, name)
            out[name] = list(v) if name == "row_len_hist" else int(v)
        return out


class SddmmError(RuntimeError):
    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        super().__init__(f"{where}: status {code} ({STATUS.get(code, '?')}) {detail}".strip())


_engine_lib = None
_dataset_lib = None

_i32p = C.POINTER(C.c_int32)
_f32p = C.POINTER(C.c_float)


def load_engine_lib() -> C.CDLL:
    """Load libsddmm_b200.so (raises if it has not been built)."""
    global _engine_lib
    if _engine_lib is not None:
        return _engine_lib
    if not ENGINE_LIB.exists():
        raise RuntimeError(f"{ENGINE_LIB} is missing: run `python -m dphpc_b200.build` (needs nvcc)")
    lib = C.CDLL(str(ENGINE_LIB))
    H = C.c_void_p
    lib.sddmm_b200_create.argtypes = [C.POINTER(H), C.c_int, C.c_int, C.c_uint32]
    lib.sddmm_b200_destroy.argtypes = [H]
    lib.sddmm_b200_upload_csr.argtypes = [H, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 5
    lib.sddmm_b200_upload_coo.argtypes = [H, C.c_int64, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 5
    lib.sddmm_b200_upload_csr_device.argtypes = [H, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 5
    lib.sddmm_b200_update_dense.argtypes = [H, C.c_void_p, C.c_void_p]
    lib.sddmm_b200_update_values.argtypes = [H, C.c_void_p]
    lib.sddmm_b200_run.argtypes = [H]
    lib.sddmm_b200_sync.argtypes = [H]
    lib.sddmm_b200_download.argtypes = [H, C.c_void_p]
    lib.sddmm_b200_p_device.argtypes = [H, C.POINTER(C.c_void_p)]
    lib.sddmm_b200_last_run_ms.argtypes = [H, C.POINTER(C.c_float)]
    lib.sddmm_b200_last_kernel_ms.argtypes = [H, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_char_p)]
    lib.sddmm_b200_set_kernel_timing.argtypes = [H, C.c_int]
    lib.sddmm_b200_get_plan.argtypes = [H, C.POINTER(PlanInfo)]
    lib.sddmm_b200_set_knob.argtypes = [H, C.c_char_p, C.c_double]
    lib.sddmm_b200_spmm.argtypes = [H, C.c_int64, C.c_void_p, C.c_void_p]
    lib.sddmm_b200_selftest_wait_timeout.argtypes = [H, C.c_int]
    lib.sddmm_b200_row_cuts.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_int64, C.c_void_p]
    lib.sddmm_b200_coo_cuts.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int64, C.c_void_p, C.c_void_p]
    lib.sddmm_b200_upload_coo_rows.argtypes = [H, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 5
    lib.sddmm_b200_stage_b.argtypes = [C.POINTER(H), C.c_int, C.c_int64, C.c_int64, C.c_void_p]
    lib.sddmm_b200_last_spmm_ms.argtypes = [H, C.POINTER(C.c_float)]
    lib.sddmm_b200_algorithmic_bytes.argtypes = [H]
    lib.sddmm_b200_algorithmic_bytes.restype = C.c_int64
    lib.sddmm_b200_flops.argtypes = [H]
    lib.sddmm_b200_flops.restype = C.c_int64
    lib.sddmm_b200_last_error.argtypes = [H]
    lib.sddmm_b200_last_error.restype = C.c_char_p
    lib.sddmm_b200_stream.argtypes = [H]
    lib.sddmm_b200_stream.restype = C.c_void_p
    lib.sddmm_b200_device_count.restype = C.c_int
    lib.sddmm_b200_version.restype = C.c_char_p
    lib.sddmm_b200_host_alloc.argtypes = [C.POINTER(C.c_void_p), C.c_int64]
    lib.sddmm_b200_host_free.argtypes = [C.c_void_p]
    lib.sddmm_b200_sddmm_csr_prealloc.argtypes = [C.c_int, C.c_void_p] + [C.c_int64] * 4 + [C.c_void_p] * 6
    lib.sddmm_b200_pipeline_create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_uint32, C.c_int]
    lib.sddmm_b200_pipeline_destroy.argtypes = [H]
    lib.sddmm_b200_pipeline_sddmm_csr.argtypes = [H, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 6
    lib.sddmm_b200_pipeline_sddmm_coo.argtypes = [H, C.c_int64, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 6
    lib.sddmm_b200_pipeline_update_csr.argtypes = [H] + [C.c_void_p] * 4
    lib.sddmm_b200_pipeline_last_chunks.argtypes = [H]
    lib.sddmm_b200_pipeline_set_min_chunk_bytes.argtypes = [H, C.c_int64]
    lib.sddmm_b200_pipeline_last_error.argtypes = [H]
    lib.sddmm_b200_pipeline_last_error.restype = C.c_char_p
    _engine_lib = lib
    return lib


def load_dataset_lib() -> C.CDLL:
    global _dataset_lib
    if _dataset_lib is not None:
        return _dataset_lib
    if not DATASETS_LIB.exists():
        raise RuntimeError(f"{DATASETS_LIB} is missing: run `python -m dphpc_b200.build`")
    lib = C.CDLL(str(DATASETS_LIB))
    H = C.c_void_p
    lib.sddmm_dataset_create.argtypes = [C.POINTER(H), C.c_int, C.c_int64, C.c_double, C.c_uint64, C.c_int]
    lib.sddmm_dataset_create_uniform.argtypes = [C.POINTER(H), C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_uint64]
    lib.sddmm_dataset_destroy.argtypes = [H]
    lib.sddmm_dataset_destroy.restype = None
    lib.sddmm_dataset_dims.argtypes = [H] + [C.POINTER(C.c_int64)] * 4
    lib.sddmm_dataset_dims.restype = None
    lib.sddmm_dataset_name.argtypes = [H]
    lib.sddmm_dataset_name.restype = C.c_char_p
    for fn, ty in (("row_ptr", _i32p), ("col_idx", _i32p), ("s_val", _f32p), ("A", _f32p), ("B", _f32p)):
        f = getattr(lib, f"sddmm_dataset_{fn}")
        f.argtypes = [H]
        f.restype = ty
    _dataset_lib = lib
    return lib


def _ptr(a) -> C.c_void_p:
    """Host pointer of a contiguous numpy array, or an int device/host address."""
    if a is None:
        return C.c_void_p(0)
    if isinstance(a, (int, np.integer)):
        return C.c_void_p(int(a))
    assert a.flags["C_CONTIGUOUS"], "array must be C-contiguous"
    return C.c_void_p(a.ctypes.data)


def _as(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


class Engine:
    """One SDDMM engine on one CUDA device (see include/sddmm_b200.h)."""

    def __init__(self, device: int = 0, mode="fp32", flags: int = 0):
        self.lib = load_engine_lib()
        self.h = C.c_void_p()
        m = MODES[mode] if isinstance(mode, str) else int(mode)
        st = self.lib.sddmm_b200_create(C.byref(self.h), int(device), m, int(flags))
        if st:
            self.h = C.c_void_p()
            raise SddmmError(st, "sddmm_b200_create", "(no usable CUDA device?)" if st == 4 else "")
        self.nnz = 0
        self._keep = None

    # -- helpers
    def _check(self, st: int, where: str):
        if st:
            raise SddmmError(st, where, self.lib.sddmm_b200_last_error(self.h).decode())

    def close(self):
        if getattr(self, "h", None) and self.h.value:
            self.lib.sddmm_b200_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- API
    def upload_csr(self, M, N, K, row_ptr, col_idx, s_val, A, B):
        row_ptr, col_idx = _as(row_ptr, np.int32), _as(col_idx, np.int32)
        s_val, A, B = _as(s_val, np.float32), _as(A, np.float32), _as(B, np.float32)
        assert row_ptr.size == M + 1 and A.size == M * K and B.size == N * K
        self._check(self.lib.sddmm_b200_upload_csr(self.h, M, N, K, _ptr(row_ptr), _ptr(col_idx), _ptr(s_val), _ptr(A), _ptr(B)),
                    "upload_csr")
        self.nnz = int(row_ptr[M])

    def upload_csr_raw(self, M, N, K, row_ptr, col_idx, s_val, A, B):
        """Host pointers given as integers (e.g. pinned buffers); no conversion, no size check."""
        self._check(self.lib.sddmm_b200_upload_csr(self.h, M, N, K, _ptr(row_ptr), _ptr(col_idx), _ptr(s_val), _ptr(A), _ptr(B)),
                    "upload_csr")

    def upload_coo(self, M, N, K, row_idx, col_idx, s_val, A, B):
        row_idx, col_idx = _as(row_idx, np.int32), _as(col_idx, np.int32)
        s_val, A, B = _as(s_val, np.float32), _as(A, np.float32), _as(B, np.float32)
        assert row_idx.size == col_idx.size == s_val.size
        self._check(self.lib.sddmm_b200_upload_coo(self.h, M, N, K, row_idx.size, _ptr(row_idx), _ptr(col_idx), _ptr(s_val),
                                                   _ptr(A), _ptr(B)), "upload_coo")
        self.nnz = int(row_idx.size)

    def upload_coo_rows(self, M, N, K, row_base, row_idx, col_idx, s_val, A, B):
        """Rows [row_base, row_base + M) of a larger COO matrix; row_idx keeps the matrix' own row numbers."""
        row_idx, col_idx = _as(row_idx, np.int32), _as(col_idx, np.int32)
        s_val, A, B = _as(s_val, np.float32), _as(A, np.float32), _as(B, np.float32)
        assert row_idx.size == col_idx.size == s_val.size
        self._check(self.lib.sddmm_b200_upload_coo_rows(self.h, M, N, K, row_idx.size, int(row_base), _ptr(row_idx), _ptr(col_idx),
                                                        _ptr(s_val), _ptr(A), _ptr(B)), "upload_coo_rows")
        self.nnz = int(row_idx.size)

    def upload_csr_device(self, M, N, K, nnz, row_ptr, col_idx, s_val, A, B):
        """All five arguments are device addresses (ints) on this engine's device."""
        self._check(self.lib.sddmm_b200_upload_csr_device(self.h, M, N, K, _ptr(row_ptr), _ptr(col_idx), _ptr(s_val), _ptr(A),
                                                          _ptr(B)), "upload_csr_device")
        self.nnz = int(nnz)

    def update_dense(self, A=None, B=None):
        A = None if A is None else _as(A, np.float32)
        B = None if B is None else _as(B, np.float32)
        self._check(self.lib.sddmm_b200_update_dense(self.h, _ptr(A), _ptr(B)), "update_dense")

    def update_values(self, s_val):
        self._check(self.lib.sddmm_b200_update_values(self.h, _ptr(_as(s_val, np.float32))), "update_values")

    def update_raw(self, A=None, B=None, s_val=None):
        """update_dense / update_values with host pointers given as integers (e.g. pinned buffers)."""
        if A is not None or B is not None:
            self._check(self.lib.sddmm_b200_update_dense(self.h, _ptr(A), _ptr(B)), "update_dense")
        if s_val is not None:
            self._check(self.lib.sddmm_b200_update_values(self.h, _ptr(s_val)), "update_values")

    def run(self):
        self._check(self.lib.sddmm_b200_run(self.h), "run")

    def sync(self):
        self._check(self.lib.sddmm_b200_sync(self.h), "sync")

    def download(self, out=None) -> np.ndarray:
        if out is None:
            out = np.empty(self.nnz, dtype=np.float32)
        self._check(self.lib.sddmm_b200_download(self.h, _ptr(out)), "download")
        return out

    def download_raw(self, host_ptr: int):
        self._check(self.lib.sddmm_b200_download(self.h, _ptr(host_ptr)), "download")

    def p_device(self) -> int:
        p = C.c_void_p()
        self._check(self.lib.sddmm_b200_p_device(self.h, C.byref(p)), "p_device")
        return int(p.value or 0)

    def last_run_ms(self) -> float:
        ms = C.c_float()
        self._check(self.lib.sddmm_b200_last_run_ms(self.h, C.byref(ms)), "last_run_ms")
        return float(ms.value)

    def set_kernel_timing(self, enabled: bool = True):
        """Record an event pair around every kernel of the following run() calls (costs microseconds per launch)."""
        self._check(self.lib.sddmm_b200_set_kernel_timing(self.h, 1 if enabled else 0), "set_kernel_timing")

    def kernel_times(self) -> list:
        """[(kernel name, device ms)] of the last run(); ms is -1 unless set_kernel_timing(True) was in effect."""
        out = []
        for i in range(self.plan()["n_kernels"]):
            ms, name = C.c_float(), C.c_char_p()
            self._check(self.lib.sddmm_b200_last_kernel_ms(self.h, i, C.byref(ms), C.byref(name)), "last_kernel_ms")
            out.append(((name.value or b"?").decode(), float(ms.value)))
        return out

    def spmm(self, X, out=None, rows: int | None = None) -> np.ndarray:
        """Y = P X for the P of the last run(), computed on the device (P.val is not downloaded).  X: N x K2."""
        pl = self.plan() if (X is None or rows is None) else None
        X = None if X is None else _as(X, np.float32)   # None: X = B, the engine's own copy
        K2 = int(pl["k"]) if X is None else X.shape[1]
        M = int(rows if rows is not None else pl["rows"])
        if out is None:
            out = np.empty((M, K2), dtype=np.float32)
        self._check(self.lib.sddmm_b200_spmm(self.h, K2, _ptr(X), _ptr(out)), "spmm")
        return out

    def spmm_raw(self, K2: int, x_ptr: int, y_ptr: int):
        self._check(self.lib.sddmm_b200_spmm(self.h, int(K2), _ptr(x_ptr), _ptr(y_ptr)), "spmm")

    def last_spmm_ms(self) -> float:
        ms = C.c_float()
        self._check(self.lib.sddmm_b200_last_spmm_ms(self.h, C.byref(ms)), "last_spmm_ms")
        return float(ms.value)

    def set_knob(self, name: str, value: float):
        """Planner knob (see sddmm_b200_set_knob); a negative value hands the decision back to the planner."""
        self._check(self.lib.sddmm_b200_set_knob(self.h, name.encode(), float(value)), "set_knob")

    def plan(self) -> dict:
        info = PlanInfo()
        self._check(self.lib.sddmm_b200_get_plan(self.h, C.byref(info)), "get_plan")
        return info.as_dict()

    def algorithmic_bytes(self) -> int:
        return int(self.lib.sddmm_b200_algorithmic_bytes(self.h))

    def flops(self) -> int:
        return int(self.lib.sddmm_b200_flops(self.h))

    def stream(self) -> int:
        return int(self.lib.sddmm_b200_stream(self.h) or 0)

    def sddmm_csr(self, M, N, K, row_ptr, col_idx, s_val, A, B) -> np.ndarray:
        """upload -> run -> download, the init/run/cleanup sequence of one competitor call."""
        self.upload_csr(M, N, K, row_ptr, col_idx, s_val, A, B)
        self.run()
        return self.download()

    def sddmm_coo(self, M, N, K, row_idx, col_idx, s_val, A, B) -> np.ndarray:
        self.upload_coo(M, N, K, row_idx, col_idx, s_val, A, B)
        self.run()
        return self.download()


class Pipeline:
    """Chunked host-to-host SDDMM on one device (sddmm_b200_pipeline_* in include/sddmm_b200.h): upload, run and
    download of consecutive row chunks overlapped."""

    def __init__(self, device: int = 0, mode="fp32", flags: int = 0, chunks: int = 4, min_chunk_bytes: int | None = None):
        self.lib = load_engine_lib()
        self.h = C.c_void_p()
        m = MODES[mode] if isinstance(mode, str) else int(mode)
        st = self.lib.sddmm_b200_pipeline_create(C.byref(self.h), int(device), m, int(flags), int(chunks))
        if st:
            self.h = C.c_void_p()
            raise SddmmError(st, "sddmm_b200_pipeline_create", "(no usable CUDA device?)" if st == 4 else "")
        if min_chunk_bytes is not None and self.lib.sddmm_b200_pipeline_set_min_chunk_bytes(self.h, int(min_chunk_bytes)):
            raise SddmmError(1, "sddmm_b200_pipeline_set_min_chunk_bytes")

    def close(self):
        if getattr(self, "h", None) and self.h.value:
            self.lib.sddmm_b200_pipeline_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def sddmm_csr_raw(self, M, N, K, row_ptr, col_idx, s_val, A, B, p_val):
        """Host pointers given as integers (e.g. pinned buffers); no conversion, no size check."""
        st = self.lib.sddmm_b200_pipeline_sddmm_csr(self.h, M, N, K, _ptr(row_ptr), _ptr(col_idx), _ptr(s_val), _ptr(A), _ptr(B),
                                                    _ptr(p_val))
        if st:
            raise SddmmError(st, "pipeline_sddmm_csr", self.lib.sddmm_b200_pipeline_last_error(self.h).decode())

    def sddmm_csr(self, M, N, K, row_ptr, col_idx, s_val, A, B) -> np.ndarray:
        row_ptr, col_idx = _as(row_ptr, np.int32), _as(col_idx, np.int32)
        s_val, A, B = _as(s_val, np.float32), _as(A, np.float32), _as(B, np.float32)
        assert row_ptr.size == M + 1 and A.size == M * K and B.size == N * K
        out = np.empty(int(row_ptr[M]) if row_ptr[M] > 0 else 0, dtype=np.float32)
        self.sddmm_csr_raw(M, N, K, row_ptr, col_idx, s_val, A, B, out)
        return out

    def sddmm_coo(self, M, N, K, row_idx, col_idx, s_val, A, B) -> np.ndarray:
        row_idx, col_idx = _as(row_idx, np.int32), _as(col_idx, np.int32)
        s_val, A, B = _as(s_val, np.float32), _as(A, np.float32), _as(B, np.float32)
        assert row_idx.size == col_idx.size == s_val.size and A.size == M * K and B.size == N * K
        out = np.empty(row_idx.size, dtype=np.float32)
        st = self.lib.sddmm_b200_pipeline_sddmm_coo(self.h, M, N, K, row_idx.size, _ptr(row_idx), _ptr(col_idx), _ptr(s_val), _ptr(A),
                                                    _ptr(B), _ptr(out))
        if st:
            raise SddmmError(st, "pipeline_sddmm_coo", self.lib.sddmm_b200_pipeline_last_error(self.h).decode())
        return out

    def update_csr_raw(self, s_val, A, B, p_val):
        """New S.val, A, B for the pattern of the last sddmm_csr call; host arrays or addresses, result into p_val."""
        st = self.lib.sddmm_b200_pipeline_update_csr(self.h, _ptr(s_val), _ptr(A), _ptr(B), _ptr(p_val))
        if st:
            raise SddmmError(st, "pipeline_update_csr", self.lib.sddmm_b200_pipeline_last_error(self.h).decode())

    def last_chunks(self) -> int:
        return int(self.lib.sddmm_b200_pipeline_last_chunks(self.h))


def device_count() -> int:
    return int(load_engine_lib().sddmm_b200_device_count())


class Dataset:
    """Seeded synthetic SDDMM input (see include/sddmm_datasets.h). Arrays are views into native memory."""

    def __init__(self, config: int | None = None, K: int = 32, scale: float = 1.0, seed: int | None = None, variant: int = 0,
                 uniform: tuple | None = None):
        self.lib = load_dataset_lib()
        self.h = C.c_void_p()
        if uniform is not None:
            M, N, nnz = uniform
            self.seed = 0x5DD0 if seed is None else seed
            st = self.lib.sddmm_dataset_create_uniform(C.byref(self.h), M, N, K, nnz, self.seed)
        else:
            self.seed = (0x5DD0 + config) if seed is None else seed
            st = self.lib.sddmm_dataset_create(C.byref(self.h), config, K, float(scale), self.seed, variant)
        if st:
            raise RuntimeError(f"dataset generation failed (status {st})")
        m, n, k, z = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64()
        self.lib.sddmm_dataset_dims(self.h, C.byref(m), C.byref(n), C.byref(k), C.byref(z))
        self.M, self.N, self.K, self.nnz = m.value, n.value, k.value, z.value
        self.name = self.lib.sddmm_dataset_name(self.h).decode()
        self.config = config

        def view(ptr, n, dtype):
            if n == 0:
                return np.zeros(0, dtype=dtype)
            return np.ctypeslib.as_array(ptr, shape=(n,))

        self.row_ptr = view(self.lib.sddmm_dataset_row_ptr(self.h), self.M + 1, np.int32)
        self.col_idx = view(self.lib.sddmm_dataset_col_idx(self.h), self.nnz, np.int32)
        self.s_val = view(self.lib.sddmm_dataset_s_val(self.h), self.nnz, np.float32)
        self.A = view(self.lib.sddmm_dataset_A(self.h), self.M * self.K, np.float32).reshape(self.M, self.K)
        self.B = view(self.lib.sddmm_dataset_B(self.h), self.N * self.K, np.float32).reshape(self.N, self.K)

    def row_idx(self) -> np.ndarray:
        """COO row indices (what COO<T>(CSR<T>&) of the reference expands, src/matrices/COO.hpp:55-74)."""
        return np.repeat(np.arange(self.M, dtype=np.int32), np.diff(self.row_ptr)).astype(np.int32)

    def close(self):
        if getattr(self, "h", None) and self.h.value:
            for name in ("row_ptr", "col_idx", "s_val", "A", "B"):
                setattr(self, name, None)
            self.lib.sddmm_dataset_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
