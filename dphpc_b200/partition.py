"""nnz-balanced contiguous row ranges for sharding S across GPUs.

Every output nonzero depends on one A row, one B row and one S value, so the
SDDMM shards by row ranges with no exchange in the compute step: rank g gets
rows [cut[g], cut[g+1]), the matching slices of col_idx / S.val / A, and all of B.
The cut points are the row boundaries closest to g * nnz / G -- the same
"equal nonzeros per worker" goal as the reference's per-thread dispatcher
(CSR<T>::_dispatch, src/matrices/CSR.hpp:214-264), computed by one binary search
per cut instead of a search over segment capacities.
"""
from __future__ import annotations

import numpy as np


def row_cuts(row_ptr: np.ndarray, parts: int, align: int = 1) -> np.ndarray:
    """parts+1 row indices, cut[0] = 0, cut[parts] = M, non-decreasing (sddmm_b200_row_cuts of the C ABI: the one
    definition the chunked call, the multi-device competitor and the one-process-per-GPU bench share).

    align > 1 moves every inner cut to the nearest multiple of `align` rows: with align = 64 the 64x64
    tiles of each shard coincide with those of the whole matrix, so a block that is dense globally is
    still one dense tile locally (the tensor-core path looks at aligned tiles of what it is given)."""
    import ctypes as C

    from .capi import load_engine_lib

    rp = np.ascontiguousarray(row_ptr, dtype=np.int32)
    cuts = np.zeros(parts + 1, dtype=np.int64)
    st = load_engine_lib().sddmm_b200_row_cuts(C.c_void_p(rp.ctypes.data), C.c_int64(rp.size - 1), C.c_int(parts), C.c_int64(align),
                                               C.c_void_p(cuts.ctypes.data))
    if st:
        raise ValueError(f"sddmm_b200_row_cuts: status {st}")
    return cuts


def coo_cuts(row_idx: np.ndarray, M: int, parts: int, align: int = 1):
    """(cuts, offsets) of a COO row array sorted by row (sddmm_b200_coo_cuts): part g holds rows [cuts[g], cuts[g+1]) =
    entries [offsets[g], offsets[g+1]); no row_ptr is built."""
    import ctypes as C

    from .capi import load_engine_lib

    rows = np.ascontiguousarray(row_idx, dtype=np.int32)
    cuts = np.zeros(parts + 1, dtype=np.int64)
    offs = np.zeros(parts + 1, dtype=np.int64)
    st = load_engine_lib().sddmm_b200_coo_cuts(C.c_void_p(rows.ctypes.data), C.c_int64(rows.size), C.c_int64(M), C.c_int(parts),
                                               C.c_int64(align), C.c_void_p(cuts.ctypes.data), C.c_void_p(offs.ctypes.data))
    if st:
        raise ValueError(f"sddmm_b200_coo_cuts: status {st}")
    return cuts, offs


def shard(row_ptr, col_idx, s_val, A, rank: int, parts: int, align: int = 1):
    """(row0, row1, rebased row_ptr, col slice, val slice, A slice) of one rank; views where possible."""
    cuts = row_cuts(row_ptr, parts, align)
    r0, r1 = int(cuts[rank]), int(cuts[rank + 1])
    a, b = int(row_ptr[r0]), int(row_ptr[r1])
    rp = (np.asarray(row_ptr[r0:r1 + 1], dtype=np.int64) - a).astype(np.int32)
    return r0, r1, rp, col_idx[a:b], s_val[a:b], A[r0:r1]
