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
    """parts+1 row indices, cut[0] = 0, cut[parts] = M, non-decreasing.

    align > 1 moves every inner cut to the nearest multiple of `align` rows: with align = 64 the 64x64
    tiles of each shard coincide with those of the whole matrix, so a block that is dense globally is
    still one dense tile locally (the tensor-core path looks at aligned tiles of what it is given)."""
    row_ptr = np.asarray(row_ptr)
    M = row_ptr.size - 1
    nnz = int(row_ptr[M])
    targets = (np.arange(1, parts, dtype=np.int64) * nnz) // parts
    hi = np.minimum(np.searchsorted(row_ptr, targets, side="left").astype(np.int64), M)   # first boundary at or past the target
    lo = np.maximum(hi - 1, 0)
    rp = row_ptr.astype(np.int64)
    inner = np.where(targets - rp[lo] < rp[hi] - targets, lo, hi)                          # the closer row boundary wins
    if align > 1:
        inner = np.minimum((inner + align // 2) // align * align, M)
    cuts = np.concatenate(([0], inner, [M]))
    return np.maximum.accumulate(cuts)


def shard(row_ptr, col_idx, s_val, A, rank: int, parts: int, align: int = 1):
    """(row0, row1, rebased row_ptr, col slice, val slice, A slice) of one rank; views where possible."""
    cuts = row_cuts(row_ptr, parts, align)
    r0, r1 = int(cuts[rank]), int(cuts[rank + 1])
    a, b = int(row_ptr[r0]), int(row_ptr[r1])
    rp = (np.asarray(row_ptr[r0:r1 + 1], dtype=np.int64) - a).astype(np.int32)
    return r0, r1, rp, col_idx[a:b], s_val[a:b], A[r0:r1]
