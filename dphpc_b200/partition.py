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


def block_grid(world: int, M: int, N: int, K: int, nnz: int, elem_bytes: int = 4, l2_bytes: int = 126 << 20):
    """(row parts, column parts) of a 2-D block partition over `world` devices, row parts x column parts = world.

    Row shards replicate B: every device gathers from all of it, and when B is larger than L2 most gathers are HBM reads
    whatever the shard size.  Cutting the COLUMNS as well gives each device a slice of B that stays in its L2 -- the
    devices' caches add up -- at the price of shorter runs per row.  Column parts double while the slice of B is larger
    than half the L2 and a row keeps at least three nonzeros per part on average.  Plain row shards stay where that does
    not pay: operands that fit L2; rows short on average (the engine then cuts only their long rows into panels itself);
    rows of A and B longer than 256 bytes, where re-reading A once per column part costs more than the gathers save, and
    bf16 storage, whose kernels are bound by their arithmetic (measured on 4 GPUs, Poisson rows: fp32 K = 32 145 -> 131 us,
    K = 64 285 -> 258 us per step, but K = 128 584 -> 616 us, bf16 K = 64 190 -> 196 us)."""
    import os
    forced = os.environ.get("SDDMM_B200_GRID")   # "RxC": experiments with other grids
    if forced:
        r, c = (int(v) for v in forced.lower().split("x"))
        if r * c == world:
            return r, c
    mean_row = nnz / max(1, M)
    b_bytes = N * K * elem_bytes
    cols = 1
    if elem_bytes == 4 and K * elem_bytes <= 256 and b_bytes > 1.25 * l2_bytes and mean_row >= 16:
        while cols * 2 <= min(world, 4) and b_bytes / cols > 0.5 * l2_bytes and mean_row / (2 * cols) >= 3:   # (measured up to 4 column parts)
            cols *= 2
        if b_bytes / cols > l2_bytes:   # the slice would still not fit (2 GPUs, K = 64: 549 us with row ranges, 574 us with 1 x 2)
            cols = 1
    return world // cols, cols


def block_shard(row_ptr, col_idx, s_val, A, B, rank: int, grid, align: int = 1):
    """Block (rank // C, rank % C) of the R x C partition `grid` as a problem of its own: a dict with the local CSR arrays
    (column indices re-based to the block's first column), the rows of A and of B the block needs, its position in the
    whole matrix (r0, r1, c0, c1) and `sel`, the positions of its nonzeros in the whole matrix' CSR order (None for a
    plain row range, whose nonzeros are the contiguous range [j0, j1)).  Row ranges are balanced by nonzeros
    (row_cuts), column ranges are equal."""
    R, C = grid
    gr, gc = rank // C, rank % C
    M, N = len(row_ptr) - 1, B.shape[0]
    cuts = row_cuts(row_ptr, R, align)
    r0, r1 = int(cuts[gr]), int(cuts[gr + 1])
    j0, j1 = int(row_ptr[r0]), int(row_ptr[r1])
    rp = (np.asarray(row_ptr[r0:r1 + 1], dtype=np.int64) - j0)
    if C == 1:
        return {"r0": r0, "r1": r1, "c0": 0, "c1": N, "j0": j0, "j1": j1, "sel": None, "M": r1 - r0, "N": N, "nnz": j1 - j0,
                "rp": rp.astype(np.int32), "col": col_idx[j0:j1], "val": s_val[j0:j1], "A": A[r0:r1], "B": B, "grid": (R, C)}
    c0, c1 = (N * gc) // C, (N * (gc + 1)) // C
    cols = np.asarray(col_idx[j0:j1])
    inside = (cols >= c0) & (cols < c1)
    kept = np.concatenate(([0], np.cumsum(inside, dtype=np.int64)))   # nonzeros of the block before each position of the range
    sel = np.flatnonzero(inside)
    return {"r0": r0, "r1": r1, "c0": c0, "c1": c1, "j0": j0, "j1": j1, "sel": sel + j0, "M": r1 - r0, "N": c1 - c0, "nnz": int(sel.size),
            "rp": kept[rp].astype(np.int32), "col": (cols[sel] - c0).astype(np.int32), "val": np.ascontiguousarray(np.asarray(s_val[j0:j1])[sel]),
            "A": A[r0:r1], "B": B[c0:c1], "grid": (R, C)}
