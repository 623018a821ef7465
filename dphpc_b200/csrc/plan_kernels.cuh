// Upload-time kernels: validation of the uploaded pattern, the row-length
// histogram, COO -> row_ptr, the nnz-balanced work-item table and storage
// conversion.  They replace host loops of the reference
// (CSR::_dispatch, src/matrices/CSR.hpp:214-264; GPUPreprocessing::init_csr,
// src/competitors/gpu/gpu_preprocessing.hpp:56-128; gpu_convert_kernel,
// src/competitors/gpu/gpu_convert.cu:8-18) and run once per upload, outside
// the timed compute phase.
#pragma once

#include "device_utils.cuh"
#include "../../include/sddmm_b200.h"

namespace sddmm {

struct PlanCounters {
    unsigned long long hist[SDDMM_B200_HIST_BINS];
    unsigned long long hist_nnz[SDDMM_B200_HIST_BINS];   // nonzeros held by the rows of each length bin
    unsigned long long rows_nonempty;
    unsigned long long cols_touched;
    unsigned long long dense_nnz;
    unsigned long long rowgroup_nnz;
    unsigned long long group_cover[9];   // nonzeros inside matching row groups: 2, 3, 4 rows per group x first full group at row 0 .. G-1
    int max_row_nnz;
    int bad_row_ptr;   // row_ptr not monotone / wrong ends
    int bad_col;       // column index outside [0, N)
    int unsorted_cols; // a column index smaller than its predecessor inside a row
    int dup_cols;      // a column index equal to its predecessor inside a row
    int bad_coo;       // COO row index out of range or decreasing
    int dense_tiles;
    int rowgroups;
    int group_count[9];                  // matching row groups, same slots
    int residual_items;
    unsigned long long units;            // row segments of the row-segment path
    unsigned long long window_nnz;       // nonzeros inside the selected 64x64 windows (summed per window)
    int n_anchors;                       // candidate origins of the arbitrary-offset tile detection
};

__device__ __forceinline__ int len_bin(int len) {
    if (len <= 0) return 0;
    int b = 32 - __clz(len);  // len in [2^(b-1), 2^b)
    return b < SDDMM_B200_HIST_BINS ? b : SDDMM_B200_HIST_BINS - 1;
}

// one thread per row: monotonicity, histogram, max, nonempty count, row-start bits
__global__ void k_row_stats(const int32_t *__restrict__ rp, int32_t M, int64_t nnz, uint32_t *__restrict__ row_start_bits,
                            PlanCounters *__restrict__ pc) {
    __shared__ unsigned int sh[SDDMM_B200_HIST_BINS];
    __shared__ unsigned long long sh_nnz[SDDMM_B200_HIST_BINS];
    __shared__ unsigned int s_nonempty;
    __shared__ int s_max;
    if (threadIdx.x < SDDMM_B200_HIST_BINS) { sh[threadIdx.x] = 0; sh_nnz[threadIdx.x] = 0; }
    if (threadIdx.x == 0) { s_nonempty = 0; s_max = 0; }
    __syncthreads();
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i < M) {
        const int a = rp[i], b = rp[i + 1];
        const int len = b - a;
        if (len < 0 || a < 0 || b > nnz) {
            pc->bad_row_ptr = 1;
        } else {
            atomicAdd(&sh[len_bin(len)], 1u);
            if (len > 0) {
                atomicAdd(&sh_nnz[len_bin(len)], static_cast<unsigned long long>(len));
                atomicAdd(&s_nonempty, 1u);
                atomicMax(&s_max, len);
                atomicOr(&row_start_bits[a >> 5], 1u << (a & 31));
            }
        }
        if (i == 0 && a != 0) pc->bad_row_ptr = 1;
        if (i == M - 1 && b != nnz) pc->bad_row_ptr = 1;
    }
    __syncthreads();
    if (threadIdx.x < SDDMM_B200_HIST_BINS && sh[threadIdx.x]) {
        atomicAdd(&pc->hist[threadIdx.x], (unsigned long long)sh[threadIdx.x]);
        if (sh_nnz[threadIdx.x]) atomicAdd(&pc->hist_nnz[threadIdx.x], sh_nnz[threadIdx.x]);
    }
    if (threadIdx.x == 0) {
        if (s_nonempty) atomicAdd(&pc->rows_nonempty, (unsigned long long)s_nonempty);
        if (s_max) atomicMax(&pc->max_row_nnz, s_max);
    }
}

// one thread per nonzero: column range, touched-column flags, in-row ordering
__global__ void k_col_scan(const int32_t *__restrict__ col, int64_t nnz, int32_t N, const uint32_t *__restrict__ row_start_bits,
                           unsigned char *__restrict__ touched, PlanCounters *__restrict__ pc) {
    for (int64_t j = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; j < nnz;
         j += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int c = col[j];
        if (c < 0 || c >= N) {
            pc->bad_col = 1;
            continue;
        }
        if (!touched[c]) touched[c] = 1;
        const bool is_start = (row_start_bits[j >> 5] >> (j & 31)) & 1u;
        if (!is_start && j > 0) {
            const int prev = col[j - 1];
            if (prev > c) pc->unsorted_cols = 1;
            if (prev == c) pc->dup_cols = 1;
        }
    }
}

__global__ void k_count_bytes(const unsigned char *__restrict__ flags, int64_t n, unsigned long long *__restrict__ out) {
    unsigned int local = 0;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        local += flags[i] ? 1u : 0u;
    for (int off = 16; off > 0; off >>= 1) local += __shfl_xor_sync(kFullMask, local, off);
    if ((threadIdx.x & 31) == 0 && local) atomicAdd(out, (unsigned long long)local);
}

// COO (sorted by row) -> row_ptr.  Thread j owns the rows in (row[j-1], row[j]].  `base` is subtracted from every row index
// (a slice of a larger matrix that starts at row `base`).
__global__ void k_coo_to_row_ptr(const int32_t *__restrict__ row, int64_t nnz, int32_t M, int32_t base, int32_t *__restrict__ rp,
                                 PlanCounters *__restrict__ pc) {
    for (int64_t j = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; j <= nnz;
         j += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t prev = (j == 0) ? -1 : static_cast<int64_t>(row[j - 1]) - base;
        const int64_t cur = (j == nnz) ? M : static_cast<int64_t>(row[j]) - base;
        if (prev < -1 || prev >= M || cur < 0 || cur > M || (j < nnz && cur >= M) || cur < prev) {
            pc->bad_coo = 1;
            continue;
        }
        for (int64_t r = prev + 1; r <= cur; ++r) rp[r] = static_cast<int32_t>(j);
    }
}

// one thread per work item: rows holding its first and last nonzero
__global__ void k_item_rows(const int32_t *__restrict__ rp, int32_t M, int64_t nnz, int32_t item_nnz, int32_t n_items,
                            int2 *__restrict__ item_rows) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_items) return;
    const int64_t j0 = static_cast<int64_t>(t) * item_nnz;
    const int64_t j1 = min(nnz, j0 + item_nnz) - 1;
    int2 out;
    {
        int lo = 0, hi = M;
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (rp[mid] <= j0) lo = mid; else hi = mid; }
        out.x = lo;
    }
    {
        int lo = out.x, hi = M;
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (rp[mid] <= j1) lo = mid; else hi = mid; }
        out.y = lo;
    }
    item_rows[t] = out;
}

// ---- dense-tile detection (64x64 aligned tiles at least half full) -----------------------
// One warp per row: lanes take contiguous chunks of the (sorted) row so that runs of
// nonzeros inside one tile are counted locally and flushed with one atomic per run.
__global__ void k_tile_count(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t M, int32_t tiles_per_row,
                             int32_t *__restrict__ counts) {
    const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= M) return;
    const int a = rp[w], b = rp[w + 1];
    const int len = b - a;
    if (len == 0) return;
    const int per = (len + 31) >> 5;
    const int lo = a + lane * per, hi = min(b, lo + per);
    const int64_t base = static_cast<int64_t>(w >> 6) * tiles_per_row;
    int cur = -1, run = 0;
    for (int j = lo; j < hi; ++j) {
        const int t = col[j] >> 6;
        if (t != cur) {
            if (run) atomicAdd(&counts[base + cur], run);
            cur = t;
            run = 0;
        }
        ++run;
    }
    if (run) atomicAdd(&counts[base + cur], run);
}

// aligned tiles with >= min_count nonzeros: append their origin (first row, first column) to the dense list
__global__ void k_tile_select(const int32_t *__restrict__ counts, int64_t n_tiles, int32_t tiles_per_row, int32_t min_count,
                              int2 *__restrict__ origins, int32_t cap, PlanCounters *__restrict__ pc) {
    for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < n_tiles;
         t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        if (counts[t] >= min_count) {
            const int slot = atomicAdd(&pc->dense_tiles, 1);
            if (slot < cap) {
                origins[slot] = make_int2(static_cast<int32_t>(t / tiles_per_row) * 64, static_cast<int32_t>(t % tiles_per_row) * 64);
                atomicAdd(&pc->window_nnz, static_cast<unsigned long long>(counts[t]));
            }
        }
    }
}

// first position of [lo, hi) whose column is >= c (columns sorted inside a row)
__device__ __forceinline__ int32_t lower_col(const int32_t *__restrict__ col, int32_t lo, int32_t hi, int64_t c) {
    while (lo < hi) {
        const int32_t mid = (lo + hi) >> 1;
        if (col[mid] < c) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// ---- dense 64x64 windows at ARBITRARY offsets ("randomly placed blocks") ---------------------------------------------
// Step 1, one warp per row: nonzero j is a CANDIDATE when at least `half` nonzeros of its row lie in the 64 columns
// that start at its own column.  One bit per nonzero.
__global__ void k_window_candidates(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t M, int32_t half,
                                    uint32_t *__restrict__ cand) {
    const int lane = threadIdx.x & 31;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t r = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5; r < M; r += n_warps) {
        const int32_t a = rp[r], b = rp[r + 1];
        if (b - a < half) continue;
        for (int32_t j = a + lane; j < b; j += 32) {
            if (j + half > b) continue;
            // `half` nonzeros from j on fit into 64 columns <=> the (half-1)-th successor is closer than 64 columns
            if (col[j + half - 1] - col[j] < 64) atomicOr(&cand[j >> 5], 1u << (j & 31));
        }
    }
}

// nonzeros of row r inside columns [c, c + 64)
__device__ __forceinline__ int32_t window_count(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t r, int32_t c) {
    const int32_t a = rp[r], b = rp[r + 1];
    const int32_t lo = lower_col(col, a, b, c);
    return lower_col(col, lo, min(b, lo + 64), static_cast<int64_t>(c) + 64) - lo;
}

// Step 2, one thread per row: the row's candidates are cut greedily, left to right, into 64-column windows (a window
// starts at the first candidate at or after the end of the previous one), so every window of a row is visited once.  A
// window whose row above is NOT dense in the same columns is the top edge of a block and anchors a tile there -- and
// further tiles every 64 rows below it for as long as those rows stay dense in the same columns.
__global__ void k_window_anchors(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t M, int32_t half,
                                 const uint32_t *__restrict__ cand, int2 *__restrict__ anchors, int32_t cap, int *__restrict__ n_anchors) {
    // first candidate position in [j, b), or b
    auto next_cand = [&](int32_t j, int32_t b) -> int32_t {
        while (j < b) {
            const uint32_t word = cand[j >> 5] >> (j & 31);
            if (word) return min(b, j + __ffs(word) - 1);
            j = (j | 31) + 1;
        }
        return b;
    };
    for (int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; r < M; r += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int32_t a = rp[r], b = rp[r + 1];
        if (b - a < half) continue;
        for (int32_t w = next_cand(a, b); w < b;) {
            const int32_t c = col[w];
            const bool top = (r == 0) || window_count(rp, col, static_cast<int32_t>(r) - 1, c) < half;
            if (top) {
                for (int32_t rr = static_cast<int32_t>(r); rr < M; rr += 64) {
                    if (rr != r && window_count(rp, col, rr, c) < half) break;
                    const int slot = atomicAdd(n_anchors, 1);
                    if (slot < cap) anchors[slot] = make_int2(rr, c);
                }
            }
            w = next_cand(lower_col(col, w, b, static_cast<int64_t>(c) + 64), b);
        }
    }
}

// Step 3, one thread per (anchor, row): nonzeros inside the anchored window, summed per anchor
__global__ void k_anchor_counts(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t M, const int2 *__restrict__ anchors,
                                int32_t n_anchors, int32_t *__restrict__ counts) {
    const int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (g >= static_cast<int64_t>(n_anchors) * 64) return;
    const int2 o = anchors[g >> 6];
    const int32_t row = o.x + static_cast<int32_t>(g & 63);
    int32_t n = row < M ? window_count(rp, col, row, o.y) : 0;
    for (int off = 16; off > 0; off >>= 1) n += __shfl_xor_sync(kFullMask, n, off);   // (64 rows of an anchor = 2 warps)
    if ((threadIdx.x & 31) == 0 && n) atomicAdd(&counts[g >> 6], n);
}
// Step 4: anchors whose window holds >= min_count nonzeros become dense tiles
__global__ void k_anchor_select(const int2 *__restrict__ anchors, const int32_t *__restrict__ counts, int32_t n_anchors, int32_t min_count,
                                int2 *__restrict__ origins, int32_t cap, PlanCounters *__restrict__ pc) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_anchors || counts[t] < min_count) return;
    const int slot = atomicAdd(&pc->dense_tiles, 1);
    if (slot < cap) {
        origins[slot] = anchors[t];
        atomicAdd(&pc->window_nnz, static_cast<unsigned long long>(counts[t]));
    }
}

// Overlapping tiles (windows at arbitrary offsets): who computes a nonzero that lies in several of them is decided by a
// key, not by a race -- every (tile, row) proposes (row offset << 6 | column offset) for each of its nonzeros, the
// smallest key wins (two tiles that hold the same nonzero differ in their origin, hence in the key), so the same matrix
// always gets the same owners and the same tiles survive k_tile_keep.  owner: one word per nonzero, preset to ~0.
__global__ void k_tile_propose(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t M, const int2 *__restrict__ origins,
                               int32_t n_dense, uint32_t *__restrict__ owner) {
    const int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (g >= static_cast<int64_t>(n_dense) * 64) return;
    const int t = static_cast<int>(g >> 6), r = static_cast<int>(g & 63);
    const int2 o = origins[t];
    const int row = o.x + r;
    if (row >= M) return;
    const int end = rp[row + 1];
    for (int j = lower_col(col, rp[row], end, o.y); j < end; ++j) {
        const int c = col[j] - o.y;
        if (c >= 64) break;
        atomicMin(&owner[j], (static_cast<uint32_t>(r) << 6) | static_cast<uint32_t>(c));
    }
}

// one thread per (dense tile, row): first CSR position of the row inside the tile's column range, presence mask of its 64
// columns, and the OWN mask -- the nonzeros this tile computes.  Tiles on the 64-grid never overlap (owner == nullptr: a
// nonzero is claimed in the `covered` bitmap and every claim succeeds); overlapping tiles own what k_tile_propose gave
// them.  Owned nonzeros are credited to their work items.
template <typename Desc>
__global__ void k_tile_rows(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t M, const int2 *__restrict__ origins,
                            int32_t n_dense, Desc *__restrict__ descs, uint32_t *__restrict__ covered, int32_t item_nnz,
                            int32_t *__restrict__ item_covered, int32_t *__restrict__ tile_owned, PlanCounters *__restrict__ pc,
                            const uint32_t *__restrict__ owner) {
    const int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (g >= static_cast<int64_t>(n_dense) * 64) return;
    const int t = static_cast<int>(g >> 6), r = static_cast<int>(g & 63);
    const int2 o = origins[t];
    const int row = o.x + r;
    const int c0 = o.y;
    int start = 0;
    unsigned long long mask = 0ull, own = 0ull;
    if (row < M) {
        const int end = rp[row + 1];
        start = lower_col(col, rp[row], end, c0);
        int n = 0;
        for (int j = start; j < end; ++j) {
            const int c = col[j] - c0;
            if (c >= 64) break;
            mask |= 1ull << c;
            ++n;
        }
        // bit k of `got` = nonzero start + k is ours: by its key (overlapping tiles), else by claiming [start, start + n)
        // in the bitmap word by word
        unsigned long long got = 0ull;
        if (owner) {
            for (int k = 0; k < n; ++k)
                if (owner[start + k] == ((static_cast<uint32_t>(r) << 6) | static_cast<uint32_t>(col[start + k] - c0))) got |= 1ull << k;
        }
        for (int j = start; j < start + n;) {
            const int w = j >> 5, first = j & 31;
            const int take = min(32 - first, start + n - j);
            uint32_t bits = (take == 32 ? 0xffffffffu : ((1u << take) - 1u)) << first;
            if (owner) {
                bits &= static_cast<uint32_t>(got >> (j - start)) << first;   // mark what is ours as covered
                if (bits) atomicOr(&covered[w], bits);
            } else {
                const uint32_t old = atomicOr(&covered[w], bits);
                got |= static_cast<unsigned long long>((bits & ~old) >> first) << (j - start);
            }
            j += take;
        }
        // rank k of the run -> its column bit
        int k = 0, owned = 0;
        for (unsigned long long m = mask; m; m &= m - 1, ++k)
            if ((got >> k) & 1ull) {
                own |= m & (~m + 1);
                ++owned;
            }
        if (owned) {
            atomicAdd(&pc->dense_nnz, static_cast<unsigned long long>(owned));
            atomicAdd(&tile_owned[t], owned);
        }
        // credit the owned nonzeros to the work items they lie in
        for (int kk = 0; kk < n;) {
            const int j = start + kk;
            const int item = j / item_nnz;
            const int take = min(n - kk, (item + 1) * item_nnz - j);
            const unsigned long long seg = (take == 64 ? ~0ull : ((1ull << take) - 1ull)) << kk;
            const int c = __popcll(got & seg);
            if (c) atomicAdd(&item_covered[item], c);
            kk += take;
        }
    }
    descs[t].start[r] = start;
    descs[t].mask[r] = mask;
    descs[t].own[r] = own;
}

// Overlapping windows: a tile that ended up owning too few nonzeros (most of its window went to its neighbours) is not
// worth a job.  The tiles that own enough are copied to a second list, on which the ownership is then decided afresh.
__global__ void k_tile_keep(const int2 *__restrict__ origins, const int32_t *__restrict__ tile_owned, int32_t n_dense, int32_t min_owned,
                            int2 *__restrict__ kept, PlanCounters *__restrict__ pc) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_dense || tile_owned[t] < min_owned) return;
    kept[atomicAdd(&pc->dense_tiles, 1)] = origins[t];
}

// work items that still hold nonzeros outside the dense tiles
__global__ void k_residual_items(const int32_t *__restrict__ item_covered, int32_t n_items, int32_t item_nnz, int64_t nnz,
                                 int32_t *__restrict__ item_ids, PlanCounters *__restrict__ pc) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_items) return;
    const int64_t size = min(nnz, static_cast<int64_t>(t + 1) * item_nnz) - static_cast<int64_t>(t) * item_nnz;
    if (item_covered[t] < size) item_ids[atomicAdd(&pc->residual_items, 1)] = t;
}

// fp32-grade products from tf32 tensor cores: with hi = tf32(x), lo = tf32(x - hi),
//   a.b ~= a_lo*b_hi + a_hi*b_lo + a_hi*b_hi   (the dropped lo*lo term is ~2^-22 relative).
// The three products become ONE dot product of 3K-long rows:
//   first_operand = 1:  out row = [ lo | hi | hi ]     (used for A)
//   first_operand = 0:  out row = [ hi | lo | hi ]     (used for B)
__global__ void k_split_concat_tf32(const float *__restrict__ in, float *__restrict__ out, int64_t rows, int32_t K, int first_operand) {
    const int64_t n = rows * K;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const float x = in[i];
        uint32_t h, l;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
        const float hf = __uint_as_float(h);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(x - hf));
        const float lf = __uint_as_float(l);
        const int64_t r = i / K, k = i - r * K;
        float *o = out + r * 3 * K + k;
        o[0] = first_operand ? lf : hf;
        o[K] = first_operand ? hf : lf;
        o[2 * K] = hf;
    }
}

// bf16 storage: out = bf16(in), and `in` keeps the rounded value (as fp32) for the tensor-core path
__global__ void k_f32_to_bf16(float *__restrict__ in, __nv_bfloat16 *__restrict__ out, int64_t n) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const __nv_bfloat16 r = __float2bfloat16_rn(in[i]);
        out[i] = r;
        in[i] = __bfloat162float(r);
    }
}

}  // namespace sddmm
