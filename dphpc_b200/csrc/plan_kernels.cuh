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
    __shared__ unsigned int s_nonempty;
    __shared__ int s_max;
    if (threadIdx.x < SDDMM_B200_HIST_BINS) sh[threadIdx.x] = 0;
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
                atomicAdd(&s_nonempty, 1u);
                atomicMax(&s_max, len);
                atomicOr(&row_start_bits[a >> 5], 1u << (a & 31));
            }
        }
        if (i == 0 && a != 0) pc->bad_row_ptr = 1;
        if (i == M - 1 && b != nnz) pc->bad_row_ptr = 1;
    }
    __syncthreads();
    if (threadIdx.x < SDDMM_B200_HIST_BINS && sh[threadIdx.x]) atomicAdd(&pc->hist[threadIdx.x], (unsigned long long)sh[threadIdx.x]);
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

// tiles with >= min_count nonzeros: set their bit, append them to the dense list
__global__ void k_tile_select(const int32_t *__restrict__ counts, int64_t n_tiles, int32_t min_count, uint32_t *__restrict__ bitmap,
                              int32_t *__restrict__ dense_ids, int32_t cap, PlanCounters *__restrict__ pc) {
    for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < n_tiles;
         t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int c = counts[t];
        if (c >= min_count) {
            const int slot = atomicAdd(&pc->dense_tiles, 1);
            if (slot < cap) {
                dense_ids[slot] = static_cast<int32_t>(t);
                atomicOr(&bitmap[t >> 5], 1u << (t & 31));
                atomicAdd(&pc->dense_nnz, static_cast<unsigned long long>(c));
            }
        }
    }
}

// one thread per (dense tile, row): first CSR position of the row inside the tile's column
// range, presence mask of its 64 columns; also credits the covered nonzeros to their work items
template <typename Desc>
__global__ void k_tile_rows(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t M, int32_t tiles_per_row,
                            const int32_t *__restrict__ dense_ids, int32_t n_dense, Desc *__restrict__ descs, int32_t item_nnz,
                            int32_t *__restrict__ item_covered) {
    const int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (g >= static_cast<int64_t>(n_dense) * 64) return;
    const int t = static_cast<int>(g >> 6), r = static_cast<int>(g & 63);
    const int id = dense_ids[t];
    const int row = (id / tiles_per_row) * 64 + r;
    const int c0 = (id % tiles_per_row) * 64;
    int start = 0;
    unsigned long long mask = 0ull;
    if (row < M) {
        int lo = rp[row], hi = rp[row + 1];
        const int end = hi;
        while (lo < hi) {  // first position with col >= c0
            const int mid = (lo + hi) >> 1;
            if (col[mid] < c0) lo = mid + 1; else hi = mid;
        }
        start = lo;
        int n = 0;
        for (int j = lo; j < end; ++j) {
            const int c = col[j] - c0;
            if (c >= 64) break;
            mask |= 1ull << c;
            ++n;
        }
        // credit [start, start+n) to the work items it overlaps
        int j = start, left = n;
        while (left > 0) {
            const int item = j / item_nnz;
            const int take = min(left, (item + 1) * item_nnz - j);
            atomicAdd(&item_covered[item], take);
            j += take;
            left -= take;
        }
    }
    descs[t].start[r] = start;
    descs[t].mask[r] = mask;
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
