// Row-group SDDMM kernel: consecutive rows of S that have IDENTICAL column lists
// (the dense G x G blocks of multi-degree-of-freedom discretisations: every one of
// the G rows of a block row touches the same columns) share one gather of B.
//
// Rows are taken in groups of G consecutive rows starting at row `first` (0 <= first < G; the
// rows before it form a leading group that never matches, so that a row shard cut anywhere
// still lines up with the block rows).  A group whose rows
// all have the same column list is processed as one unit: each B row is read ONCE
// into registers and dotted with the G rows of A, so the traffic between L2/L1
// and the SM -- what bounds the general kernel -- drops by the factor G.  Groups
// that do not match are processed row by row by the same code (unit of one row).
//
// One warp per group (static round-robin, so neighbouring groups -- which touch
// neighbouring rows of B in banded matrices -- run on the same SM).  A warp walks
// the shared column list in windows of 32: lane l loads column l of the window;
// each 8-lane group owns 8 of the 32 columns, lane = one 16-byte chunk of a
// 128-byte piece of the B row (K > 32: several pieces), the K-dot is reduced with
// the transposing shuffle tree that leaves column c of the group on lane c, so for
// every row of the unit S.val is read and P.val written as one coalesced 128-byte
// access.  The A rows of the unit stay in registers for the whole column list.
//
// fp32 storage, K = 32 * CPL, CPL in {1, 2}.
#pragma once

#include "device_utils.cuh"
#include "plan_kernels.cuh"

namespace sddmm {

struct RowGroupArgs {
    const int32_t *row_ptr;   // M+1
    const int32_t *col_idx;   // nnz
    const float *s_val;       // nnz
    float *p_val;             // nnz
    const float *A;           // M x K
    const float *B;           // N x K
    const uint8_t *group_ok;  // per group: 1 if its G rows have one column list
    int32_t M, K;
    int32_t first;            // group 0 = rows [0, first); group g >= 1 = rows [first + (g-1) G, first + g G)
    int32_t n_groups;         // 1 + ceil((M - first) / G)
};

// rows of group g
__device__ __forceinline__ void group_rows(int32_t g, int32_t G, int32_t first, int32_t M, int32_t &r0, int32_t &r1) {
    r0 = g == 0 ? 0 : first + (g - 1) * G;
    r1 = g == 0 ? first : min(r0 + G, M);
}

constexpr int kRowGroupWarps = 8;

// Which groups of G rows share one column list.  One warp per group; only every `every`-th group is
// looked at (every > 1: a sample, to choose G and `first` cheaply; group_ok is then not written).
// cover += nonzeros inside matching groups; groups += matching groups.
__global__ void k_group_match(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t M, int32_t G, int32_t first,
                              int32_t n_groups, int32_t every, uint8_t *__restrict__ group_ok, unsigned long long *__restrict__ cover,
                              int *__restrict__ groups) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    const int64_t n_warps = (gridDim.x * static_cast<int64_t>(blockDim.x)) >> 5;
    for (int64_t g = warp0 * every; g < n_groups; g += n_warps * every) {
        int32_t r0, r1;
        group_rows(static_cast<int32_t>(g), G, first, M, r0, r1);
        bool ok = g > 0 && r1 - r0 == G;
        int32_t len = 0;
        if (ok) {
            const int32_t s0 = rp[r0];
            len = rp[r0 + 1] - s0;
            ok = len > 0;
            for (int t = 1; t < G && ok; ++t) {
                const int32_t st = rp[r0 + t];
                ok = (rp[r0 + t + 1] - st) == len;
                if (ok) {
                    bool same = true;
                    for (int32_t j = lane; j < len; j += 32) same = same && (col[s0 + j] == col[st + j]);
                    ok = __all_sync(kFullMask, same);
                }
            }
        }
        if (lane == 0) {
            if (group_ok) group_ok[g] = ok ? 1 : 0;
            if (ok) {
                atomicAdd(cover, static_cast<unsigned long long>(len) * static_cast<unsigned long long>(G));
                atomicAdd(groups, 1);
            }
        }
    }
}

// NR rows (first row r) with one column list: all of its windows.
template <int NR, int CPL>
__device__ __forceinline__ void rowgroup_unit(const RowGroupArgs &a, int32_t r, int lane) {
    const int gl = lane & 7;           // chunk inside the 128-byte piece
    const int gbase = lane & 24;       // first lane of this 8-lane group
    const int32_t s0 = a.row_ptr[r];
    const int32_t len = a.row_ptr[r + 1] - s0;
    if (len <= 0) return;
    const int kq = a.K >> 2;           // float4 per dense row
    const float4 *__restrict__ A4 = reinterpret_cast<const float4 *>(a.A);
    const float4 *__restrict__ B4 = reinterpret_cast<const float4 *>(a.B);
    int32_t sp[NR];
    float4 av[NR][CPL];
#pragma unroll
    for (int t = 0; t < NR; ++t) {
        sp[t] = a.row_ptr[r + t];
#pragma unroll
        for (int k = 0; k < CPL; ++k) av[t][k] = __ldg(A4 + static_cast<int64_t>(r + t) * kq + gl + 8 * k);
    }
    int32_t cj_next = __ldg(a.col_idx + s0 + min(lane, len - 1));   // tail lanes repeat the last column (never stored)
    for (int32_t w0 = 0; w0 < len; w0 += 32) {
        const int32_t j = w0 + lane;
        const int32_t cj = cj_next;
        if (w0 + 32 < len) cj_next = __ldg(a.col_idx + s0 + min(j + 32, len - 1));   // next window's columns: requested a window ahead
        float sv[NR];   // S.val of this window for every row of the unit: requested before the gathers, used after the dots
#pragma unroll
        for (int t = 0; t < NR; ++t) sv[t] = (j < len) ? __ldcs(a.s_val + sp[t] + j) : 0.f;
        float4 bv[8][CPL];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int32_t cc = __shfl_sync(kFullMask, cj, gbase + c);
#pragma unroll
            for (int k = 0; k < CPL; ++k) bv[c][k] = __ldg(B4 + static_cast<int64_t>(cc) * kq + gl + 8 * k);
        }
#pragma unroll
        for (int t = 0; t < NR; ++t) {
            float acc[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float s = 0.f;
#pragma unroll
                for (int k = 0; k < CPL; ++k) s = dot4(av[t][k], bv[c][k], s);
                acc[c] = s;
            }
            const float dot = group8_transpose_reduce(acc, gl);   // lane gl of the group: column gbase + gl of the window = column j
            if (j < len) __stcs(a.p_val + sp[t] + j, sv[t] * dot);
        }
    }
}

template <int G, int CPL>
__global__ void __launch_bounds__(kRowGroupWarps * 32, 2) sddmm_rowgroup_kernel(const RowGroupArgs a) {
    const int lane = threadIdx.x & 31;
    const int32_t warp0 = blockIdx.x * kRowGroupWarps + (threadIdx.x >> 5);
    const int32_t n_warps = gridDim.x * kRowGroupWarps;
    for (int32_t g = warp0; g < a.n_groups; g += n_warps) {
        int32_t r0, r1;
        group_rows(g, G, a.first, a.M, r0, r1);
        if (a.group_ok[g]) {   // warp-uniform
            rowgroup_unit<G, CPL>(a, r0, lane);
        } else {
            for (int32_t r = r0; r < r1; ++r) rowgroup_unit<1, CPL>(a, r, lane);
        }
    }
}

}  // namespace sddmm
