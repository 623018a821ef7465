// Consumer of the SDDMM result on the device: Y = P X, with P the CSR matrix whose values the SDDMM kernels have just
// written (they never leave the GPU) and X a dense N x K2 matrix.  This is the step that follows SDDMM in the
// applications the reference's report names (SpMM after SDDMM in graph attention and ALS-style factorisations); the
// reference itself stops at copying P back to the host (src/competitors/gpu/gpu_convert.hpp:58-64).
//
// Same decomposition as the row-segment SDDMM kernel: rows cut into segments of at most 8 nonzeros (unit list built on
// the device), a warp step takes 4 units, one per 8-lane group; lane l loads column index l and P value l of the segment,
// every X row is read as one contiguous line by the group (lane = one 16-byte chunk, K2 > 32: more chunks per lane),
// the lane accumulates p * x for its chunk over the 8 nonzeros and adds the partial row to Y with one vector
// reduction (red.global.add.v4.f32) per chunk -- Y is zeroed before the launch.  The order in which the partial sums of
// a row arrive is not fixed, so Y is reproducible only to fp32 rounding.
#pragma once

#include "device_utils.cuh"

namespace sddmm {

struct SpmmArgs {
    const int2 *units;        // n_units (> 0): .x = CSR position of the segment's first nonzero, .y = row * 8 + (count - 1)
    const int32_t *col_idx;   // nnz
    const float *p_val;       // nnz
    const float *X;           // N x K2
    float *Y;                 // M x K2, zeroed
    int32_t n_units;
    int32_t K2;
};

constexpr int kSpmmWarps = 8;

__device__ __forceinline__ void red_add_f4(float *dst, const float4 &v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

template <int CPL, bool EXACT>
__global__ void __launch_bounds__(kSpmmWarps * 32, (CPL == 1) ? 4 : 2) sddmm_spmm_kernel(const SpmmArgs args) {
    const int lane = threadIdx.x & 31;
    const int gl = lane & 7;
    const int gbase = lane & 24;
    const int grp = lane >> 3;
    const int nchunks = EXACT ? 8 * CPL : (args.K2 >> 2);
    const uint32_t row_bytes = static_cast<uint32_t>(nchunks) * sizeof(float4);

    const int64_t n_quads = (static_cast<int64_t>(args.n_units) + 3) >> 2;
    const int64_t n_warps = static_cast<int64_t>(gridDim.x) * kSpmmWarps;
    int64_t q = static_cast<int64_t>(blockIdx.x) * kSpmmWarps + (threadIdx.x >> 5);
    if (q >= n_quads) return;
    const int last_unit = args.n_units - 1;

    uint32_t ch_off[CPL];
    bool ch_on[CPL];
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
        const int ch = gl + 8 * c;
        ch_on[c] = EXACT || ch < nchunks;
        ch_off[c] = static_cast<uint32_t>(ch_on[c] ? ch : 0) * sizeof(float4);
    }
    const unsigned char *Xb = reinterpret_cast<const unsigned char *>(args.X);

    // loads are unconditional and in range (clamped unit, clamped slot); a slot past the segment's end carries p = 0
    auto load_unit = [&](int64_t qq) -> int2 {
        const int64_t u = 4 * qq + grp;
        return __ldcs(args.units + (u < last_unit ? u : last_unit));
    };
    auto own_slot = [&](const int2 &u) -> int { return u.x + min(gl, u.y & 7); };

    int2 u_cur = load_unit(q);
    int2 u_nxt = load_unit(q + n_warps);
    int c_own = __ldcs(args.col_idx + own_slot(u_cur));
    float p_own = __ldcs(args.p_val + own_slot(u_cur));

    while (true) {
        const int row = u_cur.y >> 3;
        const bool live = 4 * q + grp <= last_unit;
        const float p_lane = (live && gl <= (u_cur.y & 7)) ? p_own : 0.f;

        const unsigned char *xrow[8];
        float pv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            xrow[i] = Xb + static_cast<uint64_t>(static_cast<uint32_t>(__shfl_sync(kFullMask, c_own, gbase + i))) * row_bytes;
            pv[i] = __shfl_sync(kFullMask, p_lane, gbase + i);
        }
        float4 y[CPL];
#pragma unroll
        for (int c = 0; c < CPL; ++c) y[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 xq[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) xq[i] = __ldg(reinterpret_cast<const float4 *>(xrow[i] + ch_off[0]));
        const int64_t q_next = q + n_warps;
        const int2 u_nxt2 = load_unit(q_next + n_warps);
        c_own = __ldcs(args.col_idx + own_slot(u_nxt));
        p_own = __ldcs(args.p_val + own_slot(u_nxt));
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                y[c].x = fmaf(pv[i], xq[i].x, y[c].x);
                y[c].y = fmaf(pv[i], xq[i].y, y[c].y);
                y[c].z = fmaf(pv[i], xq[i].z, y[c].z);
                y[c].w = fmaf(pv[i], xq[i].w, y[c].w);
            }
            if (c + 1 < CPL) {
#pragma unroll
                for (int i = 0; i < 8; ++i) xq[i] = __ldg(reinterpret_cast<const float4 *>(xrow[i] + ch_off[c + 1]));
            }
        }
        if (live) {
            float *yrow = args.Y + static_cast<uint64_t>(static_cast<uint32_t>(row)) * static_cast<uint32_t>(args.K2);
#pragma unroll
            for (int c = 0; c < CPL; ++c)
                if (ch_on[c]) red_add_f4(yrow + 4 * (gl + 8 * c), y[c]);
        }
        q = q_next;
        if (q >= n_quads) break;   // warp-uniform
        u_cur = u_nxt;
        u_nxt = u_nxt2;
    }
}

}  // namespace sddmm
