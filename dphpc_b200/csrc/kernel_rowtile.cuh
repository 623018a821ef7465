// Row-tile SDDMM kernel: the general path for short, power-law and long rows.
//
// Work decomposition (no atomics, exactly one writer per nonzero):
//   * the nonzero index space [0, nnz) is cut into items of `item_nnz`
//     consecutive nonzeros (nnz-balanced, independent of the row-length
//     distribution); `item_row[t]` is the row that holds the first nonzero of
//     item t (built once per upload on the device);
//   * a CTA walks the rows its item spans in stages of at most
//     `rows_per_stage` rows: the row_ptr slice and the A rows of the stage are
//     brought into shared memory, the A rows by ONE bulk async copy
//     (cp.async.bulk, completion on an mbarrier), since consecutive rows of a
//     row-major A are one contiguous byte range;
//   * a warp takes 32 consecutive nonzeros: one coalesced 128-byte load each of
//     col_idx and S.val, a binary search of the staged row_ptr slice for the
//     row of each nonzero, then each 8-lane group gathers the B rows of its 8
//     nonzeros (8 independent 16-byte loads per lane in flight, each B row read
//     as one contiguous line by the group), multiplies with the A chunks held
//     in shared memory and reduces over K with a transposing shuffle tree that
//     leaves nonzero g on lane g -> one coalesced 128-byte store of P per warp.
//
// CPL = chunks per lane (a chunk is 4 K-elements).  K <= 32*CPL, K % 4 == 0.
#pragma once

#include "device_utils.cuh"

namespace sddmm {

struct RowTileArgs {
    const int32_t *row_ptr;   // M+1
    const int32_t *col_idx;   // nnz
    const float *s_val;       // nnz
    float *p_val;             // nnz
    const void *A;            // M x K, element type ET
    const void *B;            // N x K, element type ET
    const int2 *item_rows;    // per item: {row of its first nonzero, row of its last nonzero}
    const int32_t *item_ids;  // optional indirection (items that still hold work), or nullptr
    const uint32_t *skip_tile_bitmap;  // optional: nonzeros whose 64x64 tile bit is set are owned by another kernel
    int32_t skip_tiles_per_row;        // number of 64-column tiles per tile row in the bitmap
    int32_t *err;             // device error word
    int64_t nnz;
    int32_t M, K;
    int32_t n_items;          // entries of item_ids if given, else total items
    int32_t item_nnz;         // multiple of 32
    int32_t rows_per_stage;   // R
};

template <int CPL, typename ET>
__global__ void __launch_bounds__(256) sddmm_rowtile_kernel(const RowTileArgs args) {
    using chunk_t = typename ChunkOf<ET>::type;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar;

    const int K = args.K;
    const int R = args.rows_per_stage;
    const int nchunks = K >> 2;
    ET *sA = reinterpret_cast<ET *>(smem_raw);
    const uint32_t a_stage_bytes = (static_cast<uint32_t>(R) * K * sizeof(ET) + 15u) & ~15u;
    int32_t *sRp = reinterpret_cast<int32_t *>(smem_raw + a_stage_bytes);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int nwarps = blockDim.x >> 5;
    const int gl = lane & 7;          // lane inside its 8-lane group
    const int gbase = lane & ~7;      // first lane of the group

    if (tid == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    __syncthreads();
    uint32_t phase = 0;

    const chunk_t *Bc = reinterpret_cast<const chunk_t *>(args.B);

    for (int it = blockIdx.x; it < args.n_items; it += gridDim.x) {
        const int item = args.item_ids ? args.item_ids[it] : it;
        const int64_t j_lo = static_cast<int64_t>(item) * args.item_nnz;
        const int64_t j_hi = min(args.nnz, j_lo + args.item_nnz);
        const int2 rr = args.item_rows[item];
        const int r_lo = rr.x, r_hi = rr.y;

        for (int r0 = r_lo; r0 <= r_hi; r0 += R) {
            const int nr = min(R, r_hi - r0 + 1);
            for (int t = tid; t <= nr; t += blockDim.x) sRp[t] = args.row_ptr[r0 + t];
            if (tid == 0) {
                const uint32_t bytes = static_cast<uint32_t>(nr) * K * sizeof(ET);
                mbar_expect_tx(&bar, bytes);
                bulk_g2s(sA, reinterpret_cast<const ET *>(args.A) + static_cast<int64_t>(r0) * K, bytes, &bar);
            }
            __syncthreads();
            if (!mbar_wait_bounded(&bar, phase)) {
                atomicCAS(args.err, kDevOk, kDevMbarrierTimeout);
                return;  // every thread of the CTA waits on the same phase, so all leave together
            }
            phase ^= 1u;

            const int64_t s_lo = max(j_lo, static_cast<int64_t>(sRp[0]));
            const int64_t s_hi = min(j_hi, static_cast<int64_t>(sRp[nr]));
            // 32-aligned warp windows so every col/val/P access is a full 128-byte line
            for (int64_t wb = (s_lo & ~int64_t(31)) + warp * 32; wb < s_hi; wb += nwarps * 32) {
                const int64_t j = wb + lane;
                bool valid = (j >= s_lo) && (j < s_hi);
                int c = 0;
                float s = 0.f;
                if (valid) {
                    c = __ldcs(args.col_idx + j);
                    s = __ldcs(args.s_val + j);
                }
                // row of nonzero j inside the staged slice: largest t with sRp[t] <= j
                const int jj = static_cast<int>(min(max(j, s_lo), s_hi - 1));
                int lo = 0, hi = nr;
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (sRp[mid] <= jj) lo = mid; else hi = mid;
                }
                const int lr = lo;
                if (valid && args.skip_tile_bitmap) {
                    const int64_t bit = static_cast<int64_t>((r0 + lr) >> 6) * args.skip_tiles_per_row + (c >> 6);
                    if ((args.skip_tile_bitmap[bit >> 5] >> (bit & 31)) & 1u) valid = false;
                }
                const unsigned vmask = __ballot_sync(kFullMask, valid);
                if (vmask == 0u) continue;

                float acc[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = 0.f;
                int ci[8], ri[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    ci[i] = __shfl_sync(kFullMask, c, gbase + i);
                    ri[i] = __shfl_sync(kFullMask, lr, gbase + i);
                }
                const unsigned gmask = (vmask >> gbase) & 0xffu;

                constexpr int QS = (CPL >= 2) ? 2 : 1;  // chunks gathered per nonzero per step
#pragma unroll
                for (int q0 = 0; q0 < CPL; q0 += QS) {
                    chunk_t bq[8][QS];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
#pragma unroll
                        for (int qq = 0; qq < QS; ++qq) {
                            const int ch = gl + 8 * (q0 + qq);
                            if (((gmask >> i) & 1u) && ch < nchunks) {
                                bq[i][qq] = ldg_chunk(Bc + static_cast<int64_t>(ci[i]) * nchunks + ch);
                            } else {
                                bq[i][qq] = zero_chunk(chunk_t());
                            }
                        }
                    }
                    int cur = -1;
                    float4 a[QS];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (ri[i] != cur) {
                            cur = ri[i];
                            const chunk_t *sArow = reinterpret_cast<const chunk_t *>(sA) + static_cast<int64_t>(cur) * nchunks;
#pragma unroll
                            for (int qq = 0; qq < QS; ++qq) {
                                const int ch = gl + 8 * (q0 + qq);
                                a[qq] = (ch < nchunks) ? chunk_to_f4(sArow[ch]) : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
#pragma unroll
                        for (int qq = 0; qq < QS; ++qq) acc[i] = dot4(a[qq], chunk_to_f4(bq[i][qq]), acc[i]);
                    }
                }
                const float dot = group8_transpose_reduce(acc, gl);
                if (valid) __stcs(args.p_val + j, dot * s);
            }
            __syncthreads();  // all reads of sA / sRp done before the next stage overwrites them
        }
    }
}

// Fallback for K % 4 != 0 (and for K too large to stage): one thread per
// nonzero, sequential k loop, row found by binary search of row_ptr.
__global__ void __launch_bounds__(256) sddmm_scalar_kernel(const int32_t *__restrict__ row_ptr,
                                                           const int32_t *__restrict__ col_idx,
                                                           const float *__restrict__ s_val, float *__restrict__ p_val,
                                                           const float *__restrict__ A, const float *__restrict__ B,
                                                           int32_t M, int32_t K, int64_t nnz) {
    for (int64_t j = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; j < nnz;
         j += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int lo = 0, hi = M;  // row_ptr[lo] <= j < row_ptr[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (row_ptr[mid] <= j) lo = mid; else hi = mid;
        }
        const float *a = A + static_cast<int64_t>(lo) * K;
        const float *b = B + static_cast<int64_t>(col_idx[j]) * K;
        float acc = 0.f;
        for (int k = 0; k < K; ++k) acc = fmaf(a[k], b[k], acc);
        p_val[j] = acc * s_val[j];
    }
}

}  // namespace sddmm
