// Row-tile SDDMM kernel: the general path for short, power-law and long rows.
//
// Work decomposition (no atomics, exactly one writer per nonzero):
//   * the nonzero index space [0, nnz) is cut into items of `item_nnz`
//     consecutive nonzeros (nnz-balanced, independent of the row-length
//     distribution); `item_rows[t]` holds the rows of the first and last
//     nonzero of item t (built once per upload on the device);
//   * a CTA walks the rows its item spans in stages of at most
//     `rows_per_stage` rows: the row_ptr slice and the A rows of the stage are
//     brought into shared memory, the A rows by ONE bulk async copy
//     (cp.async.bulk, completion on an mbarrier), since consecutive rows of a
//     row-major A are one contiguous byte range;
//   * a warp takes a 32-aligned window of 32 consecutive nonzeros: each 8-lane
//     group reads the 8 column indices of its nonzeros as two 16-byte loads,
//     gathers the 8 B rows (8 independent 16-byte loads per lane in flight, a B
//     row is read as one contiguous line by the group), multiplies with the A
//     chunks and reduces over K with a transposing shuffle tree that leaves
//     nonzero g on lane g -> one coalesced 128-byte store of P per warp;
//   * the A chunks come from registers while a window lies inside one row
//     (long rows: A_i is reused across all its nonzeros), otherwise from the
//     staged tile in shared memory through per-nonzero row offsets.
//
// A "chunk" is 4 consecutive K elements.  CPL = chunks per lane, so K <= 32*CPL.
// EXACT = (K == 32*CPL): no chunk-range predicates in the inner loop.
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
    const uint32_t *covered;           // optional, one bit per nonzero: set = owned by another kernel (the dense tiles)
    int32_t *err;             // device error word
    int64_t nnz;
    int32_t M, K;
    int32_t n_items;          // entries of item_ids if given, else total items
    int32_t item_nnz;         // multiple of 32
    int32_t rows_per_stage;   // R
};

constexpr int kRowTileWarps = 8;

// Dynamic shared memory of the row-tile kernel: two stage buffers, each = R staged rows of A (row_bytes each,
// rounded up to 16 bytes) + R + 1 row_ptr entries, rounded up to 16 bytes.
__host__ __device__ inline uint32_t rowtile_buffer_bytes(int rows_per_stage, uint32_t row_bytes) {
    const uint32_t a_stage_bytes = (static_cast<uint32_t>(rows_per_stage) * row_bytes + 15u) & ~15u;
    return (a_stage_bytes + (static_cast<uint32_t>(rows_per_stage) + 1u) * 4u + 15u) & ~15u;
}
__host__ __device__ inline uint32_t rowtile_smem_bytes(int rows_per_stage, uint32_t row_bytes) {
    return 2u * rowtile_buffer_bytes(rows_per_stage, row_bytes);
}
#ifndef SDDMM_ROWTILE_MINB1
#define SDDMM_ROWTILE_MINB1 4   // resident CTAs per SM the compiler must allow for, K <= 32
#endif
#ifndef SDDMM_ROWTILE_MINBN
#define SDDMM_ROWTILE_MINBN 2   // same, K > 32
#endif

template <int CPL, bool EXACT, typename ET>
__global__ void __launch_bounds__(kRowTileWarps * 32, (CPL == 1) ? SDDMM_ROWTILE_MINB1 : SDDMM_ROWTILE_MINBN) sddmm_rowtile_kernel(const RowTileArgs args) {
    using chunk_t = typename ChunkOf<ET>::type;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar[2];
    __shared__ __align__(16) int32_t sRowOff[kRowTileWarps][32];

    const int K = args.K;
    const int R = args.rows_per_stage;
    const int nchunks = EXACT ? 8 * CPL : (K >> 2);
    const uint32_t row_bytes = static_cast<uint32_t>(nchunks) * sizeof(chunk_t);
    const uint32_t a_stage_bytes = (static_cast<uint32_t>(R) * row_bytes + 15u) & ~15u;
    const uint32_t buf_bytes = rowtile_buffer_bytes(R, row_bytes);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int gl = lane & 7;          // lane inside its 8-lane group
    const int gbase = lane & ~7;      // first lane of the group

    if (tid == 0) {
        mbar_init(&bar[0], 1);
        mbar_init(&bar[1], 1);
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    __syncthreads();
    uint32_t phases = 0;   // bit b: parity the next wait on bar[b] uses

    // this lane's chunk of every B row
    const unsigned char *Bl = reinterpret_cast<const unsigned char *>(args.B) + gl * sizeof(chunk_t);
    constexpr int QS = (CPL >= 2) ? 2 : 1;  // chunks gathered per nonzero per step

    // A stage = up to R consecutive rows of one work item.  The stages of a CTA form one sequence (stages of an
    // item, then the next item of the CTA); the rows and row_ptr entries of stage s+1 are requested (bulk copy +
    // 4-byte asynchronous copies, into the other buffer) before stage s is processed.
    const int nnz32 = static_cast<int>(args.nnz);   // nonzero indices fit 32 bits (int32 row_ptr; nnz < 2^31 - 8192)
    auto load_item = [&](int it, int &j_lo, int &j_hi, int &r_lo, int &r_hi) {
        const int item = args.item_ids ? args.item_ids[it] : it;
        j_lo = item * args.item_nnz;
        j_hi = j_lo + min(nnz32 - j_lo, args.item_nnz);
        const int2 rr = args.item_rows[item];
        r_lo = rr.x;
        r_hi = rr.y;
    };
    auto issue_stage = [&](int b, int r0, int nr) {
        unsigned char *base = smem_raw + static_cast<uint32_t>(b) * buf_bytes;
        int32_t *rp_s = reinterpret_cast<int32_t *>(base + a_stage_bytes);
        for (int t = tid; t <= nr; t += blockDim.x) cp_async_4(&rp_s[t], args.row_ptr + r0 + t);
        if (tid == 0) {
            const uint32_t bytes = static_cast<uint32_t>(nr) * row_bytes;
            fence_proxy_async_smem();   // the buffer was read (generic proxy) in the stage before the previous one
            mbar_expect_tx(&bar[b], bytes);
            bulk_g2s(base, reinterpret_cast<const unsigned char *>(args.A) + static_cast<uint64_t>(r0) * row_bytes, bytes, &bar[b]);
        }
    };

    int it = blockIdx.x;
    if (it >= args.n_items) return;
    int j_lo, j_hi, r_lo, r_hi;
    load_item(it, j_lo, j_hi, r_lo, r_hi);
    int r0 = r_lo;
    int nr = min(R, r_hi - r0 + 1);
    int b = 0;
    issue_stage(0, r0, nr);
    cp_async_commit();

    while (true) {
        // ---- request the stage after this one (its parameters are recomputed when the CTA moves on: nothing
        //      but `has_next` stays live across the window loop) ------------------------------------------
        bool has_next = true;
        {
            int n_r0 = r0 + R, n_r_hi = r_hi;
            if (n_r0 > r_hi) {
                const int n_it = it + gridDim.x;
                if (n_it < args.n_items) {
                    int n_j_lo, n_j_hi;
                    load_item(n_it, n_j_lo, n_j_hi, n_r0, n_r_hi);
                } else {
                    has_next = false;
                }
            }
            if (has_next) issue_stage(b ^ 1, n_r0, min(R, n_r_hi - n_r0 + 1));
        }
        cp_async_commit();   // (an empty group when there is no next stage: the count below stays valid)

        {
            const chunk_t *sAc = reinterpret_cast<const chunk_t *>(smem_raw + static_cast<uint32_t>(b) * buf_bytes);
            const int32_t *sRp = reinterpret_cast<const int32_t *>(smem_raw + static_cast<uint32_t>(b) * buf_bytes + a_stage_bytes);
            cp_async_wait_group<1>();   // this thread's row_ptr entries of the current stage
            __syncthreads();            // ... and everybody else's

            const int s_lo = max(j_lo, sRp[0]);
            const int s_hi = min(j_hi, sRp[nr]);
            int cached_row = -1;      // row whose A chunks sit in areg
            int cached_end = 0;       // first nonzero index past that row
            float4 areg[CPL];
#pragma unroll
            for (int q = 0; q < CPL; ++q) areg[q] = make_float4(0.f, 0.f, 0.f, 0.f);

            // 32-aligned warp windows so every col/val/P access is a full 128-byte line.  The column
            // indices and S values of the NEXT window are requested before the current one is
            // processed, so the gather of B rows never waits behind an index load.
            int wb = (s_lo & ~31) + warp * 32;
            int4 pc0 = make_int4(0, 0, 0, 0), pc1 = make_int4(0, 0, 0, 0);
            float ps = 0.f;
            auto request_window = [&](int w) {
                const int jw = w + lane;
                if ((w >= s_lo) && (w + 32 <= s_hi)) {
                    pc0 = __ldcs(reinterpret_cast<const int4 *>(args.col_idx + w + gbase));
                    pc1 = __ldcs(reinterpret_cast<const int4 *>(args.col_idx + w + gbase + 4));
                    ps = __ldcs(args.s_val + jw);
                } else {
                    pc0.x = 0;
                    ps = 0.f;
                    if ((jw >= s_lo) && (jw < s_hi)) {
                        pc0.x = __ldcs(args.col_idx + jw);
                        ps = __ldcs(args.s_val + jw);
                    }
                }
            };
            if (wb < s_hi) request_window(wb);   // in flight while the A rows land
            if (!mbar_wait_bounded(&bar[b], (phases >> b) & 1u)) {
                atomicCAS(args.err, kDevOk, kDevMbarrierTimeout);
                // every thread of the CTA waits on the same phase, so all leave together -- after the copies
                // already requested for the next stage have landed (bounded again)
                cp_async_wait_all();
                if (has_next) mbar_wait_bounded(&bar[b ^ 1], (phases >> (b ^ 1)) & 1u);
                return;
            }
            phases ^= 1u << b;
            for (; wb < s_hi; wb += kRowTileWarps * 32) {
                const int j = wb + lane;
                const bool full = (wb >= s_lo) && (wb + 32 <= s_hi);   // warp-uniform
                bool valid = full || ((j >= s_lo) && (j < s_hi));

                // ---- column indices of this group's 8 nonzeros, S value of this lane's nonzero ----
                int ci[8];
                const float s = ps;
                if (full) {
                    ci[0] = pc0.x; ci[1] = pc0.y; ci[2] = pc0.z; ci[3] = pc0.w;
                    ci[4] = pc1.x; ci[5] = pc1.y; ci[6] = pc1.z; ci[7] = pc1.w;
                } else {
                    const int c_own = pc0.x;
#pragma unroll
                    for (int i = 0; i < 8; ++i) ci[i] = __shfl_sync(kFullMask, c_own, gbase + i);  // invalid -> row 0 of B, result unused
                }
                if (wb + kRowTileWarps * 32 < s_hi) request_window(wb + kRowTileWarps * 32);

                // ---- row of every nonzero of the window --------------------------------------
                bool uni;
                int lr;
                if (full && cached_row >= 0 && wb + 32 <= cached_end) {
                    uni = true;
                    lr = cached_row;
                } else {
                    // largest t with sRp[t] <= j (out-of-window lanes are clamped so rows stay monotone)
                    const int jj = min(max(j, s_lo), s_hi - 1);
                    int lo = 0, hi = nr;
                    while (hi - lo > 1) {
                        const int mid = (lo + hi) >> 1;
                        if (sRp[mid] <= jj) lo = mid; else hi = mid;
                    }
                    lr = lo;
                    const int rf = __shfl_sync(kFullMask, lr, 0), rl = __shfl_sync(kFullMask, lr, 31);
                    uni = (rf == rl);
                    if (uni) {
                        if (rf != cached_row) {
                            cached_row = rf;
#pragma unroll
                            for (int q = 0; q < CPL; ++q) {
                                const int ch = gl + 8 * q;
                                areg[q] = (EXACT || ch < nchunks) ? chunk_to_f4(sAc[rf * nchunks + ch]) : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
                        cached_end = sRp[rf + 1];
                    }
                }
                if (args.covered) {   // the window is 32-aligned: its 32 ownership bits are one word
                    const uint32_t word = __ldg(args.covered + (wb >> 5));
                    if ((word >> lane) & 1u) valid = false;
                    if (__ballot_sync(kFullMask, valid) == 0u) continue;
                }

                // ---- gather B rows, multiply with A chunks --------------------------------------
                float acc[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = 0.f;

                if (uni) {
#pragma unroll
                    for (int q0 = 0; q0 < CPL; q0 += QS) {
                        chunk_t bq[8][QS];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const unsigned char *brow = Bl + static_cast<uint64_t>(static_cast<uint32_t>(ci[i])) * row_bytes;
#pragma unroll
                            for (int qq = 0; qq < QS; ++qq) {
                                const int ch = gl + 8 * (q0 + qq);
                                bq[i][qq] = (EXACT || ch < nchunks)
                                                ? ldg_chunk(reinterpret_cast<const chunk_t *>(brow) + 8 * (q0 + qq))
                                                : zero_chunk(chunk_t());
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i)
#pragma unroll
                            for (int qq = 0; qq < QS; ++qq) acc[i] = dot4(areg[q0 + qq], chunk_to_f4(bq[i][qq]), acc[i]);
                    }
                } else {
                    // per-nonzero row offsets (in chunks) of this group's 8 nonzeros, through a warp-private smem line
                    __syncwarp();
                    sRowOff[warp][lane] = lr * nchunks;  // row start in chunks
                    __syncwarp();
                    const int4 o0 = *reinterpret_cast<const int4 *>(&sRowOff[warp][gbase]);
                    const int4 o1 = *reinterpret_cast<const int4 *>(&sRowOff[warp][gbase + 4]);
                    const int ro[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
                    for (int q0 = 0; q0 < CPL; q0 += QS) {
                        chunk_t bq[8][QS];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const unsigned char *brow = Bl + static_cast<uint64_t>(static_cast<uint32_t>(ci[i])) * row_bytes;
#pragma unroll
                            for (int qq = 0; qq < QS; ++qq) {
                                const int ch = gl + 8 * (q0 + qq);
                                bq[i][qq] = (EXACT || ch < nchunks)
                                                ? ldg_chunk(reinterpret_cast<const chunk_t *>(brow) + 8 * (q0 + qq))
                                                : zero_chunk(chunk_t());
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
#pragma unroll
                            for (int qq = 0; qq < QS; ++qq) {
                                const int ch = gl + 8 * (q0 + qq);
                                const float4 a = (EXACT || ch < nchunks) ? chunk_to_f4(sAc[ro[i] + ch]) : make_float4(0.f, 0.f, 0.f, 0.f);
                                acc[i] = dot4(a, chunk_to_f4(bq[i][qq]), acc[i]);
                            }
                        }
                    }
                }
                const float dot = group8_transpose_reduce(acc, gl);
                if (valid) __stcs(args.p_val + j, dot * s);
            }
            __syncthreads();  // all reads of this buffer done before the stage after the next one overwrites it
        }
        if (!has_next) break;
        if (r0 + R <= r_hi) {
            r0 += R;
        } else {
            it += gridDim.x;
            load_item(it, j_lo, j_hi, r_lo, r_hi);
            r0 = r_lo;
        }
        nr = min(R, r_hi - r0 + 1);
        b ^= 1;
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
