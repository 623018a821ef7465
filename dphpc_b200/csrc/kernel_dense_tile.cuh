// Dense-tile SDDMM kernel: 64x64 tiles of S that are at least half full are
// computed as dense A_tile * B_tile^T products on the 5th-generation tensor
// cores (tcgen05.mma, fp32 accumulators in tensor memory) and then sampled
// through a per-row presence mask.
//
// A job is a PAIR of dense tiles.  Their 64 A rows each are stacked into one
// 128-row operand, their 64 B rows each into one 128-row operand, and ONE
// M=128, N=128 MMA computes both 64x64 products on the diagonal blocks of the
// accumulator (the two off-diagonal blocks are never read; tensor throughput is
// not what bounds this path).  Accumulator row r lives in TMEM lane r.
//
// Per job:
//   producer thread   TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, no
//                     multicast) of the operand rows into shared memory,
//                     completion on an mbarrier; then issues the tcgen05.mma
//                     k-steps and tcgen05.commit
//   8 epilogue warps  tcgen05.ld the accumulator (thread = row), park it in
//                     shared memory, then one warp per tile row streams that
//                     row: lane l owns columns 2l and 2l+1, a 64-bit presence
//                     mask says which of them are nonzeros of S, the rank of
//                     the column inside the mask is the offset from the row's
//                     first nonzero in the tile.  S.val is read and P.val is
//                     written in CSR order in contiguous runs; col_idx is not
//                     read at all (the mask, built once per upload, replaces it).
//                     The S.val run of every tile row is staged in shared memory
//                     by asynchronous 16-byte copies issued most of a job ahead,
//                     the row records (first position, mask) two jobs ahead: no
//                     warp waits for global memory inside a job.
//
// Modes: plain tf32 operands (rel 1e-2), or fp32-grade results from tf32 tensor cores: the
// engine stores A' = [A_lo | A_hi | A_hi] and B' = [B_hi | B_lo | B_hi] (hi = tf32(x),
// lo = tf32(x - hi)), so that A'.B'^T = lo*hi + hi*lo + hi*hi is just a 3x longer K for this
// kernel -- one code path for both modes.
// K' must be a multiple of 32; every 32-wide k-block is one 128-byte swizzle atom.  There is one
// operand buffer: the next k-block is requested as soon as the MMAs of the current one have read
// it, which for K' = 32 still overlaps the whole epilogue of the job (shared memory goes to the
// S.val staging instead, so that two CTAs fit on an SM).
//
// Every wait on an mbarrier is bounded; on a timeout the CTA sets the error
// word, stops issuing work, and still frees its tensor memory.
#pragma once

#include <cuda.h>

#include "device_utils.cuh"

#ifndef SDDMM_DENSE_BATCH
#define SDDMM_DENSE_BATCH 4
#endif

namespace sddmm {

constexpr int kDenseTile = 64;               // tile edge
constexpr int kDenseEpiWarps = 8;
constexpr int kDenseThreads = (kDenseEpiWarps + 1) * 32;   // + producer/MMA warp
constexpr int kDenseAccStride = 66;          // floats per accumulator row in smem (even: rows are read and written as 8-byte column pairs)
constexpr int kDenseSvalStride = 72;         // floats per staged S.val row: 64 + up to 3 before + up to 3 after (16-byte granules), 288 bytes
constexpr uint32_t kOperandBytes = 128 * 128;  // 128 rows x one 128-byte k-block
constexpr uint32_t kHalfOperandBytes = 64 * 128;
constexpr int kTmemCols = 128;
constexpr int kDenseCtasPerSm = 2;          // resident CTAs per SM the kernel is sized for (shared memory, registers)

// Per dense tile: first nonzero of each of its 64 rows inside the tile's column
// range (CSR position), which of the 64 columns are present, and which of those
// this tile computes (tiles at arbitrary offsets may overlap: a nonzero is owned
// by exactly one of them; for tiles that do not overlap own == mask).
struct DenseTileDesc {
    int32_t start[kDenseTile];
    unsigned long long mask[kDenseTile];
    unsigned long long own[kDenseTile];
};

struct DenseArgs {
    const int2 *origins;            // n_tiles dense tiles: {first row, first column}, any offset
    const DenseTileDesc *descs;     // n_tiles
    const float *s_val;
    float *p_val;
    int32_t *err;
    int32_t n_tiles;
    int32_t k_blocks;               // operand row length / 32
    int64_t nnz;                    // bound of every S.val / P.val position (checked builds only)
};

// shared memory carve-up (dynamic, 1024-byte aligned by hand).
// SPLIT3 (the fp32-grade mode, three tf32 products per 32 columns of K): three 16 KB operand slots instead of one
// A block + one B block, and room for the accumulator of ONE tile of the pair at a time -- see the kernel.
template <bool SPLIT3>
struct DenseSmemT {
    static constexpr uint32_t kStageBytes = (SPLIT3 ? 3 : 2) * kOperandBytes;   // A block + B block (+ a third slot)
    static constexpr uint32_t kStage0 = 0;                        // operand slots, 16 KB each, back to back
    static constexpr uint32_t kAcc = kStageBytes;
    static constexpr uint32_t kAccRows = SPLIT3 ? 64 : 128;
    static constexpr uint32_t kAccBytes = kAccRows * kDenseAccStride * 4;
    static constexpr uint32_t kSval = kAcc + kAccBytes;           // 128 rows x kDenseSvalStride floats: the S.val run of each tile row, as it lies in memory
    static constexpr uint32_t kSvalBytes = 128 * kDenseSvalStride * 4;
    static constexpr uint32_t kRows = kSval + kSvalBytes;         // 3 buffers x 128 row records {first CSR position, 16-byte granules of the run, mask lo, mask hi}
    static constexpr uint32_t kOwn = kRows + 3 * 128 * 16;        // 3 buffers x 128 own masks {lo, hi}
    static constexpr uint32_t kBars = kOwn + 3 * 128 * 8;         // 10 mbarriers (4 used without SPLIT3)
    static constexpr uint32_t kTmemPtr = kBars + 10 * 8;
    static constexpr uint32_t kTmemColumns = SPLIT3 ? 2 * kTmemCols : kTmemCols;   // SPLIT3: two accumulators, used alternately
    static constexpr uint32_t kTotal = kTmemPtr + 16;
    static constexpr uint32_t kDynamicBytes = kTotal + 1024;      // slack for the manual 1024-byte alignment
};
using DenseSmem = DenseSmemT<false>;

__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(dst_smem)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart, sm_100 descriptor version 1
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                       // leading byte offset (unused for swizzled K-major)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;               // stride byte offset: next 8-row group
    d |= static_cast<uint64_t>(1) << 46;                       // descriptor version
    d |= static_cast<uint64_t>(2) << 61;                       // SWIZZLE_128B
    return d;
}

// kind::tf32, fp32 accumulate, both operands K-major, M = 128, N = 128
constexpr uint32_t kIdescTf32 = (1u << 4) | (2u << 7) | (2u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(kIdescTf32), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// TMEM -> registers, 32 lanes x 32 columns.  The load is asynchronous: its destination registers
// are only defined after tcgen05.wait::ld, so both instructions live in ONE asm statement --
// otherwise the compiler is free to consume or recycle the registers in between.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void epi_barrier() {  // the 8 epilogue warps only
    asm volatile("bar.sync 1, %0;" ::"n"(kDenseEpiWarps * 32) : "memory");
}

// OWN = false: the tiles do not overlap (tiles on the 64-grid), every present nonzero is the tile's own and the own masks
// are neither fetched nor looked at.
//
// SPLIT3 = true (fp32-grade mode; operand rows [A_lo | A_hi | A_hi] and [B_hi | B_lo | B_hi], each part K wide): per
// 32 columns of K the accumulator takes A_hi.B_lo + A_hi.B_hi + A_lo.B_hi.  With one A block + one B block in shared
// memory that is three TMA round trips in a row per job, which -- not the epilogue -- then sets the pace.  Here the
// four distinct 16 KB operand blocks go through THREE slots: X <- A_hi, Y <- B_lo, Z <- B_hi are requested together,
// MMA(X, Y) and MMA(X, Z) run as they land, Y is refilled with A_lo as soon as MMA(X, Y) has read it, then MMA(Y, Z):
// two round trips per job, and X of the next job is requested while Y is on its way.  The third slot is paid for by
// parking the accumulator of one tile of the pair at a time (64 rows instead of 128): tile 0 is moved out of tensor
// memory and sampled, then tile 1 -- the epilogue has the time, the tensor memory is released after the second move.
template <bool OWN, bool SPLIT3>
__global__ void __launch_bounds__(kDenseThreads, kDenseCtasPerSm)
sddmm_dense_tile_kernel(const DenseArgs args, const __grid_constant__ CUtensorMap map_a,
                        const __grid_constant__ CUtensorMap map_b) {
    using DenseSmem = DenseSmemT<SPLIT3>;
    extern __shared__ unsigned char dense_smem_raw[];
    // 1024-byte alignment by an OFFSET into the shared array (not by rounding a generic address): every pointer below
    // stays a shared-memory pointer for the compiler, so its loads and stores are shared-space instructions that it may
    // reorder against the global stores of the sampling loop
    unsigned char *smem = dense_smem_raw + ((1024u - (smem_u32(dense_smem_raw) & 1023u)) & 1023u);
    float *sAcc = reinterpret_cast<float *>(smem + DenseSmem::kAcc);
    float *sSval = reinterpret_cast<float *>(smem + DenseSmem::kSval);
    uint4 *sRows = reinterpret_cast<uint4 *>(smem + DenseSmem::kRows);
    uint2 *sOwn = reinterpret_cast<uint2 *>(smem + DenseSmem::kOwn);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + DenseSmem::kBars);
    uint64_t *ops_full = &bars[0], *ops_free = &bars[1], *acc_full = &bars[2], *acc_free = &bars[3];
    uint64_t *slot_full = &bars[4];   // SPLIT3: [4..6] = slot X, Y, Z filled (bars[0], [1], [7] = slot released)
    auto slot_free = [&](int sl) -> uint64_t * { return sl == 0 ? &bars[0] : sl == 1 ? &bars[1] : &bars[7]; };
    // SPLIT3 keeps two accumulators in tensor memory (job n in buffer n & 1: bars[2], [3] for buffer 0, bars[8], [9] for buffer 1),
    // so the MMAs of the next job never wait for the epilogue of this one
    auto acc_full_of = [&](uint32_t b) -> uint64_t * { return b ? &bars[8] : acc_full; };
    auto acc_free_of = [&](uint32_t b) -> uint64_t * { return b ? &bars[9] : acc_free; };
    uint32_t *tmem_ptr_smem = reinterpret_cast<uint32_t *>(smem + DenseSmem::kTmemPtr);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int n_jobs = (args.n_tiles + 1) >> 1;

    // Start-up, kept short: the producer thread initialises the barriers itself and requests the operands of its first
    // job at once; the epilogue warps request the row records of their first job; only then does the CTA meet at the
    // barrier behind which the tensor memory address is known.
    const bool is_producer = (tid == kDenseEpiWarps * 32);
    int2 first0 = make_int2(0, 0), first1 = make_int2(0, 0);   // producer: tile origins of the CTA's first job
    if (is_producer) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
        if (static_cast<int>(blockIdx.x) < n_jobs) {
            first0 = args.origins[2 * blockIdx.x];
            first1 = (2 * static_cast<int>(blockIdx.x) + 1 < args.n_tiles) ? args.origins[2 * blockIdx.x + 1] : first0;
        }
        mbar_init(ops_full, 1);
        mbar_init(ops_free, 1);
        mbar_init(acc_full, 1);
        mbar_init(acc_free, kDenseEpiWarps);
        if (SPLIT3) {
            mbar_init(&bars[4], 1);
            mbar_init(&bars[5], 1);
            mbar_init(&bars[6], 1);
            mbar_init(&bars[7], 1);
            mbar_init(&bars[8], 1);
            mbar_init(&bars[9], kDenseEpiWarps);
        }
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == 0) {  // one warp allocates the tensor memory for the CTA
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr_smem)), "r"(DenseSmem::kTmemColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // ---- producer state and helpers (used by the one producer thread) ----
    // Iterations = (job, k-block) pairs of this CTA in order.  The TMA of iteration it + 1 is issued
    // right after the MMAs of iteration it (it waits for them to release the operand buffer).
    const int kbs = args.k_blocks;
    const int my_jobs = (n_jobs - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    const uint32_t total = static_cast<uint32_t>(my_jobs) * static_cast<uint32_t>(kbs);
    int2 cur0 = first0, cur1 = first1, nxt0 = first0, nxt1 = first0;   // origins of the job being requested / of the one after (read a job ahead of their use)
    bool prod_ok = true;
    // tile origins of a job (the second tile of the last job may be missing: its operands repeat the first)
    auto load_ids = [&](uint32_t j, int2 &t0, int2 &t1) {
        const int job = static_cast<int>(blockIdx.x) + static_cast<int>(j) * static_cast<int>(gridDim.x);
        t0 = args.origins[2 * job];
        t1 = ((2 * job + 1) < args.n_tiles) ? args.origins[2 * job + 1] : t0;
    };
    // request operand k-block `it` (called once per it, in order)
    auto issue_tma = [&](uint32_t it) -> bool {
        const uint32_t ph = it & 1u;
        const uint32_t j = it / kbs;
        const int kb = static_cast<int>(it % kbs);
        if (kb == 0 && it > 0) {
            cur0 = nxt0;
            cur1 = nxt1;
            if (j + 1 < static_cast<uint32_t>(my_jobs)) load_ids(j + 1, nxt0, nxt1);
        }
        // (TMA coordinates: x = k offset, a multiple of 32 floats = 128 bytes; y = any row index, rows past the end read as zero)
        const int r0 = cur0.x, c0 = cur0.y, r1 = cur1.x, c1 = cur1.y;
        // operand buffer free again?  (read by the MMAs of k-block it - 1)
        if (!mbar_wait_bounded(ops_free, ph ^ 1u)) return false;
        unsigned char *sa = smem + DenseSmem::kStage0;
        unsigned char *sb = sa + kOperandBytes;
        mbar_expect_tx(ops_full, DenseSmem::kStageBytes);
        const int x = kb * 32;
        tma_load_2d(sa, &map_a, x, r0, ops_full);
        tma_load_2d(sa + kHalfOperandBytes, &map_a, x, r1, ops_full);
        tma_load_2d(sb, &map_b, x, c0, ops_full);
        tma_load_2d(sb + kHalfOperandBytes, &map_b, x, c1, ops_full);
        return true;
    };
    // raw descriptors of one job -> record buffer `buf` (threads 0..127: one tile row each)
    auto fetch_rows = [&](int job, int buf) {
        if (tid < 128 && job < n_jobs) {
            uint4 *dst = sRows + buf * 128 + tid;
            const int t = 2 * job + (tid >> 6);
            if (t < args.n_tiles) {
                const DenseTileDesc *d = args.descs + t;
                cp_async_4(&dst->x, &d->start[tid & 63]);
                cp_async_8(&dst->z, &d->mask[tid & 63]);
                if (OWN) cp_async_8(sOwn + buf * 128 + tid, &d->own[tid & 63]);
            } else {
                *dst = make_uint4(0u, 0u, 0u, 0u);
                if (OWN) sOwn[buf * 128 + tid] = make_uint2(0u, 0u);
            }
        }
    };

    // ---- SPLIT3 producer: three operand slots (0 = X, 1 = Y, 2 = Z), iterations = (job, 32 columns of K) ----
    const int kk_per_job = kbs / 3;                     // 32-column pieces of K
    const int k_cols = kk_per_job * 32;                 // K: the width of each of the three parts of an operand row
    const uint32_t total3 = static_cast<uint32_t>(my_jobs) * static_cast<uint32_t>(kk_per_job);
    uint32_t n_rel[3] = {0u, 0u, 0u};                   // fills requested per slot (the k-th waits for the (k-1)-th release)
    uint32_t n_fill[3] = {0u, 0u, 0u};                  // fills consumed per slot
    auto slot_ptr = [&](int sl) -> unsigned char * { return smem + DenseSmem::kStage0 + static_cast<uint32_t>(sl) * kOperandBytes; };
    // request 128 operand rows (64 of each tile of the pair) x 32 columns starting at column x into a slot
    auto fill_slot = [&](int sl, const CUtensorMap *map, int x, int row_a, int row_b) -> bool {
        if (!mbar_wait_bounded(slot_free(sl), (n_rel[sl] & 1u) ^ 1u)) return false;   // read by the MMAs that used it last?
        ++n_rel[sl];
        unsigned char *dst = slot_ptr(sl);
        mbar_expect_tx(&slot_full[sl], kOperandBytes);
        tma_load_2d(dst, map, x, row_a, &slot_full[sl]);
        tma_load_2d(dst + kHalfOperandBytes, map, x, row_b, &slot_full[sl]);
        return true;
    };
    auto slot_landed = [&](int sl) -> bool {
        const bool landed = mbar_wait_bounded(&slot_full[sl], n_fill[sl] & 1u);
        ++n_fill[sl];
        return landed;
    };

    // ---- before the CTA barrier: first operand request (producer), first row records (epilogue warps) ----
    if (is_producer) {
        if (my_jobs > 1) load_ids(1, nxt0, nxt1);
        if (SPLIT3) {
            if (total3 > 0)   // A_hi, B_lo, B_hi of the first 32 columns of the first job
                prod_ok = fill_slot(0, &map_a, k_cols, cur0.x, cur1.x) && fill_slot(1, &map_b, k_cols, cur0.y, cur1.y) &&
                          fill_slot(2, &map_b, 0, cur0.y, cur1.y);
        } else if (total > 0) {
            prod_ok = issue_tma(0);
        }
    } else if (warp < kDenseEpiWarps && static_cast<int>(blockIdx.x) < n_jobs) {
        fetch_rows(blockIdx.x, 0);
        cp_async_commit();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;

    if (warp == kDenseEpiWarps) {
        // ===================== producer + MMA issuer (one thread) =====================
        if (lane == 0 && SPLIT3) {
            bool ok = prod_ok;
            uint32_t jb = 0;  // jobs whose MMAs have been issued (phase of acc_free / acc_full)
            auto mma4 = [&](int sa, int sb, bool fresh) {   // 4 k-steps of 8 tf32 = 32 bytes inside the swizzle atom
                const uint32_t a_s = smem_u32(slot_ptr(sa)), b_s = smem_u32(slot_ptr(sb));
                const uint32_t d_tmem = tmem_base + (jb & 1u) * static_cast<uint32_t>(kTmemCols);   // this job's accumulator
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint32_t adv = static_cast<uint32_t>(ks) * 32u;
                    umma_tf32(d_tmem, umma_smem_desc(a_s + adv), umma_smem_desc(b_s + adv), (fresh && ks == 0) ? 0u : 1u);
                }
            };
            for (uint32_t it = 0; it < total3 && ok; ++it) {
                const int kk = static_cast<int>(it % static_cast<uint32_t>(kk_per_job));
                const bool last_kk = kk == kk_per_job - 1;
                const bool more = it + 1 < total3;
                // the iteration after this one: same job, next 32 columns -- or the first 32 columns of the next job
                const int kk_n = last_kk ? 0 : kk + 1;
                const int2 n0 = last_kk ? nxt0 : cur0, n1 = last_kk ? nxt1 : cur1;
                if (!slot_landed(0) || !slot_landed(1)) { ok = false; break; }           // A_hi, B_lo
                // this job's accumulator drained by the epilogue of the job before last?
                if (kk == 0 && !mbar_wait_bounded(acc_free_of(jb & 1u), ((jb >> 1) & 1u) ^ 1u)) { ok = false; break; }
                tcgen05_fence_after();
                mma4(0, 1, kk == 0);                                                     // A_hi . B_lo
                umma_commit(slot_free(1));
                if (!slot_landed(2)) { ok = false; break; }                              // B_hi
                tcgen05_fence_after();
                mma4(0, 2, false);                                                       // A_hi . B_hi
                umma_commit(slot_free(0));
                if (!fill_slot(1, &map_a, 32 * kk, cur0.x, cur1.x)) { ok = false; break; }                     // Y <- A_lo (once A_hi . B_lo has read it)
                if (more && !fill_slot(0, &map_a, k_cols + 32 * kk_n, n0.x, n1.x)) { ok = false; break; }      // X <- A_hi of the next iteration, on its way meanwhile
                if (!slot_landed(1)) { ok = false; break; }
                tcgen05_fence_after();
                mma4(1, 2, false);                                                       // A_lo . B_hi
                umma_commit(slot_free(1));
                umma_commit(slot_free(2));
                if (last_kk) {
                    umma_commit(acc_full_of(jb & 1u));   // arrives once the accumulator of this job is complete
                    ++jb;
                }
                if (more && !(fill_slot(1, &map_b, k_cols + 32 * kk_n, n0.y, n1.y) && fill_slot(2, &map_b, 32 * kk_n, n0.y, n1.y))) { ok = false; break; }
                if (last_kk && more) {
                    cur0 = nxt0;
                    cur1 = nxt1;
                    const uint32_t j = it / static_cast<uint32_t>(kk_per_job);
                    if (j + 2 < static_cast<uint32_t>(my_jobs)) load_ids(j + 2, nxt0, nxt1);
                }
            }
            if (!ok) atomicCAS(args.err, kDevOk, kDevMbarrierTimeout);
        } else if (lane == 0) {
            bool ok = prod_ok;
            uint32_t jb = 0;  // jobs whose MMAs have been issued (phase of acc_free / acc_full)
            for (uint32_t it = 0; it < total && ok; ++it) {
                const int kb = static_cast<int>(it % kbs);
                if (!mbar_wait_bounded(ops_full, it & 1u)) { ok = false; break; }
                if (kb == 0) {
                    // accumulator drained by the epilogue of the previous job?
                    if (!mbar_wait_bounded(acc_free, (jb & 1u) ^ 1u)) { ok = false; break; }
                }
                tcgen05_fence_after();
                const uint32_t a_s = smem_u32(smem + DenseSmem::kStage0);
                const uint32_t b_s = a_s + kOperandBytes;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {  // 4 k-steps of 8 tf32 = 32 bytes inside the swizzle atom
                    const uint32_t adv = static_cast<uint32_t>(ks) * 32u;
                    umma_tf32(tmem_base, umma_smem_desc(a_s + adv), umma_smem_desc(b_s + adv), (kb > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(ops_free);       // arrives once the MMAs above have read their operands
                if (kb == kbs - 1) {
                    umma_commit(acc_full);   // arrives once the accumulator of this job is complete
                    ++jb;
                }
                if (it + 1 < total && !issue_tma(it + 1)) { ok = false; break; }   // refill the operand buffer
            }
            if (!ok) atomicCAS(args.err, kDevOk, kDevMbarrierTimeout);
        }
    } else {
        // ===================== epilogue warps =====================
        // Tile row r belongs to warp r % 8 for the whole kernel (16 rows per warp, two halves of 8).
        // S.val: the nonzeros of a tile row are one contiguous CSR run; widened to 16-byte granules it
        // is at most 18 of them, copied with asynchronous 16-byte copies (one per lane, two rows per
        // instruction) into the row's slot of sSval.  A half is requested for the next job as soon as the warp has
        // sampled it for this job, so the copies run most of a job ahead and no warp waits for
        // global memory.  Row records (first position, granules, presence mask) run two jobs ahead.
        // Sampling: lane l owns the adjacent tile columns 2l and 2l+1 (one 8-byte read of the parked
        // accumulator); the mask says which are nonzeros and the popcount below column 2l is the offset
        // inside the run -> S.val from shared memory, P.val written in contiguous CSR runs; col_idx is
        // never read.
        //
        // cp.async groups of a thread, oldest first, at the points that wait (always "all but 2"):
        //   before the mid barrier of job n:  [R(n+1)] [A(n)] [B(n)]      -> records of job n+1 landed
        //   before sampling half A of job n:  [A(n)] [B(n)] [R(n+2)]      -> A(n) landed
        //   before sampling half B of job n:  [B(n)] [R(n+2)] [A(n+1)]    -> B(n) landed
        const int q = warp & 3;               // TMEM lane quarter this warp may read: rows 32q .. 32q+31
        const int h = warp >> 2;              // which 32 of the tile's 64 columns this warp moves
        const int tile_of_q = q >> 1;         // rows 0-63: first tile, rows 64-127: second tile
        const bool upper = lane >= 16;                        // columns 2l, 2l+1 sit in the upper mask word
        const uint32_t pshift = (2u * lane) & 31u;            // bit of column 2l inside its mask word
        const uint32_t pbelow = (1u << pshift) - 1u;
        const int stride_jobs = static_cast<int>(gridDim.x);

        // ... and, once they have landed (same thread), the number of 16-byte granules that cover the run
        auto finish_rows = [&](int job, int buf) {
            if (tid < 128 && job < n_jobs) {
                uint4 *dst = sRows + buf * 128 + tid;
                const uint4 d = *dst;
                const uint32_t lo = __popc(d.z), cnt = lo + __popc(d.w);
                dst->y = (cnt ? ((d.x & 3u) + cnt + 3u) >> 2 : 0u) | (lo << 8);   // granules | nonzeros in columns 0..31
            }
        };
        // two rows per instruction: lanes 0..15 copy granules 0..15 of one row, lanes 16..31 those of the next;
        // a run of 64 that does not start on a granule boundary needs granules 16 (and 17): a second, rarely taken, step
        auto request_half = [&](int buf, int half) {
            const int side = lane >> 4, g = lane & 15;
#pragma unroll
            for (int u = 0; u < 8; u += 2) {
                const int r = (8 * half + u + side) * kDenseEpiWarps + warp;
                const uint4 d = sRows[buf * 128 + r];
                const int n = static_cast<int>(d.y & 0xFFu);
                float *dst = sSval + r * kDenseSvalStride;
                const float *src = args.s_val + (d.x & ~3u);
                if (g < n) cp_async_16(dst + 4 * g, src + 4 * g);
                if (__any_sync(kFullMask, n > 16)) {
                    if (g + 16 < n) cp_async_16(dst + 4 * (g + 16), src + 4 * (g + 16));
                }
            }
        };
        auto sample_half = [&](int buf, int half) {
            // four rows at a time, every shared-memory read of the batch issued before the first store: the reads are
            // unconditional (an absent nonzero reads a word of the row's own slot and drops it), so nothing orders them
            // behind the predicated global stores of the previous row
            constexpr int kBatch = SDDMM_DENSE_BATCH;
#pragma unroll
            for (int u0 = 0; u0 < 8; u0 += kBatch) {
                uint4 d[kBatch];
                uint2 o[kBatch];
                float2 a[kBatch];
                float s0[kBatch], s1[kBatch];
                int pos[kBatch];
                uint32_t present[kBatch], pair[kBatch];
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    const int r = (8 * half + u0 + i) * kDenseEpiWarps + warp;
                    d[i] = sRows[buf * 128 + r];
                    o[i] = OWN ? sOwn[buf * 128 + r] : make_uint2(d[i].z, d[i].w);
                }
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    // lane l owns the adjacent columns 2l and 2l+1: one 8-byte read of the accumulator pair; the second
                    // column's nonzero (if any) directly follows the first one's in the run.  Positions come from the
                    // PRESENCE mask, what is written from the OWN mask.
                    const int r = (8 * half + u0 + i) * kDenseEpiWarps + warp;
                    const int st = static_cast<int>(d[i].x);
                    const uint32_t w = upper ? d[i].w : d[i].z;                       // the mask word that holds this lane's two bits
                    present[i] = (w >> pshift) & 3u;
                    pair[i] = ((upper ? o[i].y : o[i].x) >> pshift) & 3u;
                    const int k0 = (upper ? static_cast<int>(d[i].y >> 8) : 0) + __popc(w & pbelow);   // offset of column 2l inside the run
                    a[i] = *reinterpret_cast<const float2 *>(sAcc + (SPLIT3 ? (r & 63) : r) * kDenseAccStride + 2 * lane);
                    const float *srow = sSval + r * kDenseSvalStride + (st & 3) + k0;
                    s0[i] = srow[0];
                    s1[i] = srow[present[i] & 1u];
                    pos[i] = st + k0;
                }
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    float *prow = args.p_val + pos[i];
                    if (pair[i] & 1u) __stcs(prow, a[i].x * s0[i]);
                    if (pair[i] & 2u) __stcs(prow + (present[i] & 1u), a[i].y * s1[i]);
                }
            }
        };

        uint32_t jb = 0;
        bool ok = true;
        if (static_cast<int>(blockIdx.x) < n_jobs) {   // first job of the CTA: the only exposed fetches (requested before the CTA barrier)
            cp_async_wait_group<0>();
            finish_rows(blockIdx.x, 0);
            epi_barrier();
            fetch_rows(blockIdx.x + stride_jobs, 1);
            cp_async_commit();
            request_half(0, 0);
            cp_async_commit();
            request_half(0, 1);
            cp_async_commit();
        }
        for (int job = blockIdx.x; job < n_jobs; job += stride_jobs, ++jb) {
            const int buf = static_cast<int>(jb % 3u), buf1 = static_cast<int>((jb + 1u) % 3u), buf2 = static_cast<int>((jb + 2u) % 3u);
            const bool has_next = job + stride_jobs < n_jobs;
            if (ok) {   // one lane polls, then the warp re-converges before the warp-wide tcgen05.ld
                int got = 1;
                if (lane == 0) {
                    got = (SPLIT3 ? mbar_wait_bounded(acc_full_of(jb & 1u), (jb >> 1) & 1u) : mbar_wait_bounded(acc_full, jb & 1u)) ? 1 : 0;
                    if (!got) atomicCAS(args.err, kDevOk, kDevMbarrierTimeout);
                }
                __syncwarp();
                ok = __shfl_sync(kFullMask, got, 0) != 0;
            }
            // accumulator rows of this warp's tensor-memory lanes -> shared memory (thread = row), then release the tensor memory
            auto park = [&]() {
                if (ok) {
                    tcgen05_fence_after();
                    uint32_t v[32];
                    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(32 * q) << 16) + static_cast<uint32_t>(64 * tile_of_q + 32 * h) +
                                           (SPLIT3 ? (jb & 1u) * static_cast<uint32_t>(kTmemCols) : 0u);
                    tmem_ld_32x32b_x32(taddr, v);
                    tcgen05_fence_before();
                    float *row = sAcc + (32 * (SPLIT3 ? (q & 1) : q) + lane) * kDenseAccStride + 32 * h;
#pragma unroll
                    for (int c = 0; c < 32; c += 2)
                        *reinterpret_cast<float2 *>(row + c) = make_float2(__uint_as_float(v[c]), __uint_as_float(v[c + 1]));
                }
            };
            if (!SPLIT3 || tile_of_q == 0) park();
            cp_async_wait_group<2>();               // this thread's share of the next job's records
            finish_rows(job + stride_jobs, buf1);
            __syncwarp();
            if ((!SPLIT3 || tile_of_q == 0) && lane == 0) mbar_arrive(SPLIT3 ? acc_free_of(jb & 1u) : acc_free);   // (all 8 warps have arrived: that accumulator may be overwritten)
            epi_barrier();                          // accumulator + next job's records visible to all epilogue warps
            fetch_rows(job + 2 * stride_jobs, buf2);
            cp_async_commit();
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                if (SPLIT3 && half == 1) {          // the second tile of the pair takes the place of the first
                    epi_barrier();                  // every warp is done with the first tile's accumulator
                    if (tile_of_q == 1) {
                        park();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_free_of(jb & 1u));
                    }
                    epi_barrier();
                }
                cp_async_wait_group<2>();   // this lane's granules of this half ...
                __syncwarp();               // ... and every other lane's
                if (ok) sample_half(buf, half);
                __syncwarp();               // every lane is done with the slots of this half before they are overwritten
                if (has_next) request_half(buf1, half);
                cp_async_commit();
            }
            epi_barrier();  // all rows streamed before the next job overwrites sAcc / the oldest record buffer
        }
        cp_async_wait_group<0>();
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(DenseSmem::kTmemColumns) : "memory");
    }
}

}  // namespace sddmm
