// Row-segment SDDMM kernel: the path for short and power-law rows.
//
// Work decomposition (no atomics, exactly one writer per nonzero):
//   * every row is cut into SEGMENTS of at most 8 consecutive nonzeros; the list of segments
//     ("units": first CSR position, row, count) is built once per upload on the device, so the
//     kernel itself searches nothing and stages nothing -- it is one streaming loop;
//   * a warp step takes 4 consecutive units, one per 8-lane group.  Inside a group lane l loads
//     column index l and S value l of the segment (one 32-byte access per group), the 8 column
//     indices are exchanged with shuffles, every B row is read as one contiguous line by the
//     group (lane = one 16-byte chunk; K > 32: more chunks per lane, 8 independent gathers per
//     lane in flight), the lane's chunk of the ONE A row of the segment sits in registers, and
//     the K-dot is reduced with the transposing shuffle tree that leaves nonzero l on lane l, so
//     P.val is written by the lane that read S.val;
//   * the unit two steps ahead and the column indices / S values one step ahead are requested
//     before the current gathers are consumed.
//
// Column panels: when B is much larger than the L2 cache the unit list is built PANEL-MAJOR --
// the columns are cut into P panels, a row contributes one run of segments per panel it touches,
// and all segments of panel 0 come before those of panel 1 and so on.  All CTAs walk the list in
// step, so the gathers of a panel find their B rows in L2 (the B loads carry an L2 evict_last
// hint, the streams evict_first).  col_idx, S.val and P.val stay in CSR order: a run is a
// contiguous piece of its row.
//
// A "chunk" is 4 consecutive K elements (8 for wide bf16 chunks).  CPL = chunks per lane, so K <= 8 * CPL chunks.
// EXACT = (K == 8 * CPL chunks): no chunk-range predicates in the inner loop.
#pragma once

#include "device_utils.cuh"

namespace sddmm {

// unit.x = CSR position of the first nonzero of the segment; unit.y = row * 8 + (count - 1)
constexpr int kUnitRowLimit = 1 << 28;   // rows the encoding can name

struct RowSegArgs {
    const int2 *units;        // n_units (> 0)
    const int32_t *col_idx;   // nnz
    const float *s_val;       // nnz
    float *p_val;             // nnz
    const void *A;            // M x K, element type ET
    const void *B;            // N x K, element type ET
    int32_t n_units;
    int32_t K;
    int32_t b_evict_last;     // B gathers ask L2 to keep their lines (column panels)
    float b_fraction;         // share of the B lines the hint applies to (1 = all)
    // column panels: copies of the units' column indices and S values, 8 slots of {column, value} per unit in list order
    // (slots past the segment's end repeat its last nonzero): one 8-byte load per lane.  A panel run is a short piece of its
    // row, so reading col_idx / S.val in place would touch one or two 32-byte sectors of a 128-byte line per unit; the
    // copies are read front to back.  unit_sval is the same array (the values are its odd words).
    const int32_t *unit_cols;
    const float *unit_sval;
    // K in slices (large K, B far larger than L2): the launch covers columns [k0, k0 + K) of rows that are row_stride bytes
    // apart (A and B point at column k0; 0 = rows of exactly K elements) and, from the second slice on, adds to P.val
    uint32_t row_stride;
    int32_t accumulate;
};

constexpr int kRowSegWarps = 8;
#ifndef SDDMM_ROWSEG_MINB1
#define SDDMM_ROWSEG_MINB1 4   // resident CTAs per SM the compiler must allow for, K <= 32
#endif
#ifndef SDDMM_ROWSEG_MINBN
#define SDDMM_ROWSEG_MINBN 2   // same, K > 32
#endif

// ---- L2 cache policy and loads that carry one (column panels) ------------------------------
__device__ __forceinline__ uint64_t policy_evict_last(float fraction) {
    uint64_t p;
    asm("createpolicy.fractional.L2::evict_last.b64 %0, %1;" : "=l"(p) : "f"(fraction));
    return p;
}
// (read-only data and always-valid addresses: plain asm, the compiler may schedule these freely)
__device__ __forceinline__ float4 ld_chunk_hint(const float4 *p, uint64_t pol) {
    float4 v;
    asm("ld.global.nc.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ uint2 ld_chunk_hint(const uint2 *p, uint64_t pol) {
    uint2 v;
    asm("ld.global.nc.L2::cache_hint.v2.u32 {%0, %1}, [%2], %3;" : "=r"(v.x), "=r"(v.y) : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ uint4 ld_chunk_hint(const uint4 *p, uint64_t pol) {
    uint4 v;
    asm("ld.global.nc.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol));
    return v;
}

// HINT: column panels -- the B gathers carry the L2 evict_last policy and column indices / S values come from the
// per-unit copies (one instantiation with, one without: no branch per load).
// SLICED: the launch covers a 64-column slice of longer rows (args.row_stride apart) and may add to P.val.
// The add-to-P.val path (a predicated load of the old value at the top of a step, used by the final multiply-add) is
// also compiled into the HINT instantiations although only slices switch it on: measured on the Poisson-rows
// configuration with two column panels, K = 32, 575 -> 525 us per launch with it (the load is never issued; it changes
// how the compiler groups the step's gathers into waits), while the instantiations without panels lose 6 % with it
// (power-law rows 569 -> 604 us) and therefore do not carry it.
template <int CPL, bool EXACT, typename ET, bool HINT, bool SLICED = false>
__global__ void __launch_bounds__(kRowSegWarps * 32, (CPL == 1) ? SDDMM_ROWSEG_MINB1 : SDDMM_ROWSEG_MINBN) sddmm_rowseg_kernel(const RowSegArgs args) {
    using chunk_t = typename ChunkOf<ET>::type;
    using areg_t = typename ChunkOf<ET>::areg;
    const int lane = threadIdx.x & 31;
    const int gl = lane & 7;          // lane inside its 8-lane group = chunk of a 128-byte piece = nonzero of the segment
    const int gbase = lane & 24;      // first lane of the group
    const int grp = lane >> 3;        // which of the warp's 4 units
    const int nchunks = EXACT ? 8 * CPL : (args.K / ChunkOf<ET>::elems);
    const uint32_t row_bytes = SLICED ? args.row_stride : static_cast<uint32_t>(nchunks) * sizeof(chunk_t);   // distance between rows
    constexpr bool kAccumulates = HINT || SLICED;
    constexpr int QS = (CPL >= 2) ? 2 : 1;   // chunks gathered per nonzero per step
    // chunks of this lane that exist (K < 32 * CPL: the lane's last chunks lie past the row and are read as chunk 0, times zero)
    uint64_t pol_b = 0;
    if (HINT) pol_b = policy_evict_last(args.b_fraction);

    const int64_t n_quads = (static_cast<int64_t>(args.n_units) + 3) >> 2;
    const int64_t n_warps = static_cast<int64_t>(gridDim.x) * kRowSegWarps;
    int64_t q = static_cast<int64_t>(blockIdx.x) * kRowSegWarps + (threadIdx.x >> 5);
    if (q >= n_quads) return;
    const int last_unit = args.n_units - 1;

    // per lane: byte offset of its chunk c inside a row, and whether the chunk exists
    uint32_t ch_off[CPL];
    float ch_on[CPL];
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
        const int ch = gl + 8 * c;
        const bool on = EXACT || ch < nchunks;
        ch_off[c] = static_cast<uint32_t>(on ? ch : 0) * sizeof(chunk_t);
        ch_on[c] = on ? 1.f : 0.f;
    }
    const unsigned char *Ab = reinterpret_cast<const unsigned char *>(args.A);
    const unsigned char *Bb = reinterpret_cast<const unsigned char *>(args.B);

    // Every load below is unconditional and in range: a group past the end of the list repeats the last unit, a lane
    // past the end of its segment repeats the segment's last nonzero; only the final store is predicated.
    auto unit_index = [&](int64_t qq) -> int64_t { const int64_t u = 4 * qq + grp; return u < last_unit ? u : last_unit; };
    auto load_unit = [&](int64_t qq) -> int2 { return __ldcs(args.units + unit_index(qq)); };
    auto own_slot = [&](const int2 &u) -> int { return u.x + min(gl, u.y & 7); };
    // column index / S value of this lane's nonzero of a unit, read in place (u: that unit's header)
    auto own_col = [&](int64_t, const int2 &u) -> int { return __ldcs(args.col_idx + own_slot(u)); };
    auto own_val = [&](int64_t, const int2 &u) -> float { return __ldcs(args.s_val + own_slot(u)); };

    // (HINT: column index and S value of a slot lie side by side in the per-unit copies: one 8-byte load)
    auto own_pair = [&](int64_t qq) -> int2 { return __ldcs(reinterpret_cast<const int2 *>(args.unit_cols) + 8 * unit_index(qq) + gl); };
    int2 u_cur = load_unit(q);
    int2 u_nxt = load_unit(q + n_warps);
    int c_own;
    float s_own;
    if (HINT) {
        const int2 cs = own_pair(q);
        c_own = cs.x;
        s_own = __int_as_float(cs.y);
    } else {
        c_own = own_col(q, u_cur);
        s_own = own_val(q, u_cur);
    }

    while (true) {
        const int row = u_cur.y >> 3;
        const int j = u_cur.x + gl;
        const bool valid = (gl <= (u_cur.y & 7)) && (4 * q + grp <= last_unit);
        const float s = s_own;
        float p_old = 0.f;   // (a later K slice: what the earlier slices left, requested before the gathers)
        if (kAccumulates && args.accumulate && valid) p_old = __ldcs(args.p_val + j);

        // ---- this lane's chunk(s) of the segment's A row ----
        areg_t areg[CPL];
        {
            const unsigned char *arow = Ab + static_cast<uint64_t>(static_cast<uint32_t>(row)) * row_bytes;
#pragma unroll
            for (int c = 0; c < CPL; ++c) {
                areg[c] = unpack_chunk(ldg_chunk(reinterpret_cast<const chunk_t *>(arow + ch_off[c])));
                if (!EXACT) scale_chunk(areg[c], ch_on[c]);
            }
        }
        // ---- the 8 column indices of the segment ----
        const unsigned char *brow[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            brow[i] = Bb + static_cast<uint64_t>(static_cast<uint32_t>(__shfl_sync(kFullMask, c_own, gbase + i))) * row_bytes;

        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;

        // ---- gather B rows (first pass), then request what the next steps need, then multiply ----
        chunk_t bq[8][QS];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int qq = 0; qq < QS; ++qq) {
                const chunk_t *src = reinterpret_cast<const chunk_t *>(brow[i] + ch_off[qq]);
                bq[i][qq] = HINT ? ld_chunk_hint(src, pol_b) : ldg_chunk(src);
            }
        const int64_t q_next = q + n_warps;
        const int2 u_nxt2 = load_unit(q_next + n_warps);
        if (HINT) {
            const int2 cs = own_pair(q_next);
            c_own = cs.x;
            s_own = __int_as_float(cs.y);
        } else {
            c_own = own_col(q_next, u_nxt);
            s_own = own_val(q_next, u_nxt);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int qq = 0; qq < QS; ++qq) acc[i] = dot_chunk(areg[qq], unpack_chunk(bq[i][qq]), acc[i]);
        // more than QS chunks per lane: the remaining chunks of the same 8 rows
#pragma unroll
        for (int q0 = QS; q0 < CPL; q0 += QS) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int qq = 0; qq < QS; ++qq) {
                    const chunk_t *src = reinterpret_cast<const chunk_t *>(brow[i] + ch_off[q0 + qq]);
                    bq[i][qq] = HINT ? ld_chunk_hint(src, pol_b) : ldg_chunk(src);
                }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int qq = 0; qq < QS; ++qq) acc[i] = dot_chunk(areg[q0 + qq], unpack_chunk(bq[i][qq]), acc[i]);
        }
        const float dot = group8_transpose_reduce(acc, gl);   // lane gl: nonzero gl of the segment
        if (valid) __stcs(args.p_val + j, kAccumulates ? fmaf(dot, s, p_old) : dot * s);

        q = q_next;
        if (q >= n_quads) break;   // warp-uniform
        u_cur = u_nxt;
        u_nxt = u_nxt2;
    }
}

// ---- row groups: segments shared by NR consecutive rows with identical column lists ---------------
// Block-structured matrices (several unknowns per mesh node) repeat one column list over the G rows of a block row.
// A unit of such a group covers 8 columns of the shared list for all G rows: each B row is gathered ONCE and dotted
// with G rows of A, so the traffic between L2 and the SM -- what bounds the gather -- drops by the factor G.
//   ghdr[u]  .x = CSR position of the segment in the group's first row, .y = first row * 8 + (count - 1),
//            .z = row length L (row t of the group holds the segment at .x + t * L: equal lengths, consecutive rows),
//            .w = rows that share the unit (1 for rows outside matching groups, else G)
// fp32 storage, K = 32 * CPL, CPL in {1, 2}; NR = G.
struct RowSegGroupArgs {
    const int4 *ghdr;         // n_units (> 0)
    const int32_t *col_idx;   // nnz
    const float *s_val;       // nnz
    float *p_val;             // nnz
    const float *A;           // M x K
    const float *B;           // N x K
    int32_t n_units;
    int32_t K;
};

// (K = 32: three resident CTAs per SM -- 207 against 273 us on the banded 3x3-block configuration at K = 32; K = 64 needs
// the registers of two)
template <int CPL, int NR>
__global__ void __launch_bounds__(kRowSegWarps * 32, (CPL == 1) ? 3 : 2) sddmm_rowseg_group_kernel(const RowSegGroupArgs args) {
    const int lane = threadIdx.x & 31;
    const int gl = lane & 7;
    const int gbase = lane & 24;
    const int grp = lane >> 3;
    constexpr uint32_t row_bytes = 8 * CPL * sizeof(float4);

    const int64_t n_quads = (static_cast<int64_t>(args.n_units) + 3) >> 2;
    const int64_t n_warps = static_cast<int64_t>(gridDim.x) * kRowSegWarps;
    int64_t q = static_cast<int64_t>(blockIdx.x) * kRowSegWarps + (threadIdx.x >> 5);
    if (q >= n_quads) return;
    const int last_unit = args.n_units - 1;
    const unsigned char *Ab = reinterpret_cast<const unsigned char *>(args.A) + gl * sizeof(float4);
    const unsigned char *Bb = reinterpret_cast<const unsigned char *>(args.B) + gl * sizeof(float4);

    // every load is unconditional and in range (clamped unit, clamped slot, clamped row of the group); stores are predicated
    auto load_unit = [&](int64_t qq) -> int4 {
        const int64_t u = 4 * qq + grp;
        return __ldcs(args.ghdr + (u < last_unit ? u : last_unit));
    };
    auto own_slot = [&](const int4 &u) -> int { return u.x + min(gl, u.y & 7); };

    int4 u_cur = load_unit(q);
    int4 u_nxt = load_unit(q + n_warps);
    int c_own = __ldcs(args.col_idx + own_slot(u_cur));

    while (true) {
        const int row = u_cur.y >> 3;
        const int rows = u_cur.w;      // 1 .. NR
        const int L = u_cur.z;
        const int slot = own_slot(u_cur);
        const bool valid = (gl <= (u_cur.y & 7)) && (4 * q + grp <= last_unit);

        // S values of this lane's nonzero in every row of the group (used after the dots)
        float sv[NR];
#pragma unroll
        for (int t = 0; t < NR; ++t) sv[t] = __ldcs(args.s_val + slot + min(t, rows - 1) * L);
        // this lane's chunks of the group's A rows
        float4 areg[NR][CPL];
#pragma unroll
        for (int t = 0; t < NR; ++t) {
            const unsigned char *arow = Ab + static_cast<uint64_t>(static_cast<uint32_t>(row + min(t, rows - 1))) * row_bytes;
#pragma unroll
            for (int c = 0; c < CPL; ++c) areg[t][c] = __ldg(reinterpret_cast<const float4 *>(arow) + 8 * c);
        }
        const unsigned char *brow[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            brow[i] = Bb + static_cast<uint64_t>(static_cast<uint32_t>(__shfl_sync(kFullMask, c_own, gbase + i))) * row_bytes;

        float acc[NR][8];
#pragma unroll
        for (int t = 0; t < NR; ++t)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[t][i] = 0.f;

        // one 128-byte piece of the 8 B rows at a time: gathered once, used by every row of the group
        float4 bq[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) bq[i] = __ldg(reinterpret_cast<const float4 *>(brow[i]));
        const int64_t q_next = q + n_warps;
        const int4 u_nxt2 = load_unit(q_next + n_warps);
        c_own = __ldcs(args.col_idx + own_slot(u_nxt));
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
#pragma unroll
            for (int t = 0; t < NR; ++t)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[t][i] = dot4(areg[t][c], bq[i], acc[t][i]);
            if (c + 1 < CPL) {
#pragma unroll
                for (int i = 0; i < 8; ++i) bq[i] = __ldg(reinterpret_cast<const float4 *>(brow[i]) + 8 * (c + 1));
            }
        }
#pragma unroll
        for (int t = 0; t < NR; ++t) {
            const float dot = group8_transpose_reduce(acc[t], gl);
            if (valid && t < rows) __stcs(args.p_val + u_cur.x + gl + t * L, dot * sv[t]);
        }

        q = q_next;
        if (q >= n_quads) break;   // warp-uniform
        u_cur = u_nxt;
        u_nxt = u_nxt2;
    }
}

// rows of group g when groups of G rows start at row `first` (group 0 = the rows before it)
__device__ __forceinline__ void unit_group_rows(int32_t g, int32_t G, int32_t first, int32_t M, int32_t &r0, int32_t &r1) {
    r0 = g == 0 ? 0 : first + (g - 1) * G;
    r1 = g == 0 ? first : min(r0 + G, M);
}
// one thread per row: units the row contributes -- the leader of a matching group speaks for its whole group
__global__ void k_group_unit_count(const int32_t *__restrict__ rp, int32_t M, int32_t G, int32_t first, const uint8_t *__restrict__ group_ok,
                                   int32_t *__restrict__ counts) {
    for (int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; r < M; r += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int32_t g = r < first ? 0 : 1 + static_cast<int32_t>((r - first) / G);
        int32_t r0, r1;
        unit_group_rows(g, G, first, M, r0, r1);
        const int32_t len = rp[r + 1] - rp[r];
        counts[r] = (group_ok[g] && r != r0) ? 0 : (len + 7) >> 3;
    }
}
// one warp per row: write its units at the scanned offset
__global__ void k_group_unit_fill(const int32_t *__restrict__ rp, int32_t M, int32_t G, int32_t first, const uint8_t *__restrict__ group_ok,
                                  const int32_t *__restrict__ offsets, int4 *__restrict__ ghdr) {
    const int lane = threadIdx.x & 31;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t r = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5; r < M; r += n_warps) {
        const int32_t g = r < first ? 0 : 1 + static_cast<int32_t>((r - first) / G);
        int32_t r0, r1;
        unit_group_rows(g, G, first, M, r0, r1);
        const bool matched = group_ok[g] != 0;
        if (matched && r != r0) continue;
        const int32_t s = rp[r], e = rp[r + 1];
        const int32_t n_units = (e - s + 7) >> 3;
        const int32_t off = offsets[r];
        for (int32_t u = lane; u < n_units; u += 32) {
            const int32_t start = s + 8 * u;
            ghdr[off + u] = make_int4(start, static_cast<int32_t>(r) * 8 + (min(8, e - start) - 1), e - s, matched ? G : 1);
        }
    }
}

// ---- building the unit list (once per upload) -------------------------------------------
// Run of row i inside column panel p: [s, e) in CSR positions.  One panel: the whole row.
// Needs non-decreasing column indices inside a row when there is more than one panel.
// long_rows > 0: only rows of at least that many nonzeros are cut into column panels (panels 0 .. panels-2, panel_cols
// columns each); the shorter rows follow whole, as the last "panel" of the list -- a run of one or two nonzeros would
// leave most of a segment's slots empty.
__device__ __forceinline__ void panel_run(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t i, int32_t p,
                                          int32_t panels, int32_t panel_cols, int32_t long_rows, int32_t &s, int32_t &e) {
    const int32_t a = rp[i], b = rp[i + 1];
    if (panels == 1) {
        s = a;
        e = b;
        return;
    }
    if (long_rows > 0) {
        const bool is_long = b - a >= long_rows;
        if (p == panels - 1) {           // the short rows, whole
            s = a;
            e = is_long ? a : b;
            return;
        }
        if (!is_long) {
            s = e = a;
            return;
        }
        --panels;                        // the real column panels
    }
    auto lower = [&](int64_t c) {   // first position whose column is >= c
        int32_t lo = a, hi = b;
        while (lo < hi) {
            const int32_t mid = (lo + hi) >> 1;
            if (col[mid] < c) lo = mid + 1; else hi = mid;
        }
        return lo;
    };
    s = (p == 0) ? a : lower(static_cast<int64_t>(p) * panel_cols);
    e = (p == panels - 1) ? b : lower(static_cast<int64_t>(p + 1) * panel_cols);
}

// one thread per (panel, row), panel-major: number of units of that run
__global__ void k_unit_count(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t M, int32_t panels,
                             int32_t panel_cols, int32_t long_rows, int32_t *__restrict__ counts) {
    const int64_t n = static_cast<int64_t>(panels) * M;
    for (int64_t qi = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; qi < n;
         qi += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int32_t p = static_cast<int32_t>(qi / M), i = static_cast<int32_t>(qi - static_cast<int64_t>(p) * M);
        int32_t s, e;
        panel_run(rp, col, i, p, panels, panel_cols, long_rows, s, e);
        counts[qi] = (e - s + 7) >> 3;
    }
}

// one warp per (panel, row): write its units at the scanned offset
__global__ void k_unit_fill(const int32_t *__restrict__ rp, const int32_t *__restrict__ col, int32_t M, int32_t panels,
                            int32_t panel_cols, int32_t long_rows, const int32_t *__restrict__ offsets, int2 *__restrict__ units,
                            int32_t *__restrict__ ucols) {
    const int lane = threadIdx.x & 31;
    const int64_t n = static_cast<int64_t>(panels) * M;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t qi = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5; qi < n; qi += n_warps) {
        const int32_t p = static_cast<int32_t>(qi / M), i = static_cast<int32_t>(qi - static_cast<int64_t>(p) * M);
        int32_t s, e;
        panel_run(rp, col, i, p, panels, panel_cols, long_rows, s, e);
        const int32_t n_units = (e - s + 7) >> 3;
        const int32_t off = offsets[qi];
        for (int32_t u = lane; u < n_units; u += 32) {
            const int32_t first = s + 8 * u;
            const int32_t cnt = min(8, e - first);
            units[off + u] = make_int2(first, i * 8 + (cnt - 1));
        }
        if (ucols)   // per-unit copies of the column indices (slots past the end of the run repeat its last column)
            for (int32_t t = lane; t < 8 * n_units; t += 32) ucols[2 * (8 * static_cast<int64_t>(off) + t)] = col[min(s + t, e - 1)];
    }
}

// per-unit copies of the S values (one thread per slot): refreshed whenever S.val changes
__global__ void k_unit_values(const int2 *__restrict__ units, int32_t n_units, const float *__restrict__ s_val, float *__restrict__ usval) {   // usval: the {column, value} slots
    for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < 8 * static_cast<int64_t>(n_units);
         t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int2 u = units[t >> 3];
        usval[2 * t + 1] = s_val[u.x + min(static_cast<int>(t & 7), u.y & 7)];
    }
}

// ---- units over what the dense tiles left: runs of nonzeros whose bit in `covered` is clear -----------------------
// first position in [j, b) whose bit equals `want`, or b
__device__ __forceinline__ int32_t next_bit(const uint32_t *__restrict__ bits, int32_t j, int32_t b, bool want) {
    while (j < b) {
        uint32_t word = bits[j >> 5];
        if (!want) word = ~word;
        word >>= (j & 31);
        if (word) return min(b, j + __ffs(word) - 1);
        j = (j | 31) + 1;
    }
    return b;
}
// one thread per row: units of its uncovered runs
__global__ void k_residual_unit_count(const int32_t *__restrict__ rp, int32_t M, const uint32_t *__restrict__ covered, int32_t *__restrict__ counts) {
    for (int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; r < M; r += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int32_t b = rp[r + 1];
        int32_t n = 0;
        for (int32_t j = next_bit(covered, rp[r], b, false); j < b;) {
            const int32_t e = next_bit(covered, j, b, true);
            n += (e - j + 7) >> 3;
            j = next_bit(covered, e, b, false);
        }
        counts[r] = n;
    }
}
__global__ void k_residual_unit_fill(const int32_t *__restrict__ rp, int32_t M, const uint32_t *__restrict__ covered,
                                     const int32_t *__restrict__ offsets, int2 *__restrict__ units) {
    for (int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; r < M; r += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int32_t b = rp[r + 1];
        int32_t off = offsets[r];
        for (int32_t j = next_bit(covered, rp[r], b, false); j < b;) {
            const int32_t e = next_bit(covered, j, b, true);
            for (int32_t first = j; first < e; first += 8) units[off++] = make_int2(first, static_cast<int32_t>(r) * 8 + (min(8, e - first) - 1));
            j = next_bit(covered, e, b, false);
        }
    }
}

// ---- exclusive scan of int32 counts (three small kernels) -----------------------------------
constexpr int kScanBlock = 256;
constexpr int kScanPerThread = 8;
constexpr int kScanTile = kScanBlock * kScanPerThread;

__device__ __forceinline__ int32_t warp_inclusive_scan(int32_t v, int lane) {
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int32_t t = __shfl_up_sync(kFullMask, v, off);
        if (lane >= off) v += t;
    }
    return v;
}
// inclusive scan of one value per thread over a block of kScanBlock threads; returns the thread's inclusive prefix,
// *total = block sum
__device__ __forceinline__ int32_t block_inclusive_scan(int32_t v, int32_t *total) {
    __shared__ int32_t warp_sums[kScanBlock / 32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int32_t inc = warp_inclusive_scan(v, lane);
    if (lane == 31) warp_sums[w] = inc;
    __syncthreads();
    int32_t base = 0, tot = 0;
#pragma unroll
    for (int k = 0; k < kScanBlock / 32; ++k) {
        const int32_t t = warp_sums[k];
        if (k < w) base += t;
        tot += t;
    }
    __syncthreads();
    *total = tot;
    return inc + base;
}

// pass 1: sum of every tile of kScanTile values
__global__ void __launch_bounds__(kScanBlock) k_scan_tile_sums(const int32_t *__restrict__ v, int64_t n, int32_t *__restrict__ tile_sums) {
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + static_cast<int64_t>(threadIdx.x) * kScanPerThread;
    int32_t local = 0;
#pragma unroll
    for (int k = 0; k < kScanPerThread; ++k)
        if (base + k < n) local += v[base + k];
    int32_t total;
    block_inclusive_scan(local, &total);
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}
// pass 2 (one block): exclusive scan of the tile sums in place; *grand_total = sum of everything
__global__ void __launch_bounds__(kScanBlock) k_scan_sums(int32_t *__restrict__ tile_sums, int32_t n_tiles, unsigned long long *__restrict__ grand_total) {
    int64_t carry = 0;
    for (int32_t base = 0; base < n_tiles; base += kScanBlock) {
        const int32_t idx = base + static_cast<int32_t>(threadIdx.x);
        const int32_t v = idx < n_tiles ? tile_sums[idx] : 0;
        int32_t total;
        const int32_t inc = block_inclusive_scan(v, &total);
        if (idx < n_tiles) tile_sums[idx] = static_cast<int32_t>(carry) + inc - v;
        carry += total;
    }
    if (threadIdx.x == 0) *grand_total = static_cast<unsigned long long>(carry);
}
// pass 3: exclusive scan inside every tile plus the tile's offset, in place
__global__ void __launch_bounds__(kScanBlock) k_scan_apply(int32_t *__restrict__ v, int64_t n, const int32_t *__restrict__ tile_offsets) {
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + static_cast<int64_t>(threadIdx.x) * kScanPerThread;
    int32_t x[kScanPerThread];
    int32_t local = 0;
#pragma unroll
    for (int k = 0; k < kScanPerThread; ++k) {
        x[k] = (base + k < n) ? v[base + k] : 0;
        local += x[k];
    }
    int32_t total;
    const int32_t inc = block_inclusive_scan(local, &total);
    int32_t run = tile_offsets[blockIdx.x] + inc - local;
#pragma unroll
    for (int k = 0; k < kScanPerThread; ++k) {
        if (base + k < n) v[base + k] = run;
        run += x[k];
    }
}

}  // namespace sddmm
