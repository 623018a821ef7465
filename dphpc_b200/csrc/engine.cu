// C-ABI implementation of the B200 SDDMM engine (see include/sddmm_b200.h).
//
// One engine = one CUDA device, one stream, one device arena that is reused
// across uploads.  upload_*() copies the operands, validates the pattern on the
// device, builds the row-length histogram and the kernel plan; run() enqueues
// the kernels between two CUDA events; download() copies P.val back.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <utility>
#include <vector>

#include "../../include/sddmm_b200.h"
#include "host_staging.cuh"
#include "kernel_dense_tile.cuh"
#include "kernel_rowgroup.cuh"
#include "kernel_rowseg.cuh"
#include "kernel_rowtile.cuh"
#include "kernel_spmm.cuh"
#include "plan_kernels.cuh"

using namespace sddmm;

namespace {

constexpr size_t kAlign = 256;
constexpr int kBlock = 256;
constexpr int kMaxStageBytes = 32 * 1024;  // A rows per stage buffer (a CTA holds two)
constexpr int kDenseMinCount = 2048;       // a 64x64 tile is "dense" from half full

struct Arena {
    char *base = nullptr;
    size_t cap = 0;
};

struct Carve {
    size_t off = 0;
    size_t take(size_t bytes) {
        const size_t o = off;
        off += (bytes + kAlign - 1) / kAlign * kAlign;
        return o;
    }
};

}  // namespace

struct sddmm_b200_engine {
    int device = 0;
    int mode = SDDMM_B200_FP32;
    uint32_t flags = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t side_stream = nullptr;   // residual row-tile kernel runs here, concurrently with the dense tiles
    static constexpr int kMaxKernels = 4;
    cudaEvent_t ev_begin[kMaxKernels] = {nullptr, nullptr, nullptr, nullptr};  // per kernel, on the stream it runs on
    cudaEvent_t ev_end[kMaxKernels] = {nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t ev_run0 = nullptr, ev_run1 = nullptr;   // whole run(), on the main stream
    cudaEvent_t ev_join = nullptr;
    // chunked host-to-host calls (pipeline.cuh): copies of consecutive row chunks are chained through these
    cudaEvent_t ev_h2d = nullptr;                 // recorded after the upload's copies are enqueued
    cudaEvent_t h2d_after = nullptr;              // another engine's ev_h2d: this upload's copies start after it
    const float *B_on_device = nullptr;           // B already in this GPU's memory (another engine's copy): taken from there
    void (*on_copies_enqueued)(void *) = nullptr; // called once ev_h2d is recorded
    void *on_copies_user = nullptr;
    int32_t coo_row_base = 0;                     // COO upload of a row slice of a larger matrix: first row of the slice
    const char *kernel_name[kMaxKernels] = {nullptr, nullptr, nullptr, nullptr};
    int kernels_launched = 0;
    bool kernel_timing = false;    // record an event pair around every kernel (sddmm_b200_set_kernel_timing)
    bool last_run_timed = false;   // ... and whether the last run() did
    int sm_count = 148;
    char err[512] = {0};

    Arena arena;
    bool uploaded = false;
    bool ran = false;
    int64_t M = 0, N = 0, K = 0, nnz = 0;

    // device views into the arena
    int32_t *d_rp = nullptr, *d_col = nullptr;
    float *d_sval = nullptr, *d_pval = nullptr;
    float *d_A32 = nullptr, *d_B32 = nullptr;
    __nv_bfloat16 *d_A16 = nullptr, *d_B16 = nullptr;
    unsigned char *d_touched = nullptr;
    uint32_t *d_rowstart = nullptr;
    int2 *d_item_rows = nullptr;
    int32_t *d_coo_rows = nullptr;
    PlanCounters *d_pc = nullptr;
    int32_t *d_err = nullptr;
    int32_t *h_err = nullptr;  // pinned mirror of the device error word
    PlanCounters *h_pc = nullptr;  // pinned landing place of the plan counters (a pageable target would make the copy a staged, blocking one)

    // dense-tile (tensor-core) path
    bool dense_possible = false;   // buffers carved for this upload
    int64_t tile_grid = 0;         // (M/64 rounded up) * (N/64 rounded up)
    int32_t tiles_per_row = 0;
    int32_t dense_cap = 0;
    bool aligned_possible = false; // the 64-grid of aligned tiles is small enough to be counted cell by cell
    int32_t *d_tile_counts = nullptr;
    int2 *d_dense_origin = nullptr;     // {first row, first column} of every dense tile (aligned detection)
    int2 *d_dense_origin2 = nullptr;    // ... (arbitrary-offset detection); `dense_origin` points at the list in use
    const int2 *dense_origin = nullptr;
    bool dense_own = false;             // the tiles in use may overlap: the kernel looks at their own masks
    int seg_slices = 1;                 // row-segment path: K is taken in this many slices of 64 columns, one launch each
    bool dense_split3 = false;          // fp32-grade mode: operands through three slots, accumulator parked a tile at a time
    uint32_t *d_covered = nullptr;      // one bit per nonzero: owned by a dense tile
    uint32_t *d_cand = nullptr;         // one bit per nonzero: starts a half-full 64-column window of its row
    int2 *d_anchors = nullptr;          // candidate tile origins of the arbitrary-offset detection
    int32_t *d_anchor_counts = nullptr;
    int32_t anchor_cap = 0;
    DenseTileDesc *d_dense_descs = nullptr;
    int32_t *d_item_covered = nullptr;
    int32_t *d_item_ids = nullptr;
    float *d_Ax = nullptr, *d_Bx = nullptr;   // fp32_tc: [lo|hi|hi] and [hi|lo|hi] rows, 3K long
    CUtensorMap map_a, map_b;
    int32_t n_dense = 0;
    int32_t n_residual_items = 0;

    // row-group path (aligned groups of rows with one column list)
    uint8_t *d_group_ok = nullptr;
    int32_t rg_rows = 0;           // rows per group (2, 3, 4) when the row-group kernel runs, else 0
    int32_t rg_first = 0;          // first row of the first full group
    int32_t rg_groups = 0;         // ceil(M / rg_rows)

    // row-segment path (short and power-law rows; column panels when B is much larger than L2)
    int2 *d_units = nullptr;
    int32_t *d_unit_cols = nullptr;    // column panels: per-unit copies of column indices and S values, 8 slots of {column, value} per unit
    float *d_unit_sval = nullptr;      // (the same array: the values are its odd words)
    bool seg_copies = false;           // ... in use by the current plan
    int32_t *d_unit_off = nullptr;     // per (panel, row): units before it (scan of the counts)
    int32_t *d_scan_tiles = nullptr;
    int64_t unit_cap = 0;
    int32_t panels = 1;                // column panels the unit list is ordered by
    int32_t panel_cols = 0;            // columns per panel
    int32_t long_rows = 0;             // > 0: only rows of at least this many nonzeros are cut into panels, the others follow whole (as one more "panel")
    int32_t n_units = 0;
    bool use_seg = false;
    bool seg_residual = false;         // the row-segment kernel computes what the dense tiles left (units over the uncovered runs)
    int l2_bytes = 0;
    // tuning knobs (sddmm_b200_set_knob; defaults from the environment at create): < 0 = decide automatically
    double knob_panels = -1, knob_panel_mb = -1, knob_rowseg = -1, knob_b_fraction = -1, knob_group_units = -1,
           knob_offset_tiles = -1, knob_dense_split3 = -1, knob_k_slices = -1, knob_long_rows = -1;
    bool rg_units = false;             // row groups run as shared segments (row-segment group kernel) instead of the warp-per-group kernel

    HostStager stager, stager2;   // pageable host memory goes through pinned ring buffers filled by a pool of host threads (one per stream)

    // B received from another engine (sddmm_b200_stage_b): the next upload may pass B = NULL
    float *b_stage = nullptr;
    size_t b_stage_cap = 0;
    int64_t b_stage_n = 0, b_stage_k = 0;   // dimensions of the staged B (0: none)
    cudaEvent_t ev_stage = nullptr;

    // consumer of P on the device (Y = P X): its own buffers, grown on demand, and its own plain unit list
    Arena spmm_arena;
    int32_t spmm_units = 0;            // units in the consumer's list for the current upload (0: not built yet)
    int64_t spmm_k2 = 0;
    float *d_X = nullptr, *d_Y = nullptr;
    int2 *d_spmm_units = nullptr;
    cudaEvent_t ev_spmm0 = nullptr, ev_spmm1 = nullptr;

    // plan
    sddmm_b200_plan_info plan;
    bool use_scalar = false;
    int cpl = 1;
};

namespace {

int fail(sddmm_b200_engine *e, int code, const char *fmt, ...) {
    if (e) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(e->err, sizeof(e->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

#define CU_TRY(e, call)                                                                                  \
    do {                                                                                                 \
        cudaError_t _st = (call);                                                                        \
        if (_st != cudaSuccess) {                                                                        \
            return fail((e), _st == cudaErrorMemoryAllocation ? SDDMM_B200_ERR_OOM : SDDMM_B200_ERR_CUDA, \
                        "%s failed: %s (%s:%d)", #call, cudaGetErrorString(_st), __FILE__, __LINE__);    \
        }                                                                                                \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) ok = true;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

int grid_for(int64_t n, int block, int cap) {
    int64_t g = (n + block - 1) / block;
    if (g < 1) g = 1;
    if (g > cap) g = cap;
    return static_cast<int>(g);
}

int ensure_arena(sddmm_b200_engine *e, size_t bytes) {
    if (bytes <= e->arena.cap) return SDDMM_B200_OK;
    if (e->arena.base) {
        CU_TRY(e, cudaFree(e->arena.base));
        e->arena.base = nullptr;
        e->arena.cap = 0;
    }
    void *p = nullptr;
    cudaError_t st = cudaMalloc(&p, bytes);
    if (st != cudaSuccess) {
        cudaGetLastError();
        return fail(e, SDDMM_B200_ERR_OOM, "device arena of %zu bytes: %s", bytes, cudaGetErrorString(st));
    }
    e->arena.base = static_cast<char *>(p);
    e->arena.cap = bytes;
    return SDDMM_B200_OK;
}

// Upper bound of the row-tile kernel's dynamic shared memory: two buffers of kMaxStageBytes of A rows plus a row_ptr
// slice of at most kMaxStageBytes / 16 + 1 entries (the shortest staged row is 16 bytes).
constexpr int kRowTileMaxSmem = 2 * (kMaxStageBytes + (kMaxStageBytes / 16 + 1) * 4 + 32);

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a (function, device) pair, not to an engine: it is raised
// ONCE per pair to the upper bound, so that engines that share a GPU (chunked calls, a device listed twice, the
// allocation-free entry) can never leave each other with a limit below what their own launch asks for.
int ensure_dynamic_smem_limit(const void *fn, int device, int bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, int> raised;
    std::lock_guard<std::mutex> lock(mu);
    int &have = raised[{fn, device}];
    if (have >= bytes) return SDDMM_B200_OK;
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
        cudaGetLastError();
        return SDDMM_B200_ERR_CUDA;
    }
    have = bytes;
    return SDDMM_B200_OK;
}

template <typename ET>
using RowTileFn = void (*)(const RowTileArgs);

template <typename ET>
RowTileFn<ET> pick_rowtile(int cpl, bool exact) {
    switch (cpl) {
        case 1: return exact ? sddmm_rowtile_kernel<1, true, ET> : sddmm_rowtile_kernel<1, false, ET>;
        case 2: return exact ? sddmm_rowtile_kernel<2, true, ET> : sddmm_rowtile_kernel<2, false, ET>;
        case 4: return exact ? sddmm_rowtile_kernel<4, true, ET> : sddmm_rowtile_kernel<4, false, ET>;
        case 8: return exact ? sddmm_rowtile_kernel<8, true, ET> : sddmm_rowtile_kernel<8, false, ET>;
        default: return nullptr;
    }
}

int round_up_cpl(int64_t K) {
    const int64_t need = (K + 31) / 32;
    if (need <= 1) return 1;
    if (need <= 2) return 2;
    if (need <= 4) return 4;
    if (need <= 8) return 8;
    return 0;
}

size_t elem_bytes(const sddmm_b200_engine *e) { return e->mode == SDDMM_B200_BF16 ? 2 : 4; }

double env_double(const char *name, double fallback) {
    const char *v = std::getenv(name);
    return v ? std::atof(v) : fallback;
}

// Column panels of the row-segment path.  B is cut into panels when it is much larger than the L2 cache, so that the
// gathers of one panel hit in L2; every panel pass reads the A rows it touches again and shortens the runs a row
// contributes (a run of fewer than ~6 nonzeros leaves most of a segment's 8 slots empty), which bounds the count.
// Large K, fp32 storage, B far larger than L2: K is taken in slices of 64 columns, one launch of the K = 64 kernel per
// slice over the same unit list, each adding to P.val -- a slice of B is small enough for column panels to keep it in
// L2, where the whole rows are not (knob "k_slices": 0 = never, 1 = whenever K allows).
int choose_k_slices(const sddmm_b200_engine *e) {
    if (e->mode == SDDMM_B200_BF16 || e->K < 128 || e->K % 64 != 0 || e->knob_k_slices == 0) return 1;
    const double l2 = e->l2_bytes > 0 ? e->l2_bytes : 96.0 * (1 << 20);
    if (e->knob_k_slices < 0 && static_cast<double>(e->N) * e->K * 4.0 <= 4.0 * l2) return 1;
    // slices pay through the column panels they make room for; rows too short for panels are better off read whole
    // (power-law rows, mean length 14, K = 128: 2.04 ms whole against 2.12 ms in slices) -- unless the long rows get panels
    if (e->knob_k_slices < 0 && e->nnz / std::max<int64_t>(1, 8 * e->M) < 2 && e->knob_long_rows == 0) return 1;
    return static_cast<int>(e->K / 64);
}

// Rows too short for column panels on average, but B far larger than L2 (power-law row lengths: a few percent of the rows
// hold most of the nonzeros): column panels for the rows of at least `long_rows` nonzeros only, the shorter rows follow
// whole as one more entry of the panel-major list.  Returns the candidate threshold (0: not a candidate); e->panels is
// then the number of real panels.  The plan confirms it once the row-length statistics are known (build_rowseg_plan).
// Knob "long_rows": 0 = never, T >= 1 = threshold T with the panels the "panels" knob or the rule below gives.
bool long_rows_candidate(const sddmm_b200_engine *e) {
    if (e->knob_long_rows == 0) return false;
    const double l2 = e->l2_bytes > 0 ? e->l2_bytes : 96.0 * (1 << 20);
    return static_cast<double>(e->N) * (e->seg_slices > 1 ? 64 : e->K) * static_cast<double>(elem_bytes(e)) > l2 &&
           e->nnz / std::max<int64_t>(1, 8 * e->M) < 2;
}
int choose_long_rows(const sddmm_b200_engine *e) {
    if (e->knob_long_rows >= 1) return e->panels > 1 ? static_cast<int>(e->knob_long_rows) : 0;
    if (!long_rows_candidate(e) || e->panels < 2) return 0;
    return e->panels <= 4 ? 64 : 128;    // runs of 16 nonzeros or more on average (powers of two: the histogram's bins)
}

int choose_panels(const sddmm_b200_engine *e) {
    if (e->knob_panels >= 1 && e->knob_panels <= 64) return static_cast<int>(e->knob_panels);
    if (long_rows_candidate(e)) {   // measured on the power-law configuration (B 333 MB): 4 panels 458 us, 6 446 us, 8 442-447 us
        const double l2 = e->l2_bytes > 0 ? e->l2_bytes : 96.0 * (1 << 20);
        return static_cast<int>(std::max(2.0, std::min(8.0, std::ceil(static_cast<double>(e->N) * (e->seg_slices > 1 ? 64 : e->K) *
                                                                      static_cast<double>(elem_bytes(e)) / (0.5 * l2)))));
    }
    const double eb = static_cast<double>(elem_bytes(e));
    const double b_bytes = static_cast<double>(e->N) * (e->seg_slices > 1 ? 64 : e->K) * eb;
    const double l2 = e->l2_bytes > 0 ? e->l2_bytes : 96.0 * (1 << 20);
    if (b_bytes <= l2) return 1;
    if (e->mode == SDDMM_B200_BF16) return 1;   // measured: with bf16 storage the extra segments cost more than the saved DRAM reads
    // measured on B200 (126 MB of L2): panels of about 96 MB are as good as smaller ones, and a run shorter than a segment
    // wastes gather slots -- so at most one panel per 8 nonzeros of an average row, and never more than 4
    const double panel = e->knob_panel_mb > 0 ? e->knob_panel_mb * (1 << 20) : 0.75 * l2;
    int64_t p = static_cast<int64_t>((b_bytes + panel - 1) / panel);
    p = std::min<int64_t>(p, e->nnz / std::max<int64_t>(1, 8 * e->M));
    return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(p, 4)));
}

// Lay out the arena for the current dimensions and point the views into it.
int carve_arena(sddmm_b200_engine *e, bool coo, int n_items) {
    Carve c;
    const size_t nnz = static_cast<size_t>(e->nnz), M = static_cast<size_t>(e->M), N = static_cast<size_t>(e->N),
                 K = static_cast<size_t>(e->K);
    const size_t o_rp = c.take((M + 1) * 4);
    const size_t o_col = c.take(nnz * 4 + 16);
    const size_t o_sv = c.take(nnz * 4 + 16);
    const size_t o_pv = c.take(nnz * 4 + 16);
    const size_t o_A = c.take(M * K * 4);
    const size_t o_B = c.take(N * K * 4);
    const bool bf = e->mode == SDDMM_B200_BF16;
    const size_t o_A16 = bf ? c.take(M * K * 2) : 0;
    const size_t o_B16 = bf ? c.take(N * K * 2) : 0;
    const size_t o_touch = c.take(N);
    const size_t o_rs = c.take((nnz / 32 + 2) * 4);
    const size_t o_items = c.take(static_cast<size_t>(std::max(n_items, 1)) * sizeof(int2));
    const size_t o_coo = coo ? c.take(nnz * 4 + 16) : 0;
    const size_t o_pc = c.take(sizeof(PlanCounters));
    const size_t o_err = c.take(sizeof(int32_t));
    const size_t o_gok = c.take(M / 2 + 4);   // one byte per row group (groups of >= 2 rows, plus the leading partial group)
    // row-segment path: unit list (upper bound: one unit per 8 nonzeros plus one ragged unit per row and panel), scan scratch
    e->seg_slices = choose_k_slices(e);
    e->panels = choose_panels(e);
    e->long_rows = choose_long_rows(e);              // > 0: e->panels column panels for the long rows (still to be confirmed by the row statistics)
    e->panel_cols = static_cast<int32_t>((N + e->panels - 1) / e->panels);
    size_t runs = std::min(M * static_cast<size_t>(e->panels), nnz);
    if (e->long_rows > 0) {
        // a run per short row, and per panel for at most nnz / long_rows long rows
        runs = std::min(M + std::min(nnz / static_cast<size_t>(e->long_rows), M) * static_cast<size_t>(e->panels), nnz);
        e->panels += 1;                              // the short rows, whole, as the last entry of the list
    }
    e->unit_cap = static_cast<int64_t>(nnz / 8 + runs + 8);
    const size_t scan_n = M * static_cast<size_t>(e->panels);
    const size_t o_units = c.take(static_cast<size_t>(e->unit_cap) * sizeof(int4));   // (row groups use 16-byte headers)
    const size_t o_ucols = e->panels > 1 ? c.take(static_cast<size_t>(e->unit_cap) * 64) : 0;
    const size_t o_uoff = c.take((scan_n + 1) * 4);
    const size_t o_stile = c.take((scan_n / kScanTile + 2) * 4);
    // dense-tile path: only carved when the mode, K and the size of the 64x64 tile grid allow it
    e->tiles_per_row = static_cast<int32_t>((N + 63) / 64);
    e->tile_grid = static_cast<int64_t>((M + 63) / 64) * e->tiles_per_row;
    // tensor-core modes.  bf16 takes the same kind::tf32 kernel: the fp32 copies of A and B are rounded to bf16 in place at
    // upload, every bf16 value is exactly a tf32 value (8 against 11 significand bits), so the tile products are exactly the
    // bf16-input / fp32-accumulate ones.
    const bool tc_mode = e->mode == SDDMM_B200_TF32 || e->mode == SDDMM_B200_FP32_TC || e->mode == SDDMM_B200_BF16;
    e->dense_possible = tc_mode && !(e->flags & SDDMM_B200_FLAG_NO_DENSE_TILES) && K % 32 == 0 && K <= 256 && nnz >= kDenseMinCount;
    e->aligned_possible = e->dense_possible && e->tile_grid <= (int64_t(1) << 22);
    // (tiles at arbitrary offsets may overlap, so there can be more of them than nnz / 2048; what does not fit is dropped)
    e->dense_cap = e->dense_possible ? static_cast<int32_t>(2 * (e->nnz / kDenseMinCount) + 16) : 0;
    e->anchor_cap = e->dense_possible ? static_cast<int32_t>(e->nnz / 256 + 64) : 0;
    const bool split = e->dense_possible && e->mode == SDDMM_B200_FP32_TC;
    const size_t tg = static_cast<size_t>(e->tile_grid);
    const size_t o_tc = e->aligned_possible ? c.take(tg * 4) : 0;
    const size_t o_di = e->dense_possible ? c.take(static_cast<size_t>(e->dense_cap) * sizeof(int2)) : 0;
    const size_t o_di2 = e->dense_possible ? c.take(static_cast<size_t>(e->dense_cap) * sizeof(int2)) : 0;
    const size_t o_cov = e->dense_possible ? c.take((nnz / 32 + 2) * 4) : 0;
    const size_t o_cand = e->dense_possible ? c.take((nnz / 32 + 2) * 4) : 0;
    const size_t o_anc = e->dense_possible ? c.take(static_cast<size_t>(e->anchor_cap) * sizeof(int2)) : 0;
    const size_t o_ancc = e->dense_possible ? c.take(static_cast<size_t>(e->anchor_cap) * 4) : 0;
    const size_t o_dd = e->dense_possible ? c.take(static_cast<size_t>(e->dense_cap) * sizeof(DenseTileDesc)) : 0;
    const size_t o_ic = e->dense_possible ? c.take(static_cast<size_t>(std::max(n_items, 1)) * 4) : 0;
    const size_t o_ii = e->dense_possible ? c.take(static_cast<size_t>(std::max(n_items, 1)) * 4) : 0;
    const size_t o_ax = split ? c.take(M * K * 12) : 0;
    const size_t o_bx = split ? c.take(N * K * 12) : 0;
    int st = ensure_arena(e, c.off);
    if (st) return st;
    char *b = e->arena.base;
    e->d_tile_counts = e->aligned_possible ? reinterpret_cast<int32_t *>(b + o_tc) : nullptr;
    e->d_dense_origin = e->dense_possible ? reinterpret_cast<int2 *>(b + o_di) : nullptr;
    e->d_dense_origin2 = e->dense_possible ? reinterpret_cast<int2 *>(b + o_di2) : nullptr;
    e->d_covered = e->dense_possible ? reinterpret_cast<uint32_t *>(b + o_cov) : nullptr;
    e->d_cand = e->dense_possible ? reinterpret_cast<uint32_t *>(b + o_cand) : nullptr;
    e->d_anchors = e->dense_possible ? reinterpret_cast<int2 *>(b + o_anc) : nullptr;
    e->d_anchor_counts = e->dense_possible ? reinterpret_cast<int32_t *>(b + o_ancc) : nullptr;
    e->d_dense_descs = e->dense_possible ? reinterpret_cast<DenseTileDesc *>(b + o_dd) : nullptr;
    e->d_item_covered = e->dense_possible ? reinterpret_cast<int32_t *>(b + o_ic) : nullptr;
    e->d_item_ids = e->dense_possible ? reinterpret_cast<int32_t *>(b + o_ii) : nullptr;
    e->d_Ax = split ? reinterpret_cast<float *>(b + o_ax) : nullptr;
    e->d_Bx = split ? reinterpret_cast<float *>(b + o_bx) : nullptr;
    e->d_units = reinterpret_cast<int2 *>(b + o_units);
    e->d_unit_cols = e->panels > 1 ? reinterpret_cast<int32_t *>(b + o_ucols) : nullptr;
    e->d_unit_sval = e->panels > 1 ? reinterpret_cast<float *>(b + o_ucols) : nullptr;
    e->d_unit_off = reinterpret_cast<int32_t *>(b + o_uoff);
    e->d_scan_tiles = reinterpret_cast<int32_t *>(b + o_stile);
    e->d_rp = reinterpret_cast<int32_t *>(b + o_rp);
    e->d_group_ok = reinterpret_cast<uint8_t *>(b + o_gok);
    e->d_col = reinterpret_cast<int32_t *>(b + o_col);
    e->d_sval = reinterpret_cast<float *>(b + o_sv);
    e->d_pval = reinterpret_cast<float *>(b + o_pv);
    e->d_A32 = reinterpret_cast<float *>(b + o_A);
    e->d_B32 = reinterpret_cast<float *>(b + o_B);
    e->d_A16 = bf ? reinterpret_cast<__nv_bfloat16 *>(b + o_A16) : nullptr;
    e->d_B16 = bf ? reinterpret_cast<__nv_bfloat16 *>(b + o_B16) : nullptr;
    e->d_touched = reinterpret_cast<unsigned char *>(b + o_touch);
    e->d_rowstart = reinterpret_cast<uint32_t *>(b + o_rs);
    e->d_item_rows = reinterpret_cast<int2 *>(b + o_items);
    e->d_coo_rows = coo ? reinterpret_cast<int32_t *>(b + o_coo) : nullptr;
    e->d_pc = reinterpret_cast<PlanCounters *>(b + o_pc);
    e->d_err = reinterpret_cast<int32_t *>(b + o_err);
    return SDDMM_B200_OK;
}

// Work-item size: 2048 nonzeros, smaller for small matrices so that every SM gets work.
int choose_item_nnz(const sddmm_b200_engine *e) {
    if (const char *env = std::getenv("SDDMM_B200_ITEM_NNZ")) {  // tuning knob: nonzeros per work item
        const long v = std::atol(env);
        if (v >= 32 && v <= (1 << 20)) return static_cast<int>((v + 31) / 32 * 32);
    }
    const int64_t per = e->nnz / (static_cast<int64_t>(e->sm_count) * 4);
    int64_t z = (per + 31) / 32 * 32;
    z = std::max<int64_t>(256, std::min<int64_t>(2048, z));
    return static_cast<int>(z);
}

int convert_storage(sddmm_b200_engine *e) {
    const int cap = e->sm_count * 8;
    if (e->use_seg && e->seg_copies && e->n_units > 0) {   // the units' copies of S.val follow every change of S.val
        k_unit_values<<<grid_for(8 * static_cast<int64_t>(e->n_units), kBlock, cap * 4), kBlock, 0, e->stream>>>(e->d_units, e->n_units, e->d_sval,
                                                                                                           e->d_unit_sval);
        CU_TRY(e, cudaGetLastError());
    }
    if (e->d_Ax && e->n_dense > 0) {  // hi/lo-concatenated operands of the fp32-grade tensor-core mode (only when tiles were found)
        k_split_concat_tf32<<<grid_for(e->M * e->K, kBlock, cap), kBlock, 0, e->stream>>>(e->d_A32, e->d_Ax, e->M, static_cast<int32_t>(e->K), 1);
        k_split_concat_tf32<<<grid_for(e->N * e->K, kBlock, cap), kBlock, 0, e->stream>>>(e->d_B32, e->d_Bx, e->N, static_cast<int32_t>(e->K), 0);
        CU_TRY(e, cudaGetLastError());
    }
    if (e->mode != SDDMM_B200_BF16) return SDDMM_B200_OK;
    // (the fp32 copies keep the rounded values: the dense-tile kernel reads them through its tensor maps)
    k_f32_to_bf16<<<grid_for(e->M * e->K, kBlock, cap), kBlock, 0, e->stream>>>(e->d_A32, e->d_A16, e->M * e->K);
    k_f32_to_bf16<<<grid_for(e->N * e->K, kBlock, cap), kBlock, 0, e->stream>>>(e->d_B32, e->d_B16, e->N * e->K);
    CU_TRY(e, cudaGetLastError());
    return SDDMM_B200_OK;
}

// 2-D tensor map over a row-major rows x K fp32 matrix: box = 32 floats (one 128-byte
// k-block) x 64 rows, 128-byte swizzle, out-of-range rows read as zero.
int make_operand_map(sddmm_b200_engine *e, CUtensorMap *map, const float *base, int64_t rows, int64_t K) {
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CU_TRY(e, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return fail(e, SDDMM_B200_ERR_CUDA, "cuTensorMapEncodeTiled not available");
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(K) * 4};
    const cuuint32_t box[2] = {32, 64};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), gdim, gstride, box, estride,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(e, SDDMM_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    return SDDMM_B200_OK;
}

// Find the 64x64 tiles that are at least half full, build their row descriptors and the list
// of work items the row-tile kernel still has to visit.
// the plan counters as they are when the stream has drained
int read_counters(sddmm_b200_engine *e, PlanCounters *out) {
    CU_TRY(e, cudaMemcpyAsync(e->h_pc, e->d_pc, sizeof(PlanCounters), cudaMemcpyDeviceToHost, e->stream));
    CU_TRY(e, cudaStreamSynchronize(e->stream));
    *out = *e->h_pc;
    return SDDMM_B200_OK;
}

int cuda_status(sddmm_b200_engine *e, cudaError_t err);

// the instantiation of the dense-tile kernel for (own masks looked at, three-slot operand scheme)
const void *dense_function(bool own, bool split3) {
    if (split3) return own ? reinterpret_cast<const void *>(sddmm_dense_tile_kernel<true, true>) : reinterpret_cast<const void *>(sddmm_dense_tile_kernel<false, true>);
    return own ? reinterpret_cast<const void *>(sddmm_dense_tile_kernel<true, false>) : reinterpret_cast<const void *>(sddmm_dense_tile_kernel<false, false>);
}

int build_dense_plan(sddmm_b200_engine *e, const PlanCounters &base_pc, int item_nnz, int n_items) {
    e->n_dense = 0;
    e->n_residual_items = n_items;
    if (!e->dense_possible || base_pc.unsorted_cols || base_pc.dup_cols || base_pc.max_row_nnz < 32) return SDDMM_B200_OK;
    const int cap = e->sm_count * 8;
    cudaStream_t s = e->stream;
    const int32_t M = static_cast<int32_t>(e->M);
    CU_TRY(e, cudaMemsetAsync(e->d_covered, 0, (static_cast<size_t>(e->nnz) / 32 + 2) * 4, s));
    CU_TRY(e, cudaMemsetAsync(e->d_item_covered, 0, static_cast<size_t>(n_items) * 4, s));
    PlanCounters pc;
    // ---- tiles on the 64-grid: count every cell, keep those at least half full ----
    int n_aligned = 0;
    unsigned long long aligned_nnz = 0;
    if (e->aligned_possible) {
        CU_TRY(e, cudaMemsetAsync(e->d_tile_counts, 0, static_cast<size_t>(e->tile_grid) * 4, s));
        k_tile_count<<<grid_for(e->M * 32, kBlock, 1 << 30), kBlock, 0, s>>>(e->d_rp, e->d_col, M, e->tiles_per_row, e->d_tile_counts);
        k_tile_select<<<grid_for(e->tile_grid, kBlock, cap), kBlock, 0, s>>>(e->d_tile_counts, e->tile_grid, e->tiles_per_row, kDenseMinCount,
                                                                             e->d_dense_origin, e->dense_cap, e->d_pc);
        CU_TRY(e, cudaGetLastError());
        if (int rc = read_counters(e, &pc)) return rc;
        n_aligned = std::min(pc.dense_tiles, e->dense_cap);
        aligned_nnz = pc.window_nnz;
    }
    int n_dense = n_aligned;
    e->dense_origin = e->d_dense_origin;
    bool offsets_used = false;   // the tiles in use come from the arbitrary-offset detection (they may overlap)
    // ---- tiles at arbitrary offsets ("randomly placed blocks"): when the grid catches less than half of the nonzeros and
    //      the rows are long enough to hold half-full 64-column windows at all ----
    const bool try_offsets = e->knob_offset_tiles != 0 &&
                             (e->knob_offset_tiles > 0 || (2 * aligned_nnz < static_cast<unsigned long long>(e->nnz) &&
                                                           e->nnz >= 16 * static_cast<int64_t>(std::max<unsigned long long>(1, base_pc.rows_nonempty))));
    if (try_offsets) {
        const int wcap = e->sm_count * 32;
        CU_TRY(e, cudaMemsetAsync(e->d_cand, 0, (static_cast<size_t>(e->nnz) / 32 + 2) * 4, s));
        CU_TRY(e, cudaMemsetAsync(&e->d_pc->n_anchors, 0, sizeof(int), s));
        k_window_candidates<<<grid_for(e->M * 32, kBlock, wcap), kBlock, 0, s>>>(e->d_rp, e->d_col, M, 32, e->d_cand);
        k_window_anchors<<<grid_for(e->M * 32, kBlock, wcap), kBlock, 0, s>>>(e->d_rp, e->d_col, M, 32, e->d_cand, e->d_anchors, e->anchor_cap,
                                                                              &e->d_pc->n_anchors);
        CU_TRY(e, cudaGetLastError());
        if (int rc = read_counters(e, &pc)) return rc;
        const int n_anchors = std::min(pc.n_anchors, e->anchor_cap);
        if (n_anchors > 0) {
            CU_TRY(e, cudaMemsetAsync(e->d_anchor_counts, 0, static_cast<size_t>(n_anchors) * 4, s));
            CU_TRY(e, cudaMemsetAsync(&e->d_pc->dense_tiles, 0, sizeof(int), s));
            CU_TRY(e, cudaMemsetAsync(&e->d_pc->window_nnz, 0, sizeof(unsigned long long), s));
            k_anchor_counts<<<grid_for(static_cast<int64_t>(n_anchors) * 64, kBlock, 1 << 30), kBlock, 0, s>>>(e->d_rp, e->d_col, M, e->d_anchors,
                                                                                                            n_anchors, e->d_anchor_counts);
            k_anchor_select<<<grid_for(n_anchors, kBlock, 1 << 30), kBlock, 0, s>>>(e->d_anchors, e->d_anchor_counts, n_anchors, kDenseMinCount,
                                                                                    e->d_dense_origin2, e->dense_cap, e->d_pc);
            CU_TRY(e, cudaGetLastError());
            if (int rc = read_counters(e, &pc)) return rc;
            // (windows may overlap, so their sum can count a nonzero twice; it still ranks the two detections)
            if (pc.window_nnz > aligned_nnz) {
                n_dense = std::min(pc.dense_tiles, e->dense_cap);
                e->dense_origin = e->d_dense_origin2;
                offsets_used = true;
            }
        }
    }
    if (n_dense <= 0) return SDDMM_B200_OK;
    // row descriptors and ownership (tile_owned: the anchor counters are free again)
    auto describe = [&]() -> int {
        CU_TRY(e, cudaMemsetAsync(&e->d_pc->dense_nnz, 0, sizeof(unsigned long long), s));
        CU_TRY(e, cudaMemsetAsync(e->d_anchor_counts, 0, static_cast<size_t>(n_dense) * 4, s));
        // overlapping tiles: one owner key per nonzero, kept in P.val's storage (unused until the first run)
        uint32_t *owner = offsets_used ? reinterpret_cast<uint32_t *>(e->d_pval) : nullptr;
        if (owner) {
            CU_TRY(e, cudaMemsetAsync(owner, 0xFF, static_cast<size_t>(e->nnz) * 4, s));
            k_tile_propose<<<grid_for(static_cast<int64_t>(n_dense) * 64, kBlock, 1 << 30), kBlock, 0, s>>>(e->d_rp, e->d_col, M, e->dense_origin,
                                                                                                             n_dense, owner);
        }
        k_tile_rows<DenseTileDesc><<<grid_for(static_cast<int64_t>(n_dense) * 64, kBlock, 1 << 30), kBlock, 0, s>>>(
            e->d_rp, e->d_col, M, e->dense_origin, n_dense, e->d_dense_descs, e->d_covered, item_nnz, e->d_item_covered, e->d_anchor_counts,
            e->d_pc, owner);
        return cuda_status(e, cudaGetLastError());
    };
    if (int rc = describe()) return rc;
    if (offsets_used) {
        // windows at arbitrary offsets overlap: drop the tiles that own less than a quarter of a tile, then decide the
        // ownership afresh among those that stay
        int2 *kept = e->d_dense_origin;   // (the grid's list is not used)
        CU_TRY(e, cudaMemsetAsync(&e->d_pc->dense_tiles, 0, sizeof(int), s));
        k_tile_keep<<<grid_for(n_dense, kBlock, 1 << 30), kBlock, 0, s>>>(e->dense_origin, e->d_anchor_counts, n_dense, kDenseMinCount / 2, kept, e->d_pc);
        CU_TRY(e, cudaGetLastError());
        if (int rc = read_counters(e, &pc)) return rc;
        if (pc.dense_tiles < n_dense) {
            n_dense = pc.dense_tiles;
            e->dense_origin = kept;
            CU_TRY(e, cudaMemsetAsync(e->d_covered, 0, (static_cast<size_t>(e->nnz) / 32 + 2) * 4, s));
            CU_TRY(e, cudaMemsetAsync(e->d_item_covered, 0, static_cast<size_t>(n_items) * 4, s));
            if (n_dense <= 0) return SDDMM_B200_OK;
            if (int rc = describe()) return rc;
        }
    }
    k_residual_items<<<grid_for(n_items, kBlock, 1 << 30), kBlock, 0, s>>>(e->d_item_covered, n_items, item_nnz, e->nnz, e->d_item_ids,
                                                                          e->d_pc);
    CU_TRY(e, cudaGetLastError());
    if (int rc = read_counters(e, &pc)) return rc;
    const bool split = e->mode == SDDMM_B200_FP32_TC;
    const int64_t kx = split ? 3 * e->K : e->K;
    int st = make_operand_map(e, &e->map_a, split ? e->d_Ax : e->d_A32, e->M, kx);
    if (!st) st = make_operand_map(e, &e->map_b, split ? e->d_Bx : e->d_B32, e->N, kx);
    if (st) return st;
    const bool own_masks = offsets_used;   // tiles off the grid may overlap
    e->dense_own = own_masks;
    // fp32-grade mode, K >= 64: the three-slot operand scheme (measured on the 64 x 64-block configuration, K = 64 / 128:
    // 74 / 114 us against 93 / 160 us with one A block + one B block; K = 32: 63-66 us either way, the shared-memory data
    // pipe that the epilogue and the operand reads share is the limit there).  Knob "dense_split3": 0 = never, 1 = always.
    e->dense_split3 = split && (e->knob_dense_split3 > 0 || (e->knob_dense_split3 < 0 && e->K >= 64));
    const void *dense_fn = dense_function(e->dense_own, e->dense_split3);
    const uint32_t dense_smem = e->dense_split3 ? DenseSmemT<true>::kDynamicBytes : DenseSmemT<false>::kDynamicBytes;
    if (ensure_dynamic_smem_limit(dense_fn, e->device, dense_smem))
        return fail(e, SDDMM_B200_ERR_CUDA, "dense-tile kernel: cannot raise the dynamic shared memory limit");
    CU_TRY(e, cudaFuncSetAttribute(dense_fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    e->n_dense = n_dense;
    e->n_residual_items = pc.residual_items;
    sddmm_b200_plan_info &p = e->plan;
    p.dense_tiles = n_dense;
    p.dense_nnz = static_cast<int64_t>(pc.dense_nnz);
    p.dense_tile_rows = p.dense_tile_cols = kDenseTile;
    p.dense_block = kDenseThreads;
    p.dense_smem_bytes = static_cast<int32_t>(dense_smem);
    // Resident CTAs per SM, from the kernel's own resources (the runtime's occupancy query answers 1 for this kernel):
    // shared memory (+1 KB the driver reserves per CTA), registers (allocated per warp in units of 256), tensor memory columns.
    cudaFuncAttributes fa;
    CU_TRY(e, cudaFuncGetAttributes(&fa, dense_fn));
    int smem_per_sm = 0, regs_per_sm = 0;   // (single attributes: the full property query takes milliseconds)
    CU_TRY(e, cudaDeviceGetAttribute(&smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, e->device));
    CU_TRY(e, cudaDeviceGetAttribute(&regs_per_sm, cudaDevAttrMaxRegistersPerMultiprocessor, e->device));
    const int by_smem = static_cast<int>(static_cast<size_t>(smem_per_sm) / (dense_smem + fa.sharedSizeBytes + 1024));
    const int regs_per_warp = ((fa.numRegs * 32 + 255) / 256) * 256;
    const int by_regs = regs_per_sm / (regs_per_warp * (kDenseThreads / 32));
    const int by_tmem = 512 / static_cast<int>(e->dense_split3 ? DenseSmemT<true>::kTmemColumns : DenseSmemT<false>::kTmemColumns);
    int dense_ctas_per_sm = std::min(std::min(by_smem, by_regs), std::min(by_tmem, kDenseCtasPerSm));
    if (dense_ctas_per_sm < 1) return fail(e, SDDMM_B200_ERR_CUDA, "dense-tile kernel does not fit on an SM");
    if (const char *env = getenv("SDDMM_B200_DENSE_CTAS_PER_SM")) {   // tuning knob: fewer resident CTAs per SM
        const int v = atoi(env);
        if (v >= 1 && v < dense_ctas_per_sm) dense_ctas_per_sm = v;
    }
    p.dense_grid = std::min((n_dense + 1) / 2, e->sm_count * dense_ctas_per_sm);
    return SDDMM_B200_OK;
}

// Validation + histogram + plan, after the operands are in the arena.
using RowGroupFn = void (*)(const RowGroupArgs);
RowGroupFn pick_rowgroup(int rows, int cpl) {
    if (cpl == 1) return rows == 2 ? sddmm_rowgroup_kernel<2, 1> : rows == 3 ? sddmm_rowgroup_kernel<3, 1> : sddmm_rowgroup_kernel<4, 1>;
    return rows == 2 ? sddmm_rowgroup_kernel<2, 2> : rows == 3 ? sddmm_rowgroup_kernel<3, 2> : sddmm_rowgroup_kernel<4, 2>;
}

using RowSegGroupFn = void (*)(const RowSegGroupArgs);
RowSegGroupFn pick_rowseg_group(int rows, int cpl) {
    if (cpl == 1) return rows == 2 ? sddmm_rowseg_group_kernel<1, 2> : rows == 3 ? sddmm_rowseg_group_kernel<1, 3> : sddmm_rowseg_group_kernel<1, 4>;
    return rows == 2 ? sddmm_rowseg_group_kernel<2, 2> : rows == 3 ? sddmm_rowseg_group_kernel<2, 3> : sddmm_rowseg_group_kernel<2, 4>;
}

// Row groups: groups of 2, 3 or 4 consecutive rows with one column list (first full group at row 0 .. G-1) share each gather of B.
// The path is taken (for the whole matrix) when it removes at least 30 % of the gathers; fp32 storage, K = 32 or 64.
int build_rowgroup_plan(sddmm_b200_engine *e, const PlanCounters &base_pc) {
    const bool eligible = e->mode != SDDMM_B200_BF16 && !(e->flags & SDDMM_B200_FLAG_NO_ROW_GROUPS) && (e->K == 32 || e->K == 64) &&
                          e->M >= 4 && base_pc.max_row_nnz <= 8192;
    if (!eligible) return SDDMM_B200_OK;
    cudaStream_t s = e->stream;
    const int cap = e->sm_count * 8;
    // candidates: G = 2, 3, 4 rows per group, first full group starting at row 0 .. G-1 (9 counting passes, counters slot = G(G-1)/2 - 1 + first)
    auto slot = [](int G, int first) { return G * (G - 1) / 2 - 1 + first; };
    auto groups_of = [&](int G, int first) { return static_cast<int32_t>(1 + (e->M - first + G - 1) / G); };
    const int every = e->M > 65536 ? 16 : 1;   // large inputs: choose G and `first` on a 1-in-16 sample of the groups
    for (int G = 2; G <= 4; ++G)
        for (int first = 0; first < G; ++first)
            k_group_match<<<grid_for(static_cast<int64_t>(groups_of(G, first) / every + 1) * 32, kBlock, cap), kBlock, 0, s>>>(
                e->d_rp, e->d_col, static_cast<int32_t>(e->M), G, first, groups_of(G, first), every, nullptr,
                &e->d_pc->group_cover[slot(G, first)], &e->d_pc->group_count[slot(G, first)]);
    CU_TRY(e, cudaGetLastError());
    PlanCounters pc;
    if (int rc = read_counters(e, &pc)) return rc;
    int best = 0, best_first = 0;
    double best_saved = 0.0;
    for (int G = 2; G <= 4; ++G)
        for (int first = 0; first < G; ++first) {
            const double saved = static_cast<double>(pc.group_cover[slot(G, first)]) * every * (1.0 - 1.0 / G);   // gathers of B that disappear (estimate)
            if (saved > best_saved) { best_saved = saved; best = G; best_first = first; }
        }
    if (best == 0 || best_saved < 0.3 * static_cast<double>(e->nnz)) return SDDMM_B200_OK;
    const int32_t n_groups = groups_of(best, best_first);
    const int bs = slot(best, best_first);
    CU_TRY(e, cudaMemsetAsync(&e->d_pc->group_cover[bs], 0, sizeof(unsigned long long), s));
    CU_TRY(e, cudaMemsetAsync(&e->d_pc->group_count[bs], 0, sizeof(int), s));
    k_group_match<<<grid_for(static_cast<int64_t>(n_groups) * 32, kBlock, cap), kBlock, 0, s>>>(
        e->d_rp, e->d_col, static_cast<int32_t>(e->M), best, best_first, n_groups, 1, e->d_group_ok, &e->d_pc->group_cover[bs],
        &e->d_pc->group_count[bs]);
    CU_TRY(e, cudaGetLastError());
    if (int rc = read_counters(e, &pc)) return rc;   // exact counts of the chosen grouping
    if (static_cast<double>(pc.group_cover[bs]) * (1.0 - 1.0 / best) < 0.3 * static_cast<double>(e->nnz)) return SDDMM_B200_OK;   // the sample overestimated
    RowGroupFn fn = pick_rowgroup(best, static_cast<int>(e->K / 32));
    int occ = 0;
    CU_TRY(e, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, kRowGroupWarps * 32, 0));
    if (occ < 1) return fail(e, SDDMM_B200_ERR_CUDA, "row-group kernel does not fit on an SM");
    e->rg_rows = best;
    e->rg_first = best_first;
    e->rg_groups = n_groups;
    sddmm_b200_plan_info &p = e->plan;
    p.rowgroup_nnz = static_cast<int64_t>(pc.group_cover[bs]);
    p.rowgroup_groups = pc.group_count[bs];
    p.rowgroup_rows = best;
    p.rowgroup_grid = std::min((n_groups + kRowGroupWarps - 1) / kRowGroupWarps, e->sm_count * occ);
    // Shared segments: the group's column list cut into units of 8 columns that serve all G rows (row-segment group kernel).
    e->rg_units = e->knob_group_units != 0 && e->M < kUnitRowLimit;
    if (e->rg_units) {
        const int32_t M = static_cast<int32_t>(e->M);
        const int n_tiles = static_cast<int>((e->M + kScanTile - 1) / kScanTile);
        const int capb = e->sm_count * 32;
        k_group_unit_count<<<grid_for(e->M, kBlock, capb), kBlock, 0, s>>>(e->d_rp, M, best, best_first, e->d_group_ok, e->d_unit_off);
        k_scan_tile_sums<<<n_tiles, kScanBlock, 0, s>>>(e->d_unit_off, e->M, e->d_scan_tiles);
        k_scan_sums<<<1, kScanBlock, 0, s>>>(e->d_scan_tiles, n_tiles, &e->d_pc->units);
        k_scan_apply<<<n_tiles, kScanBlock, 0, s>>>(e->d_unit_off, e->M, e->d_scan_tiles);
        k_group_unit_fill<<<grid_for(e->M * 32, kBlock, capb), kBlock, 0, s>>>(e->d_rp, M, best, best_first, e->d_group_ok, e->d_unit_off,
                                                                               reinterpret_cast<int4 *>(e->d_units));
        CU_TRY(e, cudaGetLastError());
        if (int rc = read_counters(e, &pc)) return rc;
        if (pc.units == 0 || pc.units > static_cast<unsigned long long>(e->unit_cap))
            return fail(e, SDDMM_B200_ERR_CUDA, "row-group plan: %llu units for a list of %lld", pc.units, (long long)e->unit_cap);
        e->n_units = static_cast<int32_t>(pc.units);
        int occ2 = 0;
        CU_TRY(e, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ2, pick_rowseg_group(best, static_cast<int>(e->K / 32)), kRowSegWarps * 32, 0));
        if (occ2 < 1) return fail(e, SDDMM_B200_ERR_CUDA, "row-segment group kernel does not fit on an SM");
        const int64_t n_quads = (static_cast<int64_t>(e->n_units) + 3) / 4;
        p.rowseg_units = e->n_units;
        p.rowseg_panels = 1;
        p.rowgroup_grid = static_cast<int32_t>(std::min<int64_t>((n_quads + kRowSegWarps - 1) / kRowSegWarps, static_cast<int64_t>(e->sm_count) * occ2));
    }
    p.rowtile_nnz = 0;
    p.rowtile_items = 0;
    p.n_kernels = 1;
    return SDDMM_B200_OK;
}

template <typename ET>
using RowSegFn = void (*)(const RowSegArgs);

template <typename ET, bool HINT>
RowSegFn<ET> pick_rowseg_hint(int cpl, bool exact) {
    switch (cpl) {
        case 1: return exact ? sddmm_rowseg_kernel<1, true, ET, HINT> : sddmm_rowseg_kernel<1, false, ET, HINT>;
        case 2: return exact ? sddmm_rowseg_kernel<2, true, ET, HINT> : sddmm_rowseg_kernel<2, false, ET, HINT>;
        case 4: return exact ? sddmm_rowseg_kernel<4, true, ET, HINT> : sddmm_rowseg_kernel<4, false, ET, HINT>;
        case 8: return exact ? sddmm_rowseg_kernel<8, true, ET, HINT> : sddmm_rowseg_kernel<8, false, ET, HINT>;
        default: return nullptr;
    }
}
template <typename ET>
RowSegFn<ET> pick_rowseg(int cpl, bool exact, bool hint = false) {
    return hint ? pick_rowseg_hint<ET, true>(cpl, exact) : pick_rowseg_hint<ET, false>(cpl, exact);
}

// The row-segment kernel instantiation for this engine's storage and K.  bf16 storage with K >= 64 reads 16-byte chunks
// (8 elements: 8 lanes cover a 128-byte piece in one request), otherwise chunks of 4 elements.
bool seg_wide_bf16(const sddmm_b200_engine *e) { return e->mode == SDDMM_B200_BF16 && e->K >= 64; }
const void *seg_function(const sddmm_b200_engine *e, bool hint) {
    if (seg_wide_bf16(e)) {
        const int cpl = round_up_cpl((e->K + 1) / 2);   // chunks of 8: K / 64 lanes-rounds
        return reinterpret_cast<const void *>(pick_rowseg<Bf16x8>(cpl, e->K == 64 * cpl, hint));
    }
    if (e->seg_slices > 1)   // a 64-column slice of fp32 rows
        return hint ? reinterpret_cast<const void *>(sddmm_rowseg_kernel<2, true, float, true, true>)
                    : reinterpret_cast<const void *>(sddmm_rowseg_kernel<2, true, float, false, true>);
    const bool exact = e->K == 32 * e->cpl;
    return e->mode == SDDMM_B200_BF16 ? reinterpret_cast<const void *>(pick_rowseg<__nv_bfloat16>(e->cpl, exact, hint))
                                      : reinterpret_cast<const void *>(pick_rowseg<float>(e->cpl, exact, hint));
}

// What the dense tiles left, as row segments: the uncovered runs of every row cut into units, so that the residual
// kernel touches only those nonzeros (a kernel that walks all work items and skips the covered nonzeros costs as much as
// the whole matrix when the tiles leave a little in every item).
int build_residual_units(sddmm_b200_engine *e) {
    if ((e->flags & SDDMM_B200_FLAG_NO_ROW_SEGMENTS) || e->knob_rowseg == 0 || e->M >= kUnitRowLimit) return SDDMM_B200_OK;
    const int32_t M = static_cast<int32_t>(e->M);
    const int n_tiles = static_cast<int>((e->M + kScanTile - 1) / kScanTile);
    const int cap = e->sm_count * 32;
    cudaStream_t s = e->stream;
    k_residual_unit_count<<<grid_for(e->M, kBlock, cap), kBlock, 0, s>>>(e->d_rp, M, e->d_covered, e->d_unit_off);
    k_scan_tile_sums<<<n_tiles, kScanBlock, 0, s>>>(e->d_unit_off, e->M, e->d_scan_tiles);
    k_scan_sums<<<1, kScanBlock, 0, s>>>(e->d_scan_tiles, n_tiles, &e->d_pc->units);
    k_scan_apply<<<n_tiles, kScanBlock, 0, s>>>(e->d_unit_off, e->M, e->d_scan_tiles);
    CU_TRY(e, cudaGetLastError());
    PlanCounters pc;
    if (int rc = read_counters(e, &pc)) return rc;
    if (pc.units == 0 || pc.units > static_cast<unsigned long long>(e->unit_cap)) return SDDMM_B200_OK;   // (the row-tile kernel takes the residual)
    k_residual_unit_fill<<<grid_for(e->M, kBlock, cap), kBlock, 0, s>>>(e->d_rp, M, e->d_covered, e->d_unit_off, e->d_units);
    CU_TRY(e, cudaGetLastError());
    int occ = 0;
    CU_TRY(e, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, seg_function(e, false), kRowSegWarps * 32, 0));
    if (occ < 1) return SDDMM_B200_OK;
    e->n_units = static_cast<int32_t>(pc.units);
    e->seg_residual = true;
    const int64_t n_quads = (static_cast<int64_t>(e->n_units) + 3) / 4;
    e->plan.rowseg_units = e->n_units;
    e->plan.rowseg_panels = 1;
    e->plan.rowseg_passes = e->seg_slices;
    e->plan.rowseg_grid = static_cast<int32_t>(std::min<int64_t>((n_quads + kRowSegWarps - 1) / kRowSegWarps, static_cast<int64_t>(e->sm_count) * occ));
    return SDDMM_B200_OK;
}

// Row segments: the unit list (rows cut into segments of at most 8 nonzeros, panel-major when B is cut into column
// panels) is counted, scanned and written on the device; the host only reads the total.  Taken unless the rows are
// long on average (the A-row-tile kernel keeps the A chunk of a long row in registers over the whole row).
int build_rowseg_plan(sddmm_b200_engine *e, const PlanCounters &base_pc) {
    const int seg_env = e->knob_rowseg < 0 ? -1 : static_cast<int>(e->knob_rowseg);   // 0 never, 1 whenever possible
    e->use_seg = false;
    e->seg_copies = false;
    e->n_units = 0;
    if ((e->flags & SDDMM_B200_FLAG_NO_ROW_SEGMENTS) || seg_env == 0 || e->M >= kUnitRowLimit) return SDDMM_B200_OK;
    int32_t panels = base_pc.unsorted_cols ? 1 : e->panels;   // a panel run is a contiguous piece of a row only when its columns are sorted
    if (panels == 1) e->long_rows = 0;
    if (e->long_rows > 0 && e->knob_long_rows < 0) {
        // panels for the long rows only pay when those rows hold a good share of the nonzeros
        unsigned long long in_long = 0;
        for (int b = 0; b < SDDMM_B200_HIST_BINS; ++b)
            if (b >= 1 && (1ll << (b - 1)) >= e->long_rows) in_long += base_pc.hist_nnz[b];
        if (5 * in_long < 2 * static_cast<unsigned long long>(e->nnz)) {   // < 40 %: every row whole, one pass
            e->long_rows = 0;
            panels = 1;
            if (e->knob_k_slices < 0) e->seg_slices = 1;
        }
    }
    const int32_t M = static_cast<int32_t>(e->M);
    const int64_t n = static_cast<int64_t>(panels) * M;
    const int n_tiles = static_cast<int>((n + kScanTile - 1) / kScanTile);
    const int cap = e->sm_count * 32;
    cudaStream_t s = e->stream;
    k_unit_count<<<grid_for(n, kBlock, cap), kBlock, 0, s>>>(e->d_rp, e->d_col, M, panels, e->panel_cols, e->long_rows, e->d_unit_off);
    k_scan_tile_sums<<<n_tiles, kScanBlock, 0, s>>>(e->d_unit_off, n, e->d_scan_tiles);
    k_scan_sums<<<1, kScanBlock, 0, s>>>(e->d_scan_tiles, n_tiles, &e->d_pc->units);
    k_scan_apply<<<n_tiles, kScanBlock, 0, s>>>(e->d_unit_off, n, e->d_scan_tiles);
    e->seg_copies = panels > 1 && e->d_unit_cols != nullptr;
    k_unit_fill<<<grid_for(n * 32, kBlock, cap), kBlock, 0, s>>>(e->d_rp, e->d_col, M, panels, e->panel_cols, e->long_rows, e->d_unit_off, e->d_units,
                                                                  e->seg_copies ? e->d_unit_cols : nullptr);
    CU_TRY(e, cudaGetLastError());
    PlanCounters pc;
    if (int rc = read_counters(e, &pc)) return rc;
    if (pc.units == 0 || pc.units > static_cast<unsigned long long>(e->unit_cap) || pc.units >= (1ull << 31))
        return fail(e, SDDMM_B200_ERR_CUDA, "row-segment plan: %llu units for a list of %lld", pc.units, (long long)e->unit_cap);
    const void *fn = seg_function(e, false);
    int occ = 0;
    CU_TRY(e, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, kRowSegWarps * 32, 0));
    if (occ < 1) return fail(e, SDDMM_B200_ERR_CUDA, "row-segment kernel does not fit on an SM");
    e->n_units = static_cast<int32_t>(pc.units);
    e->use_seg = true;
    sddmm_b200_plan_info &p = e->plan;
    const int64_t n_quads = (static_cast<int64_t>(e->n_units) + 3) / 4;
    p.rowseg_nnz = e->nnz;
    p.rowseg_units = e->n_units;
    p.rowseg_panels = panels;
    p.rowseg_passes = e->seg_slices;
    p.rowseg_grid = static_cast<int32_t>(std::min<int64_t>((n_quads + kRowSegWarps - 1) / kRowSegWarps, static_cast<int64_t>(e->sm_count) * occ));
    p.rowtile_nnz = 0;
    p.rowtile_items = 0;
    p.n_kernels = 1;
    return SDDMM_B200_OK;
}

int build_plan(sddmm_b200_engine *e, int item_nnz, int n_items) {
    const int cap = e->sm_count * 8;
    cudaStream_t s = e->stream;
    CU_TRY(e, cudaMemsetAsync(e->d_pc, 0, sizeof(PlanCounters), s));
    CU_TRY(e, cudaMemsetAsync(e->d_err, 0, sizeof(int32_t), s));
    CU_TRY(e, cudaMemsetAsync(e->d_touched, 0, static_cast<size_t>(e->N), s));
    CU_TRY(e, cudaMemsetAsync(e->d_rowstart, 0, (static_cast<size_t>(e->nnz) / 32 + 2) * 4, s));
    if (e->d_coo_rows) {
        k_coo_to_row_ptr<<<grid_for(e->nnz + 1, kBlock, cap), kBlock, 0, s>>>(e->d_coo_rows, e->nnz, static_cast<int32_t>(e->M),
                                                                              e->coo_row_base, e->d_rp, e->d_pc);
        // refuse to interpret a row_ptr built from unsorted rows
        PlanCounters pc0;
        if (int rc = read_counters(e, &pc0)) return rc;
        if (pc0.bad_coo) return fail(e, SDDMM_B200_ERR_INDEX, "COO row indices must be sorted and inside [0, M)");
    }
    k_row_stats<<<grid_for(e->M, kBlock, 1 << 30), kBlock, 0, s>>>(e->d_rp, static_cast<int32_t>(e->M), e->nnz, e->d_rowstart, e->d_pc);
    CU_TRY(e, cudaGetLastError());
    PlanCounters pc;
    if (int rc = read_counters(e, &pc)) return rc;
    if (pc.bad_row_ptr) return fail(e, SDDMM_B200_ERR_INDEX, "row_ptr must start at 0, end at nnz and be non-decreasing");
    if (e->nnz > 0) {
        k_col_scan<<<grid_for(e->nnz, kBlock, cap), kBlock, 0, s>>>(e->d_col, e->nnz, static_cast<int32_t>(e->N), e->d_rowstart,
                                                                    e->d_touched, e->d_pc);
        k_count_bytes<<<grid_for(e->N, kBlock, cap), kBlock, 0, s>>>(e->d_touched, e->N, &e->d_pc->cols_touched);
        k_item_rows<<<grid_for(n_items, kBlock, 1 << 30), kBlock, 0, s>>>(e->d_rp, static_cast<int32_t>(e->M), e->nnz, item_nnz, n_items,
                                                                          e->d_item_rows);
        CU_TRY(e, cudaGetLastError());
    }
    if (int rc = read_counters(e, &pc)) return rc;
    if (pc.bad_col) return fail(e, SDDMM_B200_ERR_INDEX, "column index outside [0, N)");

    sddmm_b200_plan_info &p = e->plan;
    std::memset(&p, 0, sizeof(p));
    p.rows = e->M; p.cols = e->N; p.k = e->K; p.nnz = e->nnz;
    p.rows_nonempty = static_cast<int64_t>(pc.rows_nonempty);
    p.cols_touched = static_cast<int64_t>(pc.cols_touched);
    p.max_row_nnz = pc.max_row_nnz;
    for (int b = 0; b < SDDMM_B200_HIST_BINS; ++b) p.row_len_hist[b] = static_cast<int64_t>(pc.hist[b]);
    p.cols_sorted = pc.unsorted_cols ? 0 : 1;
    p.mode = e->mode;
    p.n_devices = 1;

    // ---- row-tile kernel launch shape -----------------------------------------
    const size_t eb = elem_bytes(e);
    e->cpl = round_up_cpl(e->K);
    e->use_scalar = (e->K % 4 != 0) || e->cpl == 0 || static_cast<size_t>(e->K) * eb > kMaxStageBytes;
    if (e->mode == SDDMM_B200_BF16 && (e->use_scalar || e->K % 8 != 0))
        return fail(e, SDDMM_B200_ERR_UNSUPPORTED, "bf16 storage needs K %% 8 == 0 and K <= 256 (K = %lld)", (long long)e->K);
    p.rowtile_item_nnz = item_nnz;
    p.rowtile_block = kBlock;
    e->n_dense = 0;
    e->n_residual_items = n_items;
    if (e->nnz == 0) {
        p.n_kernels = 0;
        return SDDMM_B200_OK;
    }
    e->seg_residual = false;
    if (!e->use_scalar) {
        int st = build_dense_plan(e, pc, item_nnz, n_items);
        if (st) return st;
        if (e->n_dense > 0 && e->n_residual_items > 0) {
            st = build_residual_units(e);
            if (st) return st;
        }
    }
    e->rg_rows = 0;
    e->use_seg = false;
    if (!e->use_scalar && e->n_dense == 0) {
        int st = build_rowgroup_plan(e, pc);
        if (st) return st;
        if (e->rg_rows) return SDDMM_B200_OK;
        st = build_rowseg_plan(e, pc);
        if (st) return st;
        if (e->use_seg) return SDDMM_B200_OK;
    }
    p.rowtile_nnz = e->nnz - p.dense_nnz;
    p.rowtile_items = e->n_residual_items;
    const int dense_kernels = e->n_dense > 0 ? 1 : 0;
    if (e->n_residual_items == 0) {
        p.n_kernels = dense_kernels;
        return SDDMM_B200_OK;
    }
    if (e->seg_residual) {   // the row-segment kernel computes what the tiles left
        p.rowseg_nnz = p.rowtile_nnz;
        p.rowtile_nnz = 0;
        p.rowtile_items = 0;
        p.n_kernels = 1 + dense_kernels;
        return SDDMM_B200_OK;
    }
    if (e->use_scalar) {
        p.rowtile_rows_per_stage = 0;
        p.rowtile_smem_bytes = 0;
        p.rowtile_grid = grid_for(e->nnz, kBlock, e->sm_count * 8);
        p.n_kernels = 1;
        return SDDMM_B200_OK;
    }
    const double mean_len = static_cast<double>(e->nnz) / static_cast<double>(std::max<int64_t>(1, p.rows_nonempty));
    int64_t R = static_cast<int64_t>(item_nnz / std::max(1.0, mean_len)) + 1;
    R = (R + 7) / 8 * 8;
    const int64_t r_max = std::max<int64_t>(1, static_cast<int64_t>(kMaxStageBytes / (static_cast<size_t>(e->K) * eb)));
    R = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(R, r_max), e->M));
    p.rowtile_rows_per_stage = static_cast<int32_t>(R);
    p.rowtile_smem_bytes = static_cast<int32_t>(rowtile_smem_bytes(static_cast<int>(R), static_cast<uint32_t>(e->K * eb)));

    const void *fn = (e->mode == SDDMM_B200_BF16) ? reinterpret_cast<const void *>(pick_rowtile<__nv_bfloat16>(e->cpl, e->K == 32 * e->cpl))
                                                  : reinterpret_cast<const void *>(pick_rowtile<float>(e->cpl, e->K == 32 * e->cpl));
    if (ensure_dynamic_smem_limit(fn, e->device, kRowTileMaxSmem)) return fail(e, SDDMM_B200_ERR_CUDA, "row-tile kernel: cannot raise the dynamic shared memory limit");
    int occ = 0;
    CU_TRY(e, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, kBlock, p.rowtile_smem_bytes));
    if (occ < 1) return fail(e, SDDMM_B200_ERR_CUDA, "row-tile kernel does not fit on an SM (smem %d B)", p.rowtile_smem_bytes);
    p.rowtile_grid = std::min(e->n_residual_items, e->sm_count * occ);
    p.n_kernels = 1 + dense_kernels;
    return SDDMM_B200_OK;
}

int check_dims(sddmm_b200_engine *e, int64_t M, int64_t N, int64_t K, int64_t nnz) {
    if (M < 1 || N < 1 || K < 1 || nnz < 0) return fail(e, SDDMM_B200_ERR_ARG, "need M, N, K >= 1 and nnz >= 0");
    if (M >= (int64_t(1) << 31) - 1 || N >= (int64_t(1) << 31) - 1 || nnz >= (int64_t(1) << 31) - 8192)
        return fail(e, SDDMM_B200_ERR_ARG, "int32 index range exceeded");
    return SDDMM_B200_OK;
}

int cuda_status(sddmm_b200_engine *e, cudaError_t err) {
    CU_TRY(e, err);
    return SDDMM_B200_OK;
}

// all copies of an upload: pattern on the main stream, then values and dense operands on the side stream; ev_h2d after the last
int enqueue_copies(sddmm_b200_engine *e, const int32_t *row_ptr, const int32_t *coo_rows, const int32_t *col_idx, const float *s_val,
                   const float *A, const float *B, cudaMemcpyKind kind) {
    cudaStream_t s = e->stream, s2 = e->side_stream;
    const int64_t M = e->M, N = e->N, K = e->K, nnz = e->nnz;
    // (host sources: pageable memory is staged through pinned buffers by a pool of host threads, see host_staging.cuh)
    auto copy_in = [&](void *dst, const void *src, size_t bytes, cudaStream_t st, HostStager &stg) -> cudaError_t {
        return kind == cudaMemcpyHostToDevice ? stg.upload(dst, src, bytes, st) : cudaMemcpyAsync(dst, src, bytes, kind, st);
    };
    if (row_ptr) CU_TRY(e, copy_in(e->d_rp, row_ptr, static_cast<size_t>(M + 1) * 4, s, e->stager));
    if (coo_rows && nnz) CU_TRY(e, copy_in(e->d_coo_rows, coo_rows, static_cast<size_t>(nnz) * 4, s, e->stager));
    if (nnz) CU_TRY(e, copy_in(e->d_col, col_idx, static_cast<size_t>(nnz) * 4, s, e->stager));
    CU_TRY(e, cudaEventRecord(e->ev_join, s));
    CU_TRY(e, cudaStreamWaitEvent(s2, e->ev_join, 0));   // keeps the link order: pattern first
    if (nnz) CU_TRY(e, copy_in(e->d_sval, s_val, static_cast<size_t>(nnz) * 4, s2, e->stager2));
    CU_TRY(e, copy_in(e->d_A32, A, static_cast<size_t>(M * K) * 4, s2, e->stager2));
    if (e->B_on_device) CU_TRY(e, cudaMemcpyAsync(e->d_B32, e->B_on_device, static_cast<size_t>(N * K) * 4, cudaMemcpyDeviceToDevice, s2));
    else CU_TRY(e, copy_in(e->d_B32, B, static_cast<size_t>(N * K) * 4, s2, e->stager2));
    CU_TRY(e, cudaEventRecord(e->ev_h2d, s2));
    if (e->on_copies_enqueued) e->on_copies_enqueued(e->on_copies_user);
    return SDDMM_B200_OK;
}

int upload_common(sddmm_b200_engine *e, int64_t M, int64_t N, int64_t K, int64_t nnz, const int32_t *row_ptr,
                  const int32_t *coo_rows, const int32_t *col_idx, const float *s_val, const float *A, const float *B,
                  cudaMemcpyKind kind) {
    e->uploaded = false;
    e->ran = false;
    e->spmm_units = 0;
    e->M = M; e->N = N; e->K = K; e->nnz = nnz;
    const int item_nnz = choose_item_nnz(e);
    const int n_items = static_cast<int>((nnz + item_nnz - 1) / item_nnz);
    int st = carve_arena(e, coo_rows != nullptr, n_items);
    if (st) return st;
    // The pattern goes first on the main stream and is planned there while S.val, A and B -- which the plan does not
    // read -- still cross the host link on the side stream.
    cudaStream_t s = e->stream, s2 = e->side_stream;
    if (e->h2d_after) CU_TRY(e, cudaStreamWaitEvent(s, e->h2d_after, 0));
    st = enqueue_copies(e, row_ptr, coo_rows, col_idx, s_val, A, B, kind);
    if (!st) st = build_plan(e, item_nnz, n_items);
    if (!st) st = cuda_status(e, cudaStreamWaitEvent(s, e->ev_h2d, 0));
    if (!st) st = convert_storage(e);
    if (!st) st = cuda_status(e, cudaStreamSynchronize(s));   // the caller's buffers are free again when this returns
    if (st) {   // nothing of a failed upload may still be reading the caller's buffers
        cudaStreamSynchronize(s2);
        cudaStreamSynchronize(s);
        if (e->B_on_device == e->b_stage) e->B_on_device = nullptr;
        return st;
    }
    if (e->B_on_device == e->b_stage) e->B_on_device = nullptr;
    e->uploaded = true;
    return SDDMM_B200_OK;
}

// events right before / right after kernel number `kernels_launched`, on the stream it is launched on
int begin_kernel(sddmm_b200_engine *e, cudaStream_t st) {
    if (!e->kernel_timing) return SDDMM_B200_OK;   // a timing event between two launches costs microseconds: only on request
    CU_TRY(e, cudaEventRecord(e->ev_begin[e->kernels_launched], st));
    return SDDMM_B200_OK;
}
int mark_kernel(sddmm_b200_engine *e, const char *name, cudaStream_t st) {
    CU_TRY(e, cudaGetLastError());
    const int idx = e->kernels_launched;
    e->kernel_name[idx] = name;
    if (e->kernel_timing) CU_TRY(e, cudaEventRecord(e->ev_end[idx], st));
    e->kernels_launched = idx + 1;
    return SDDMM_B200_OK;
}

// the row-segment kernel over the engine's unit list (the whole matrix, or what the dense tiles left)
int launch_rowseg(sddmm_b200_engine *e, cudaStream_t stream) {
    const sddmm_b200_plan_info &p = e->plan;
    RowSegArgs g;
    g.units = e->d_units; g.col_idx = e->d_col; g.s_val = e->d_sval; g.p_val = e->d_pval;
    g.n_units = e->n_units; g.K = static_cast<int32_t>(e->K);
    // L2 is asked to keep the gathered B rows when they can stay: one column panel at a time
    g.b_evict_last = p.rowseg_panels > 1 ? 1 : 0;
    g.b_fraction = e->knob_b_fraction > 0 ? static_cast<float>(std::min(1.0, e->knob_b_fraction)) : 1.0f;
    g.unit_cols = e->d_unit_cols; g.unit_sval = e->d_unit_sval;
    if (!e->seg_copies) g.b_evict_last = 0;   // (the hinted instantiation reads the per-unit copies)
    g.row_stride = 0;
    g.accumulate = 0;
    if (int st = begin_kernel(e, stream)) return st;
    if (e->mode == SDDMM_B200_BF16) {
        g.A = e->d_A16; g.B = e->d_B16;
    } else {
        g.A = e->d_A32; g.B = e->d_B32;
    }
    const auto fn = reinterpret_cast<RowSegFn<float>>(const_cast<void *>(seg_function(e, g.b_evict_last != 0)));
    if (e->seg_slices > 1) {   // one launch per 64-column slice of K, in stream order: each adds to what the earlier ones wrote
        g.K = 64;
        g.row_stride = static_cast<uint32_t>(e->K * 4);
        for (int sl = 0; sl < e->seg_slices; ++sl) {
            g.A = e->d_A32 + 64 * sl;
            g.B = e->d_B32 + 64 * sl;
            g.accumulate = sl > 0 ? 1 : 0;
            fn<<<p.rowseg_grid, kRowSegWarps * 32, 0, stream>>>(g);
        }
    } else {
        fn<<<p.rowseg_grid, kRowSegWarps * 32, 0, stream>>>(g);
    }
    return mark_kernel(e, "sddmm_rowseg_kernel", stream);   // (the slices of one step count as one kernel in the timing table)
}

int launch_all(sddmm_b200_engine *e) {
    const sddmm_b200_plan_info &p = e->plan;
    e->kernels_launched = 0;
    if (e->nnz == 0) return SDDMM_B200_OK;
    int st = SDDMM_B200_OK;
    if (e->use_scalar) {
        if ((st = begin_kernel(e, e->stream))) return st;
        sddmm_scalar_kernel<<<p.rowtile_grid, kBlock, 0, e->stream>>>(e->d_rp, e->d_col, e->d_sval, e->d_pval, e->d_A32, e->d_B32,
                                                                      static_cast<int32_t>(e->M), static_cast<int32_t>(e->K), e->nnz);
        return mark_kernel(e, "sddmm_scalar_kernel", e->stream);
    }
    if (e->rg_rows && e->rg_units) {
        RowSegGroupArgs g;
        g.ghdr = reinterpret_cast<const int4 *>(e->d_units); g.col_idx = e->d_col; g.s_val = e->d_sval; g.p_val = e->d_pval;
        g.A = e->d_A32; g.B = e->d_B32; g.n_units = e->n_units; g.K = static_cast<int32_t>(e->K);
        if ((st = begin_kernel(e, e->stream))) return st;
        pick_rowseg_group(e->rg_rows, static_cast<int>(e->K / 32))<<<p.rowgroup_grid, kRowSegWarps * 32, 0, e->stream>>>(g);
        return mark_kernel(e, "sddmm_rowseg_group_kernel", e->stream);
    }
    if (e->rg_rows) {
        RowGroupArgs g;
        g.row_ptr = e->d_rp; g.col_idx = e->d_col; g.s_val = e->d_sval; g.p_val = e->d_pval; g.A = e->d_A32; g.B = e->d_B32;
        g.group_ok = e->d_group_ok; g.M = static_cast<int32_t>(e->M); g.K = static_cast<int32_t>(e->K); g.first = e->rg_first; g.n_groups = e->rg_groups;
        if ((st = begin_kernel(e, e->stream))) return st;
        pick_rowgroup(e->rg_rows, static_cast<int>(e->K / 32))<<<p.rowgroup_grid, kRowGroupWarps * 32, 0, e->stream>>>(g);
        return mark_kernel(e, "sddmm_rowgroup_kernel", e->stream);
    }
    if (e->use_seg) return launch_rowseg(e, e->stream);
    // the two kernels write disjoint nonzeros: when both run, the row-tile kernel goes to the side stream
    static const bool no_side = std::getenv("SDDMM_B200_NO_SIDE_STREAM") != nullptr;   // tuning / debugging knob
    const bool both = e->n_dense > 0 && e->n_residual_items > 0 && !no_side;
    cudaStream_t rt_stream = both ? e->side_stream : e->stream;
    if (both) CU_TRY(e, cudaStreamWaitEvent(e->side_stream, e->ev_run0, 0));   // (run() has just recorded it on the main stream)
    if (e->n_dense > 0) {
        DenseArgs d;
        d.origins = e->dense_origin; d.descs = e->d_dense_descs; d.s_val = e->d_sval; d.p_val = e->d_pval; d.err = e->d_err;
        d.n_tiles = e->n_dense;
        d.k_blocks = static_cast<int32_t>((e->mode == SDDMM_B200_FP32_TC ? 3 * e->K : e->K) / 32);
        d.nnz = e->nnz;
        if ((st = begin_kernel(e, e->stream))) return st;
        using DenseFn = void (*)(const DenseArgs, const CUtensorMap, const CUtensorMap);
        reinterpret_cast<DenseFn>(const_cast<void *>(dense_function(e->dense_own, e->dense_split3)))<<<p.dense_grid, kDenseThreads, p.dense_smem_bytes, e->stream>>>(d, e->map_a, e->map_b);
        if ((st = mark_kernel(e, "sddmm_dense_tile_kernel", e->stream))) return st;
        if (e->n_residual_items == 0) return SDDMM_B200_OK;
    }
    if (e->seg_residual) {
        if ((st = launch_rowseg(e, rt_stream))) return st;
        if (both) {
            CU_TRY(e, cudaEventRecord(e->ev_join, e->side_stream));
            CU_TRY(e, cudaStreamWaitEvent(e->stream, e->ev_join, 0));
        }
        return SDDMM_B200_OK;
    }
    RowTileArgs a;
    a.row_ptr = e->d_rp; a.col_idx = e->d_col; a.s_val = e->d_sval; a.p_val = e->d_pval;
    a.item_rows = e->d_item_rows;
    a.item_ids = e->n_dense > 0 ? e->d_item_ids : nullptr;
    a.covered = e->n_dense > 0 ? e->d_covered : nullptr;
    a.err = e->d_err; a.nnz = e->nnz;
    a.M = static_cast<int32_t>(e->M); a.K = static_cast<int32_t>(e->K);
    a.n_items = p.rowtile_items; a.item_nnz = p.rowtile_item_nnz; a.rows_per_stage = p.rowtile_rows_per_stage;
    if ((st = begin_kernel(e, rt_stream))) return st;
    if (e->mode == SDDMM_B200_BF16) {
        a.A = e->d_A16; a.B = e->d_B16;
        pick_rowtile<__nv_bfloat16>(e->cpl, e->K == 32 * e->cpl)<<<p.rowtile_grid, kBlock, p.rowtile_smem_bytes, rt_stream>>>(a);
    } else {
        a.A = e->d_A32; a.B = e->d_B32;
        pick_rowtile<float>(e->cpl, e->K == 32 * e->cpl)<<<p.rowtile_grid, kBlock, p.rowtile_smem_bytes, rt_stream>>>(a);
    }
    if ((st = mark_kernel(e, "sddmm_rowtile_kernel", rt_stream))) return st;
    if (both) {
        CU_TRY(e, cudaEventRecord(e->ev_join, e->side_stream));
        CU_TRY(e, cudaStreamWaitEvent(e->stream, e->ev_join, 0));
    }
    return SDDMM_B200_OK;
}

// B = NULL in an upload: take the B that sddmm_b200_stage_b left on this engine's device (same N and K)
int take_staged_b(sddmm_b200_engine *e, int64_t N, int64_t K, const float *B) {
    if (B) return SDDMM_B200_OK;
    if (!e->b_stage || e->b_stage_n != N || e->b_stage_k != K)
        return fail(e, SDDMM_B200_ERR_ARG, "B = NULL needs a B of the same shape staged by sddmm_b200_stage_b");
    if (!e->B_on_device) e->B_on_device = e->b_stage;   // (a chunked call sets its own source)
    return SDDMM_B200_OK;
}

}  // namespace

extern "C" {

const char *sddmm_b200_version(void) { return "sddmm_b200 0.1 (sm_100a)"; }

int sddmm_b200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int sddmm_b200_create(sddmm_b200_engine **out, int device, int mode, uint32_t flags) {
    if (!out) return SDDMM_B200_ERR_ARG;
    *out = nullptr;
    if (mode < SDDMM_B200_FP32 || mode > SDDMM_B200_FP32_TC) return SDDMM_B200_ERR_ARG;
    int n = sddmm_b200_device_count();
    if (n <= 0 || device < 0 || device >= n) return SDDMM_B200_ERR_CUDA;
    sddmm_b200_engine *e = new (std::nothrow) sddmm_b200_engine();
    if (!e) return SDDMM_B200_ERR_OOM;
    e->device = device;
    e->mode = mode;
    e->flags = flags;
    e->knob_panels = env_double("SDDMM_B200_PANELS", -1);
    e->knob_panel_mb = env_double("SDDMM_B200_PANEL_MB", -1);
    e->knob_rowseg = env_double("SDDMM_B200_ROWSEG", -1);
    e->knob_b_fraction = env_double("SDDMM_B200_B_FRACTION", -1);
    e->knob_group_units = env_double("SDDMM_B200_GROUP_UNITS", -1);
    e->knob_offset_tiles = env_double("SDDMM_B200_OFFSET_TILES", -1);
    e->knob_dense_split3 = env_double("SDDMM_B200_DENSE_SPLIT3", -1);
    e->knob_k_slices = env_double("SDDMM_B200_K_SLICES", -1);
    e->knob_long_rows = env_double("SDDMM_B200_LONG_ROWS", -1);
    DeviceGuard g(device);
    bool ok = g.ok;
    ok = ok && cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&e->side_stream, cudaStreamNonBlocking) == cudaSuccess;
    for (int i = 0; i < sddmm_b200_engine::kMaxKernels; ++i)
        ok = ok && cudaEventCreate(&e->ev_begin[i]) == cudaSuccess && cudaEventCreate(&e->ev_end[i]) == cudaSuccess;
    ok = ok && cudaEventCreate(&e->ev_run0) == cudaSuccess && cudaEventCreate(&e->ev_run1) == cudaSuccess;
    ok = ok && cudaEventCreate(&e->ev_spmm0) == cudaSuccess && cudaEventCreate(&e->ev_spmm1) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&e->ev_stage, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&e->ev_join, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&e->ev_h2d, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaDeviceGetAttribute(&e->sm_count, cudaDevAttrMultiProcessorCount, device) == cudaSuccess;
    ok = ok && cudaDeviceGetAttribute(&e->l2_bytes, cudaDevAttrL2CacheSize, device) == cudaSuccess;
    ok = ok && cudaHostAlloc(reinterpret_cast<void **>(&e->h_err), sizeof(int32_t), cudaHostAllocDefault) == cudaSuccess;
    ok = ok && cudaHostAlloc(reinterpret_cast<void **>(&e->h_pc), sizeof(PlanCounters), cudaHostAllocDefault) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        sddmm_b200_destroy(e);
        return SDDMM_B200_ERR_CUDA;
    }
    *e->h_err = 0;
    *out = e;
    return SDDMM_B200_OK;
}

int sddmm_b200_destroy(sddmm_b200_engine *e) {
    if (!e) return SDDMM_B200_OK;
    {
        DeviceGuard g(e->device);
        if (e->stream) cudaStreamSynchronize(e->stream);
        if (e->arena.base) cudaFree(e->arena.base);
        if (e->spmm_arena.base) cudaFree(e->spmm_arena.base);
        e->stager.release();
        e->stager2.release();
        if (e->b_stage) cudaFree(e->b_stage);
        if (e->ev_stage) cudaEventDestroy(e->ev_stage);
        if (e->ev_spmm0) cudaEventDestroy(e->ev_spmm0);
        if (e->ev_spmm1) cudaEventDestroy(e->ev_spmm1);
        if (e->h_err) cudaFreeHost(e->h_err);
        if (e->h_pc) cudaFreeHost(e->h_pc);
        if (e->side_stream) cudaStreamSynchronize(e->side_stream);
        for (int i = 0; i < sddmm_b200_engine::kMaxKernels; ++i) {
            if (e->ev_begin[i]) cudaEventDestroy(e->ev_begin[i]);
            if (e->ev_end[i]) cudaEventDestroy(e->ev_end[i]);
        }
        for (cudaEvent_t ev : {e->ev_run0, e->ev_run1, e->ev_join, e->ev_h2d})
            if (ev) cudaEventDestroy(ev);
        if (e->side_stream) cudaStreamDestroy(e->side_stream);
        if (e->stream) cudaStreamDestroy(e->stream);
    }
    delete e;
    return SDDMM_B200_OK;
}

int sddmm_b200_upload_csr(sddmm_b200_engine *e, int64_t M, int64_t N, int64_t K, const int32_t *row_ptr,
                          const int32_t *col_idx, const float *s_val, const float *A, const float *B) {
    if (!e) return SDDMM_B200_ERR_ARG;
    if (!row_ptr || !A) return fail(e, SDDMM_B200_ERR_ARG, "null pointer argument");
    if (M < 1) return fail(e, SDDMM_B200_ERR_ARG, "need M >= 1");
    const int64_t nnz = row_ptr[M];
    int st = check_dims(e, M, N, K, nnz);
    if (st) return st;
    if (nnz > 0 && (!col_idx || !s_val)) return fail(e, SDDMM_B200_ERR_ARG, "null pointer argument");
    if ((st = take_staged_b(e, N, K, B))) return st;
    DeviceGuard g(e->device);
    return upload_common(e, M, N, K, nnz, row_ptr, nullptr, col_idx, s_val, A, B, cudaMemcpyHostToDevice);
}

int sddmm_b200_upload_coo(sddmm_b200_engine *e, int64_t M, int64_t N, int64_t K, int64_t nnz, const int32_t *row_idx,
                          const int32_t *col_idx, const float *s_val, const float *A, const float *B) {
    if (!e) return SDDMM_B200_ERR_ARG;
    if (!A) return fail(e, SDDMM_B200_ERR_ARG, "null pointer argument");
    int st = check_dims(e, M, N, K, nnz);
    if (st) return st;
    if (nnz > 0 && (!row_idx || !col_idx || !s_val)) return fail(e, SDDMM_B200_ERR_ARG, "null pointer argument");
    if ((st = take_staged_b(e, N, K, B))) return st;
    DeviceGuard g(e->device);
    static const int32_t dummy = 0;
    return upload_common(e, M, N, K, nnz, nullptr, nnz ? row_idx : &dummy, col_idx, s_val, A, B, cudaMemcpyHostToDevice);
}

int sddmm_b200_upload_coo_rows(sddmm_b200_engine *e, int64_t M, int64_t N, int64_t K, int64_t nnz, int64_t row_base, const int32_t *row_idx,
                               const int32_t *col_idx, const float *s_val, const float *A, const float *B) {
    if (!e) return SDDMM_B200_ERR_ARG;
    if (row_base < 0 || row_base + M >= (int64_t(1) << 31)) return fail(e, SDDMM_B200_ERR_ARG, "row_base outside the int32 index range");
    e->coo_row_base = static_cast<int32_t>(row_base);
    const int st = sddmm_b200_upload_coo(e, M, N, K, nnz, row_idx, col_idx, s_val, A, B);
    e->coo_row_base = 0;
    return st;
}

int sddmm_b200_upload_csr_device(sddmm_b200_engine *e, int64_t M, int64_t N, int64_t K, const int32_t *row_ptr,
                                 const int32_t *col_idx, const float *s_val, const float *A, const float *B) {
    if (!e) return SDDMM_B200_ERR_ARG;
    if (!row_ptr || !A || !B) return fail(e, SDDMM_B200_ERR_ARG, "null pointer argument");
    if (M < 1) return fail(e, SDDMM_B200_ERR_ARG, "need M >= 1");
    DeviceGuard g(e->device);
    int32_t last = 0;
    CU_TRY(e, cudaMemcpy(&last, row_ptr + M, sizeof(int32_t), cudaMemcpyDeviceToHost));
    const int64_t nnz = last;
    int st = check_dims(e, M, N, K, nnz);
    if (st) return st;
    if (nnz > 0 && (!col_idx || !s_val)) return fail(e, SDDMM_B200_ERR_ARG, "null pointer argument");
    return upload_common(e, M, N, K, nnz, row_ptr, nullptr, col_idx, s_val, A, B, cudaMemcpyDeviceToDevice);
}

int sddmm_b200_update_dense(sddmm_b200_engine *e, const float *A, const float *B) {
    if (!e) return SDDMM_B200_ERR_ARG;
    if (!e->uploaded) return fail(e, SDDMM_B200_ERR_STATE, "update_dense before upload");
    DeviceGuard g(e->device);
    if (A) CU_TRY(e, e->stager.upload(e->d_A32, A, static_cast<size_t>(e->M * e->K) * 4, e->stream));
    if (B) CU_TRY(e, e->stager.upload(e->d_B32, B, static_cast<size_t>(e->N * e->K) * 4, e->stream));
    int st = convert_storage(e);
    if (st) return st;
    CU_TRY(e, cudaStreamSynchronize(e->stream));
    return SDDMM_B200_OK;
}

int sddmm_b200_update_values(sddmm_b200_engine *e, const float *s_val) {
    if (!e) return SDDMM_B200_ERR_ARG;
    if (!e->uploaded) return fail(e, SDDMM_B200_ERR_STATE, "update_values before upload");
    if (!s_val && e->nnz) return fail(e, SDDMM_B200_ERR_ARG, "null pointer argument");
    DeviceGuard g(e->device);
    if (e->nnz) CU_TRY(e, e->stager.upload(e->d_sval, s_val, static_cast<size_t>(e->nnz) * 4, e->stream));
    if (e->use_seg && e->seg_copies && e->n_units > 0) {
        k_unit_values<<<grid_for(8 * static_cast<int64_t>(e->n_units), kBlock, e->sm_count * 32), kBlock, 0, e->stream>>>(e->d_units, e->n_units,
                                                                                                                  e->d_sval, e->d_unit_sval);
        CU_TRY(e, cudaGetLastError());
    }
    CU_TRY(e, cudaStreamSynchronize(e->stream));
    return SDDMM_B200_OK;
}

int sddmm_b200_run(sddmm_b200_engine *e) {
    if (!e) return SDDMM_B200_ERR_ARG;
    if (!e->uploaded) return fail(e, SDDMM_B200_ERR_STATE, "run before upload");
    DeviceGuard g(e->device);
    // (a wait that ran out in an earlier run must not be reported again: the error word starts every run clean)
    CU_TRY(e, cudaMemsetAsync(e->d_err, 0, sizeof(int32_t), e->stream));
    CU_TRY(e, cudaEventRecord(e->ev_run0, e->stream));
    e->last_run_timed = e->kernel_timing;
    int st = launch_all(e);
    if (st) return st;
    CU_TRY(e, cudaEventRecord(e->ev_run1, e->stream));
    CU_TRY(e, cudaMemcpyAsync(e->h_err, e->d_err, sizeof(int32_t), cudaMemcpyDeviceToHost, e->stream));
    e->ran = true;
    return SDDMM_B200_OK;
}

int sddmm_b200_sync(sddmm_b200_engine *e) {
    if (!e) return SDDMM_B200_ERR_ARG;
    DeviceGuard g(e->device);
    CU_TRY(e, cudaStreamSynchronize(e->stream));
    if (e->ran && *e->h_err != kDevOk)
        return fail(e, SDDMM_B200_ERR_DEVICE_WAIT, "device-side bounded wait ran out (code %d)", *e->h_err);
    return SDDMM_B200_OK;
}

int sddmm_b200_download(sddmm_b200_engine *e, float *p_val) {
    if (!e) return SDDMM_B200_ERR_ARG;
    if (!e->uploaded || !e->ran) return fail(e, SDDMM_B200_ERR_STATE, "download before run");
    if (!p_val && e->nnz) return fail(e, SDDMM_B200_ERR_ARG, "null pointer argument");
    DeviceGuard g(e->device);
    if (e->nnz) CU_TRY(e, e->stager.download(p_val, e->d_pval, static_cast<size_t>(e->nnz) * 4, e->stream));
    return sddmm_b200_sync(e);
}

int sddmm_b200_p_device(sddmm_b200_engine *e, float **p) {
    if (!e || !p) return SDDMM_B200_ERR_ARG;
    if (!e->uploaded) return fail(e, SDDMM_B200_ERR_STATE, "p_device before upload");
    *p = e->d_pval;
    return SDDMM_B200_OK;
}

int sddmm_b200_last_run_ms(sddmm_b200_engine *e, float *ms) {
    if (!e || !ms) return SDDMM_B200_ERR_ARG;
    if (!e->ran) return fail(e, SDDMM_B200_ERR_STATE, "last_run_ms before run");
    DeviceGuard g(e->device);
    *ms = 0.f;
    if (e->kernels_launched == 0) return SDDMM_B200_OK;
    CU_TRY(e, cudaEventSynchronize(e->ev_run1));
    CU_TRY(e, cudaEventElapsedTime(ms, e->ev_run0, e->ev_run1));
    return SDDMM_B200_OK;
}

int sddmm_b200_last_kernel_ms(sddmm_b200_engine *e, int index, float *ms, const char **name) {
    if (!e || !ms) return SDDMM_B200_ERR_ARG;
    if (!e->ran) return fail(e, SDDMM_B200_ERR_STATE, "last_kernel_ms before run");
    if (index < 0 || index >= e->kernels_launched) return fail(e, SDDMM_B200_ERR_ARG, "kernel index %d of %d", index, e->kernels_launched);
    if (name) *name = e->kernel_name[index];
    if (!e->last_run_timed) {   // names are always known, times only when the run was asked to record them
        *ms = -1.f;
        return SDDMM_B200_OK;
    }
    DeviceGuard g(e->device);
    CU_TRY(e, cudaEventSynchronize(e->ev_end[index]));
    CU_TRY(e, cudaEventElapsedTime(ms, e->ev_begin[index], e->ev_end[index]));
    return SDDMM_B200_OK;
}

int sddmm_b200_set_kernel_timing(sddmm_b200_engine *e, int enabled) {
    if (!e) return SDDMM_B200_ERR_ARG;
    e->kernel_timing = enabled != 0;
    return SDDMM_B200_OK;
}

// ---- self-test of the bounded device-side wait --------------------------------------------------------------
namespace {
// One thread waits, with the given probe limit, on an mbarrier phase that nothing ever completes, records the time-out
// in the error word exactly as the kernels do, and returns.  Nothing faults and nothing hangs: the wait is bounded.
__global__ void k_wait_timeout_selftest(int32_t *err, uint32_t limit) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
        if (!mbar_wait_bounded(&bar, 0u, limit)) atomicCAS(err, kDevOk, kDevMbarrierTimeout);
    }
}
}  // namespace

int sddmm_b200_selftest_wait_timeout(sddmm_b200_engine *e, int probes) {
    if (!e) return SDDMM_B200_ERR_ARG;
    if (!e->uploaded) return fail(e, SDDMM_B200_ERR_STATE, "selftest before upload (the error word lives in the upload's buffers)");
    if (probes < 1 || probes > (1 << 16)) return fail(e, SDDMM_B200_ERR_ARG, "probes must be in [1, 65536]");
    DeviceGuard g(e->device);
    CU_TRY(e, cudaMemsetAsync(e->d_err, 0, sizeof(int32_t), e->stream));
    k_wait_timeout_selftest<<<1, 32, 0, e->stream>>>(e->d_err, static_cast<uint32_t>(probes));
    CU_TRY(e, cudaGetLastError());
    CU_TRY(e, cudaMemcpyAsync(e->h_err, e->d_err, sizeof(int32_t), cudaMemcpyDeviceToHost, e->stream));
    e->ran = true;   // sync() reports the error word of the last enqueued work
    return sddmm_b200_sync(e);
}

int sddmm_b200_row_cuts(const int32_t *row_ptr, int64_t M, int parts, int64_t align, int64_t *cuts) {
    if (!row_ptr || !cuts || M < 0 || parts < 1) return SDDMM_B200_ERR_ARG;
    const int64_t nnz = row_ptr[M];
    cuts[0] = 0;
    cuts[parts] = M;
    for (int g = 1; g < parts; ++g) {
        const int64_t target = nnz * g / parts;
        int64_t r = std::lower_bound(row_ptr, row_ptr + M + 1, target) - row_ptr;   // first boundary at or past the target
        r = std::min<int64_t>(r, M);
        if (r > 0 && target - row_ptr[r - 1] < row_ptr[r] - target) --r;              // the closer boundary wins
        if (align > 1) r = (r + align / 2) / align * align;
        cuts[g] = std::max<int64_t>(cuts[g - 1], std::min<int64_t>(r, M));
    }
    return SDDMM_B200_OK;
}

int sddmm_b200_coo_cuts(const int32_t *row_idx, int64_t nnz, int64_t M, int parts, int64_t align, int64_t *cuts, int64_t *offsets) {
    if (!cuts || !offsets || M < 0 || nnz < 0 || parts < 1 || (nnz > 0 && !row_idx)) return SDDMM_B200_ERR_ARG;
    cuts[0] = 0;
    offsets[0] = 0;
    cuts[parts] = M;
    offsets[parts] = nnz;
    for (int g = 1; g < parts; ++g) {
        int64_t r = nnz ? row_idx[std::min<int64_t>(nnz - 1, nnz * g / parts)] : 0;   // the row holding the part's first nonzero ...
        if (r < 0 || r >= std::max<int64_t>(M, 1)) return SDDMM_B200_ERR_INDEX;
        if (align > 1) r = std::min<int64_t>((r + align / 2) / align * align, M);
        r = std::max<int64_t>(r, cuts[g - 1]);
        const int64_t pos = std::lower_bound(row_idx, row_idx + nnz, static_cast<int32_t>(r)) - row_idx;   // ... taken whole
        cuts[g] = r;
        offsets[g] = std::max<int64_t>(pos, offsets[g - 1]);
    }
    for (int g = 0; g < parts; ++g)   // nonzeros in a part without rows: the rows cannot be sorted
        if (cuts[g + 1] == cuts[g] && offsets[g + 1] != offsets[g]) return SDDMM_B200_ERR_INDEX;
    return SDDMM_B200_OK;
}

int sddmm_b200_stage_b(sddmm_b200_engine **engines, int n, int64_t N, int64_t K, const float *B) {
    if (!engines || n < 1 || !B || N < 1 || K < 1) return SDDMM_B200_ERR_ARG;
    for (int i = 0; i < n; ++i)
        if (!engines[i]) return SDDMM_B200_ERR_ARG;
    const size_t bytes = static_cast<size_t>(N) * static_cast<size_t>(K) * 4;
    // a staging buffer on every engine's device
    for (int i = 0; i < n; ++i) {
        sddmm_b200_engine *e = engines[i];
        DeviceGuard g(e->device);
        if (!g.ok) return fail(e, SDDMM_B200_ERR_COMM, "device %d cannot be selected", e->device);
        e->b_stage_n = e->b_stage_k = 0;
        if (e->b_stage_cap < bytes) {
            e->stager.release();
        e->stager2.release();
        if (e->b_stage) cudaFree(e->b_stage);
            e->b_stage = nullptr;
            e->b_stage_cap = 0;
            void *p = nullptr;
            if (cudaMalloc(&p, bytes) != cudaSuccess) {
                cudaGetLastError();
                return fail(e, SDDMM_B200_ERR_OOM, "staging buffer for B (%zu bytes) on device %d", bytes, e->device);
            }
            e->b_stage = static_cast<float *>(p);
            e->b_stage_cap = bytes;
        }
    }
    // the host link is crossed once; then the copy doubles the set of devices that hold B in every round
    // (device to device: over NVLink where the devices are peers, through the host otherwise)
    int rc = SDDMM_B200_OK;
    {
        sddmm_b200_engine *e0 = engines[0];
        DeviceGuard g(e0->device);
        if (e0->stager.upload(e0->b_stage, B, bytes, e0->stream) != cudaSuccess ||
            cudaEventRecord(e0->ev_stage, e0->stream) != cudaSuccess)
            rc = fail(e0, SDDMM_B200_ERR_COMM, "upload of B to device %d: %s", e0->device, cudaGetErrorString(cudaGetLastError()));
    }
    for (int have = 1; have < n && !rc; have *= 2) {
        for (int i = 0; i < have && have + i < n && !rc; ++i) {
            sddmm_b200_engine *src = engines[i], *dst = engines[have + i];
            DeviceGuard g(dst->device);
            cudaError_t st = cudaStreamWaitEvent(dst->stream, src->ev_stage, 0);
            if (st == cudaSuccess) {
                if (src->device == dst->device) {
                    st = cudaMemcpyAsync(dst->b_stage, src->b_stage, bytes, cudaMemcpyDeviceToDevice, dst->stream);
                } else {
                    int can = 0;
                    if (cudaDeviceCanAccessPeer(&can, dst->device, src->device) == cudaSuccess && can) {
                        const cudaError_t pe = cudaDeviceEnablePeerAccess(src->device, 0);   // (already enabled is fine)
                        if (pe != cudaSuccess) cudaGetLastError();
                    }
                    st = cudaMemcpyPeerAsync(dst->b_stage, dst->device, src->b_stage, src->device, bytes, dst->stream);
                }
            }
            if (st == cudaSuccess) st = cudaEventRecord(dst->ev_stage, dst->stream);
            if (st != cudaSuccess) {
                cudaGetLastError();
                rc = fail(dst, SDDMM_B200_ERR_COMM, "copy of B from device %d to device %d: %s", src->device, dst->device, cudaGetErrorString(st));
            }
        }
    }
    for (int i = 0; i < n; ++i) {   // drain every stream, also after a failure: nothing may still read the caller's buffer
        sddmm_b200_engine *e = engines[i];
        DeviceGuard g(e->device);
        if (cudaStreamSynchronize(e->stream) != cudaSuccess && !rc) {
            cudaGetLastError();
            rc = fail(e, SDDMM_B200_ERR_COMM, "copy of B to device %d did not complete", e->device);
        }
    }
    if (rc) return rc;
    for (int i = 0; i < n; ++i) {
        engines[i]->b_stage_n = N;
        engines[i]->b_stage_k = K;
    }
    return SDDMM_B200_OK;
}

int sddmm_b200_set_knob(sddmm_b200_engine *e, const char *name, double value) {
    if (!e || !name) return SDDMM_B200_ERR_ARG;
    struct { const char *name; double *slot; } knobs[] = {
        {"panels", &e->knob_panels}, {"panel_mb", &e->knob_panel_mb}, {"rowseg", &e->knob_rowseg},
        {"b_fraction", &e->knob_b_fraction}, {"group_units", &e->knob_group_units},
        {"offset_tiles", &e->knob_offset_tiles}, {"dense_split3", &e->knob_dense_split3}, {"k_slices", &e->knob_k_slices}, {"long_rows", &e->knob_long_rows},
    };
    for (auto &k : knobs)
        if (std::strcmp(name, k.name) == 0) {
            *k.slot = value;
            return SDDMM_B200_OK;
        }
    return fail(e, SDDMM_B200_ERR_ARG, "unknown knob '%s'", name);
}

// ---- consumer of P on the device: Y = P X ----------------------------------------------------------------
namespace {
using SpmmFn = void (*)(const SpmmArgs);
SpmmFn pick_spmm(int cpl, bool exact) {
    switch (cpl) {
        case 1: return exact ? sddmm_spmm_kernel<1, true> : sddmm_spmm_kernel<1, false>;
        case 2: return exact ? sddmm_spmm_kernel<2, true> : sddmm_spmm_kernel<2, false>;
        case 4: return exact ? sddmm_spmm_kernel<4, true> : sddmm_spmm_kernel<4, false>;
        case 8: return exact ? sddmm_spmm_kernel<8, true> : sddmm_spmm_kernel<8, false>;
        default: return nullptr;
    }
}

// X, Y and the consumer's unit list live in their own buffer (grown on demand, kept across calls)
int spmm_prepare(sddmm_b200_engine *e, int64_t K2) {
    Carve c;
    const size_t M = static_cast<size_t>(e->M), N = static_cast<size_t>(e->N), nnz = static_cast<size_t>(e->nnz);
    const size_t cap = nnz / 8 + std::min(M, nnz) + 8;
    const size_t o_x = c.take(N * K2 * 4), o_y = c.take(M * K2 * 4), o_u = c.take(cap * sizeof(int2));
    const bool grow = c.off > e->spmm_arena.cap;
    if (grow) {
        if (e->spmm_arena.base) CU_TRY(e, cudaFree(e->spmm_arena.base));
        e->spmm_arena.base = nullptr;
        e->spmm_arena.cap = 0;
        void *p = nullptr;
        if (cudaMalloc(&p, c.off) != cudaSuccess) {
            cudaGetLastError();
            return fail(e, SDDMM_B200_ERR_OOM, "consumer buffers of %zu bytes", c.off);
        }
        e->spmm_arena.base = static_cast<char *>(p);
        e->spmm_arena.cap = c.off;
        e->spmm_units = 0;
    }
    char *b = e->spmm_arena.base;
    const bool moved = e->d_spmm_units != reinterpret_cast<int2 *>(b + o_u);
    e->d_X = reinterpret_cast<float *>(b + o_x);
    e->d_Y = reinterpret_cast<float *>(b + o_y);
    e->d_spmm_units = reinterpret_cast<int2 *>(b + o_u);
    e->spmm_k2 = K2;
    if (e->spmm_units == 0 || moved) {   // plain row segments (one panel, no groups), counted / scanned / written on the device
        const int32_t Mi = static_cast<int32_t>(e->M);
        const int n_tiles = static_cast<int>((e->M + kScanTile - 1) / kScanTile);
        const int capb = e->sm_count * 32;
        cudaStream_t s = e->stream;
        k_unit_count<<<grid_for(e->M, kBlock, capb), kBlock, 0, s>>>(e->d_rp, e->d_col, Mi, 1, 0, 0, e->d_unit_off);
        k_scan_tile_sums<<<n_tiles, kScanBlock, 0, s>>>(e->d_unit_off, e->M, e->d_scan_tiles);
        k_scan_sums<<<1, kScanBlock, 0, s>>>(e->d_scan_tiles, n_tiles, &e->d_pc->units);
        k_scan_apply<<<n_tiles, kScanBlock, 0, s>>>(e->d_unit_off, e->M, e->d_scan_tiles);
        k_unit_fill<<<grid_for(e->M * 32, kBlock, capb), kBlock, 0, s>>>(e->d_rp, e->d_col, Mi, 1, 0, 0, e->d_unit_off, e->d_spmm_units, nullptr);
        CU_TRY(e, cudaGetLastError());
        PlanCounters pc;
        if (int rc = read_counters(e, &pc)) return rc;
        if (pc.units == 0 || pc.units > cap) return fail(e, SDDMM_B200_ERR_CUDA, "consumer plan: %llu units for a list of %zu", pc.units, cap);
        e->spmm_units = static_cast<int32_t>(pc.units);
    }
    return SDDMM_B200_OK;
}
}  // namespace

int sddmm_b200_spmm(sddmm_b200_engine *e, int64_t K2, const float *X, float *Y) {
    if (!e) return SDDMM_B200_ERR_ARG;
    if (!e->uploaded || !e->ran) return fail(e, SDDMM_B200_ERR_STATE, "spmm before run");
    if (K2 < 4 || K2 % 4 != 0 || K2 > 256) return fail(e, SDDMM_B200_ERR_UNSUPPORTED, "the consumer needs K2 %% 4 == 0 and 4 <= K2 <= 256 (K2 = %lld)", (long long)K2);
    if (!Y) return fail(e, SDDMM_B200_ERR_ARG, "null pointer argument");
    if (!X && K2 != e->K) return fail(e, SDDMM_B200_ERR_ARG, "X = NULL means X = B, which needs K2 == K");
    if (e->M >= kUnitRowLimit) return fail(e, SDDMM_B200_ERR_UNSUPPORTED, "the consumer handles fewer than 2^28 rows");
    DeviceGuard g(e->device);
    cudaStream_t s = e->stream;
    const size_t ybytes = static_cast<size_t>(e->M) * K2 * 4;
    if (e->nnz == 0) {
        std::memset(Y, 0, ybytes);
        return sddmm_b200_sync(e);
    }
    int st = spmm_prepare(e, K2);   // (uses the plan scratch of the main arena: nothing of the run still needs it)
    if (st) return st;
    if (X) CU_TRY(e, cudaMemcpyAsync(e->d_X, X, static_cast<size_t>(e->N) * K2 * 4, cudaMemcpyHostToDevice, s));
    CU_TRY(e, cudaEventRecord(e->ev_spmm0, s));
    CU_TRY(e, cudaMemsetAsync(e->d_Y, 0, ybytes, s));
    SpmmArgs a;
    a.units = e->d_spmm_units; a.col_idx = e->d_col; a.p_val = e->d_pval; a.X = X ? e->d_X : e->d_B32; a.Y = e->d_Y;
    a.n_units = e->spmm_units; a.K2 = static_cast<int32_t>(K2);
    const int cpl = round_up_cpl(K2);
    SpmmFn fn = pick_spmm(cpl, K2 == 32 * cpl);
    int occ = 0;
    CU_TRY(e, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, kSpmmWarps * 32, 0));
    if (occ < 1) return fail(e, SDDMM_B200_ERR_CUDA, "consumer kernel does not fit on an SM");
    const int64_t n_quads = (static_cast<int64_t>(e->spmm_units) + 3) / 4;
    const int grid = static_cast<int>(std::min<int64_t>((n_quads + kSpmmWarps - 1) / kSpmmWarps, static_cast<int64_t>(e->sm_count) * occ));
    fn<<<grid, kSpmmWarps * 32, 0, s>>>(a);
    CU_TRY(e, cudaGetLastError());
    CU_TRY(e, cudaEventRecord(e->ev_spmm1, s));
    CU_TRY(e, cudaMemcpyAsync(Y, e->d_Y, ybytes, cudaMemcpyDeviceToHost, s));
    return sddmm_b200_sync(e);
}

int sddmm_b200_last_spmm_ms(sddmm_b200_engine *e, float *ms) {
    if (!e || !ms) return SDDMM_B200_ERR_ARG;
    if (!e->spmm_k2) return fail(e, SDDMM_B200_ERR_STATE, "last_spmm_ms before spmm");
    DeviceGuard g(e->device);
    CU_TRY(e, cudaEventSynchronize(e->ev_spmm1));
    CU_TRY(e, cudaEventElapsedTime(ms, e->ev_spmm0, e->ev_spmm1));
    return SDDMM_B200_OK;
}

int sddmm_b200_get_plan(sddmm_b200_engine *e, sddmm_b200_plan_info *info) {
    if (!e || !info) return SDDMM_B200_ERR_ARG;
    if (!e->uploaded) return fail(e, SDDMM_B200_ERR_STATE, "get_plan before upload");
    *info = e->plan;
    return SDDMM_B200_OK;
}

int64_t sddmm_b200_algorithmic_bytes(sddmm_b200_engine *e) {
    if (!e || !e->uploaded) return -1;
    const int64_t eb = static_cast<int64_t>(elem_bytes(e));
    return eb * e->K * (e->plan.rows_nonempty + e->plan.cols_touched) + 12 * e->nnz + 4 * (e->M + 1);
}

int64_t sddmm_b200_flops(sddmm_b200_engine *e) {
    if (!e || !e->uploaded) return -1;
    return 2 * e->nnz * e->K;
}

const char *sddmm_b200_last_error(sddmm_b200_engine *e) { return e ? e->err : "null engine"; }

void *sddmm_b200_stream(sddmm_b200_engine *e) { return e ? static_cast<void *>(e->stream) : nullptr; }

int sddmm_b200_host_alloc(void **ptr, int64_t bytes) {
    if (!ptr || bytes < 0) return SDDMM_B200_ERR_ARG;
    cudaError_t st = cudaHostAlloc(ptr, static_cast<size_t>(std::max<int64_t>(bytes, 1)), cudaHostAllocDefault);
    if (st != cudaSuccess) {
        cudaGetLastError();
        *ptr = nullptr;
        return st == cudaErrorMemoryAllocation ? SDDMM_B200_ERR_OOM : SDDMM_B200_ERR_CUDA;
    }
    return SDDMM_B200_OK;
}

int sddmm_b200_host_free(void *ptr) {
    if (!ptr) return SDDMM_B200_OK;
    return cudaFreeHost(ptr) == cudaSuccess ? SDDMM_B200_OK : SDDMM_B200_ERR_CUDA;
}


// ---------------------------------------------------------------------------------------------
// Allocation-free SDDMM (see sddmm_b200_sddmm_csr_prealloc in the header).
//
// The row-tile kernel needs two pieces of scratch besides its operands: the table that says in which
// rows each nnz-balanced work item begins and ends, and an error word for its bounded waits.  Here
// both live in a fixed device array that is part of the loaded library image, so the call below never
// asks the CUDA allocator for anything.  The array name is only a host-side handle: its device address
// is looked up once per device with cudaGetSymbolAddress (that device current) and cached.
constexpr int64_t kPreallocMaxNnz = int64_t(1) << 27;                   // 134 217 728 nonzeros
constexpr int kPreallocItemNnz = 2048;
constexpr int64_t kPreallocMaxItems = kPreallocMaxNnz / kPreallocItemNnz;  // 65 536 work items
constexpr size_t kPreallocTableBytes = static_cast<size_t>(kPreallocMaxItems) * sizeof(int2);   // 512 KiB
constexpr size_t kPreallocScratchBytes = kPreallocTableBytes + 256;      // + the error word, on its own 256-byte line
static __device__ __align__(256) unsigned char g_prealloc_scratch[kPreallocScratchBytes];

constexpr int kPreallocMaxDevices = 64;
static unsigned char *g_prealloc_ptr[kPreallocMaxDevices] = {nullptr};   // device address of the array, per device

int sddmm_b200_sddmm_csr_prealloc(int device, void *cuda_stream, int64_t M, int64_t N, int64_t K, int64_t nnz,
                                  const int32_t *d_row_ptr, const int32_t *d_col_idx, const float *d_s_val,
                                  const float *d_A, const float *d_B, float *d_p_val) {
    if (M < 1 || N < 1 || K < 1 || nnz < 0 || device < 0 || device >= kPreallocMaxDevices) return SDDMM_B200_ERR_ARG;
    if (!d_row_ptr || !d_A || !d_B || (nnz > 0 && (!d_col_idx || !d_s_val || !d_p_val))) return SDDMM_B200_ERR_ARG;
    if (M >= (int64_t(1) << 31) - 1 || N >= (int64_t(1) << 31) - 1) return SDDMM_B200_ERR_ARG;
    // the kernel reads col_idx, A and B with 16-byte accesses (the engine's own arena is 256-byte aligned; a caller's
    // pointer into the middle of a larger buffer may not be) -- refused here rather than faulting on the GPU
    auto misaligned = [](const void *ptr, uintptr_t a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) != 0; };
    if (misaligned(d_A, 16) || misaligned(d_B, 16) || (nnz > 0 && misaligned(d_col_idx, 16))) return SDDMM_B200_ERR_ARG;
    if (misaligned(d_row_ptr, 4) || (nnz > 0 && (misaligned(d_s_val, 4) || misaligned(d_p_val, 4)))) return SDDMM_B200_ERR_ARG;
    if (nnz > kPreallocMaxNnz) return SDDMM_B200_ERR_UNSUPPORTED;        // the work-item table would not fit the fixed scratch
    const int cpl = round_up_cpl(K);
    if (K % 4 != 0 || cpl == 0) return SDDMM_B200_ERR_UNSUPPORTED;      // only the row-tile kernel (K % 4 == 0, K <= 256) is offered here
    if (nnz == 0) return SDDMM_B200_OK;
    DeviceGuard g(device);
    if (!g.ok) return SDDMM_B200_ERR_CUDA;
    if (!g_prealloc_ptr[device]) {   // first call on this device: resolve the array's device address
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_prealloc_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return SDDMM_B200_ERR_CUDA;
        }
        g_prealloc_ptr[device] = static_cast<unsigned char *>(p);
    }
    int2 *item_rows = reinterpret_cast<int2 *>(g_prealloc_ptr[device]);
    int32_t *err = reinterpret_cast<int32_t *>(g_prealloc_ptr[device] + kPreallocTableBytes);
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);

    const int n_items = static_cast<int>((nnz + kPreallocItemNnz - 1) / kPreallocItemNnz);
    // the array keeps whatever the previous call left: the error word must start at zero, the table is rewritten
    if (cudaMemsetAsync(err, 0, sizeof(int32_t), st) != cudaSuccess) return SDDMM_B200_ERR_CUDA;
    k_item_rows<<<grid_for(n_items, kBlock, 1 << 30), kBlock, 0, st>>>(d_row_ptr, static_cast<int32_t>(M), nnz, kPreallocItemNnz, n_items, item_rows);

    int64_t R = kPreallocItemNnz / std::max<int64_t>(1, nnz / M) + 1;
    R = (R + 7) / 8 * 8;
    R = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(R, kMaxStageBytes / (K * 4)), M));
    const int smem = static_cast<int>(rowtile_smem_bytes(static_cast<int>(R), static_cast<uint32_t>(K * 4)));
    const bool exact = (K == 32 * cpl);
    RowTileFn<float> fn = pick_rowtile<float>(cpl, exact);
    if (ensure_dynamic_smem_limit(reinterpret_cast<const void *>(fn), device, kRowTileMaxSmem)) return SDDMM_B200_ERR_CUDA;
    int occ = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, reinterpret_cast<const void *>(fn), kBlock, smem) != cudaSuccess || occ < 1) return SDDMM_B200_ERR_CUDA;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return SDDMM_B200_ERR_CUDA;

    RowTileArgs a;
    a.row_ptr = d_row_ptr; a.col_idx = d_col_idx; a.s_val = d_s_val; a.p_val = d_p_val; a.A = d_A; a.B = d_B;
    a.item_rows = item_rows; a.item_ids = nullptr; a.covered = nullptr;
    a.err = err; a.nnz = nnz; a.M = static_cast<int32_t>(M); a.K = static_cast<int32_t>(K);
    a.n_items = n_items; a.item_nnz = kPreallocItemNnz; a.rows_per_stage = static_cast<int32_t>(R);
    fn<<<std::min(n_items, sms * occ), kBlock, smem, st>>>(a);
    if (cudaGetLastError() != cudaSuccess) return SDDMM_B200_ERR_CUDA;
    int32_t h_err = 0;   // synchronous by contract: wait, then read the error word back
    if (cudaMemcpyAsync(&h_err, err, sizeof(int32_t), cudaMemcpyDeviceToHost, st) != cudaSuccess) return SDDMM_B200_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return SDDMM_B200_ERR_CUDA;
    return h_err == kDevOk ? SDDMM_B200_OK : SDDMM_B200_ERR_DEVICE_WAIT;
}

}  // extern "C"

#include "pipeline.cuh"
