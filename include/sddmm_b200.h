/*
 * sddmm_b200.h -- C ABI of the B200 (sm_100a) SDDMM engine.
 *
 *   P_ij = S_ij * (A_i . B_j)   for every (i,j) on the sparsity pattern of S
 *
 * A is dense M x K row-major, B is dense N x K row-major (i.e. already the
 * transposed right-hand operand), S and P share one CSR (or COO) pattern with
 * int32 indices.  Values are fp32 in host memory in every mode.
 *
 * This is the boundary a host program binds instead of the per-competitor
 * CUDA wrappers of francois141/dphpc.  Each entry point names the reference
 * interface it stands in for (paths are relative to that project's root).
 *
 * Conventions: plain C types only, caller-owned buffers, every call returns an
 * int status (0 = ok), a human-readable reason is kept per engine and returned
 * by sddmm_b200_last_error().  No call throws, none falls back to a CPU path:
 * without a CUDA device every compute entry point returns SDDMM_B200_ERR_CUDA.
 */
#ifndef SDDMM_B200_H
#define SDDMM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sddmm_b200_engine sddmm_b200_engine;

/* status codes */
enum {
    SDDMM_B200_OK            = 0,
    SDDMM_B200_ERR_ARG       = 1,  /* null pointer, negative size, K < 1 ...       */
    SDDMM_B200_ERR_INDEX     = 2,  /* row_ptr not monotone / col out of range / COO rows unsorted */
    SDDMM_B200_ERR_OOM       = 3,  /* device or host allocation failed            */
    SDDMM_B200_ERR_CUDA      = 4,  /* any other CUDA runtime failure              */
    SDDMM_B200_ERR_STATE     = 5,  /* call order violated (run before upload ...) */
    SDDMM_B200_ERR_UNSUPPORTED = 6,
    SDDMM_B200_ERR_COMM      = 7,  /* a copy between devices failed (sddmm_b200_stage_b) */
    SDDMM_B200_ERR_DEVICE_WAIT = 8 /* a bounded device-side wait ran out          */
};

/* arithmetic modes */
enum {
    SDDMM_B200_FP32 = 0,  /* fp32 storage, fp32 FMA everywhere (parity bar: rel 1e-5)                  */
    SDDMM_B200_TF32 = 1,  /* fp32 storage; >=50%-full tiles on tcgen05 kind::tf32 (rel 1e-2)           */
    SDDMM_B200_BF16 = 2,  /* A and B stored as bf16 on the device, fp32 accumulate (rel 1e-2); K % 8 == 0, K <= 256 */
    SDDMM_B200_FP32_TC = 3 /* fp32 storage; dense tiles on tcgen05 with a 3-term tf32 split (rel 1e-5) */
};

/* flags for sddmm_b200_create */
enum {
    SDDMM_B200_FLAG_NO_DENSE_TILES = 1u << 0, /* never take the tensor-core tile path */
    SDDMM_B200_FLAG_NO_ROW_GROUPS  = 1u << 1, /* never merge rows with identical column lists */
    SDDMM_B200_FLAG_NO_ROW_SEGMENTS = 1u << 2 /* never take the row-segment kernel (the A-row-tile kernel runs instead) */
};

#define SDDMM_B200_HIST_BINS 20

typedef struct sddmm_b200_plan_info {
    int64_t rows, cols, k, nnz;
    int64_t rows_nonempty;         /* M+ : rows with at least one nonzero            */
    int64_t cols_touched;          /* N+ : distinct column indices present           */
    int64_t max_row_nnz;
    int64_t row_len_hist[SDDMM_B200_HIST_BINS]; /* bin 0: empty rows, bin b>=1: 2^(b-1) <= len < 2^b */
    int32_t cols_sorted;           /* 1 if col_idx is non-decreasing inside every row */
    int32_t mode;
    /* generic (row-tile) kernel */
    int64_t rowtile_nnz;           /* nonzeros handled by the row-tile kernel        */
    int32_t rowtile_items;         /* nnz-balanced work items                        */
    int32_t rowtile_item_nnz;      /* nonzeros per work item                         */
    int32_t rowtile_rows_per_stage;/* A rows staged in shared memory at a time       */
    int32_t rowtile_grid, rowtile_block, rowtile_smem_bytes;
    /* dense-tile (tensor-core) kernel */
    int64_t dense_nnz;             /* nonzeros handled by the dense-tile kernel      */
    int32_t dense_tiles;           /* tiles at least half full                        */
    int32_t dense_tile_rows, dense_tile_cols;
    int32_t dense_grid, dense_block, dense_smem_bytes;
    /* row groups (consecutive rows with identical column lists) */
    int64_t rowgroup_nnz;          /* nonzeros inside matching groups (the row-group kernel, when it runs, handles ALL nonzeros) */
    int32_t rowgroup_groups;       /* matching groups                                  */
    int32_t rowgroup_rows;         /* rows per aligned group (2, 3, 4); 0: path not taken */
    int32_t rowgroup_grid;
    int32_t n_kernels;             /* kernels one run() launches                      */
    int32_t n_devices;
    /* row segments (rows cut into pieces of at most 8 nonzeros; the path for short and power-law rows) */
    int64_t rowseg_nnz;            /* nonzeros handled by the row-segment kernel      */
    int32_t rowseg_units;          /* segments                                        */
    int32_t rowseg_panels;         /* column panels the segment list is ordered by (1: none); with panels for the long rows only, the short rows count as one more */
    int32_t rowseg_grid;
    int32_t rowseg_passes;      /* launches of the row-segment kernel per run: K taken in slices of 64 columns (else 1, or 0) */
} sddmm_b200_plan_info;

/* ---- life cycle ---------------------------------------------------------
 * Replaces the cudaMalloc / cudaFree blocks every reference competitor has in
 * init_csr / cleanup_csr (src/competitors/gpu/gpu_convert.hpp:20-50, 58-74):
 * the engine owns one device arena that is reused across uploads. */
int sddmm_b200_create(sddmm_b200_engine **out, int device, int mode, uint32_t flags);
int sddmm_b200_destroy(sddmm_b200_engine *e);

/* ---- upload (host buffers) ----------------------------------------------
 * Replaces the H2D half of Competitor<T>::init_csr / init_coo
 * (src/benchmark/competitor.hpp:27-28; e.g. src/competitors/gpu/gpu_basic.hpp:33-60)
 * and the host-side preprocessing of GPUPreprocessing::init_csr
 * (src/competitors/gpu/gpu_preprocessing.hpp:56-128): validation, the
 * row-length histogram and the kernel plan are all built on the device here.
 * row_ptr has M+1 entries, col_idx/s_val have row_ptr[M] entries. */
int sddmm_b200_upload_csr(sddmm_b200_engine *e, int64_t M, int64_t N, int64_t K,
                          const int32_t *row_ptr, const int32_t *col_idx, const float *s_val,
                          const float *A, const float *B);
/* COO entries must be sorted by row (the reference's COO<T> always is,
 * src/matrices/COO.hpp:39); row_ptr is derived on the device. */
int sddmm_b200_upload_coo(sddmm_b200_engine *e, int64_t M, int64_t N, int64_t K, int64_t nnz,
                          const int32_t *row_idx, const int32_t *col_idx, const float *s_val,
                          const float *A, const float *B);
/* A row slice of a larger COO matrix: the slice holds rows [row_base, row_base + M) of it, row_idx keeps the
 * matrix' own (global) row numbers and the device subtracts row_base while it derives row_ptr -- the host neither
 * copies nor rewrites the index array (row shards of one matrix on several engines).  A must point at the slice's
 * first row.  SDDMM_B200_ERR_INDEX when a row index lies outside the slice. */
int sddmm_b200_upload_coo_rows(sddmm_b200_engine *e, int64_t M, int64_t N, int64_t K, int64_t nnz, int64_t row_base,
                               const int32_t *row_idx, const int32_t *col_idx, const float *s_val,
                               const float *A, const float *B);
/* Same as upload_csr but every pointer is a DEVICE pointer on the engine's
 * device (e.g. B received by an NCCL broadcast). The data is copied into the
 * engine's own aligned arena.  No reference counterpart (the reference keeps
 * nothing resident between runs). */
int sddmm_b200_upload_csr_device(sddmm_b200_engine *e, int64_t M, int64_t N, int64_t K,
                                 const int32_t *row_ptr, const int32_t *col_idx, const float *s_val,
                                 const float *A, const float *B);
/* Replace only the dense operands / only S's values, keeping pattern and plan
 * (host pointers). */
int sddmm_b200_update_dense(sddmm_b200_engine *e, const float *A, const float *B);
int sddmm_b200_update_values(sddmm_b200_engine *e, const float *s_val);

/* ---- compute --------------------------------------------------------------
 * Replaces Competitor<T>::run_csr / run_coo (src/benchmark/competitor.hpp:30-31;
 * e.g. GPUConvert::run_csr, src/competitors/gpu/gpu_convert.cu:54-74).
 * run() only enqueues on the engine's stream; sync() blocks until done and
 * reports device-side errors. */
int sddmm_b200_run(sddmm_b200_engine *e);
int sddmm_b200_sync(sddmm_b200_engine *e);

/* ---- download ---------------------------------------------------------------
 * Replaces the D2H half of cleanup_csr / cleanup_coo
 * (src/competitors/gpu/gpu_convert.hpp:58-64): writes nnz floats, in the order
 * of the uploaded col_idx. */
int sddmm_b200_download(sddmm_b200_engine *e, float *p_val);
/* device pointer to the nnz output values (valid until the next upload). */
int sddmm_b200_p_device(sddmm_b200_engine *e, float **p_val_device);

/* ---- consumer of P on the device ---------------------------------------------
 * Y = P X for the P of the last run(), which stays on the GPU: X is dense N x K2, Y dense M x K2 (host pointers,
 * row-major fp32; K2 % 4 == 0, 4 <= K2 <= 256).  X = NULL stands for X = B, the copy the engine already holds (K2 must
 * equal K; in bf16 mode that copy carries the bf16-rounded values): nothing is uploaded.  No counterpart in the reference, whose competitors end by copying P
 * back to the host (cleanup_csr, src/competitors/gpu/gpu_convert.hpp:58-64); its report names this product (SpMM after
 * SDDMM, ALS-style updates) as what SDDMM results are used for.  A caller that only needs Y skips the download of
 * P.val (4 bytes per nonzero) and copies M * K2 floats instead.  Synchronous.  Partial row sums are added to Y with
 * floating-point reductions whose order is not fixed: Y is reproducible to fp32 rounding, not bit for bit.
 * sddmm_b200_last_spmm_ms: device time of the consumer kernel (with the clearing of Y) of the last call. */
int sddmm_b200_spmm(sddmm_b200_engine *e, int64_t K2, const float *X, float *Y);
int sddmm_b200_last_spmm_ms(sddmm_b200_engine *e, float *ms);

/* ---- introspection ----------------------------------------------------------
 * Device time of the last run() (CUDA events on the engine's stream), standing
 * in for the cudaEvent pair of Benchmark<T>::timing (src/benchmark/benchmark.hpp:160-164). */
int sddmm_b200_last_run_ms(sddmm_b200_engine *e, float *ms);
/* Device time and name of kernel `index` (0 .. plan.n_kernels-1) of the last run().  The name is always
 * returned; the time only if per-kernel timing was on for that run (else *ms = -1): an event pair around
 * every kernel costs several microseconds per launch, so it is off unless asked for. */
int sddmm_b200_last_kernel_ms(sddmm_b200_engine *e, int index, float *ms, const char **name);
int sddmm_b200_set_kernel_timing(sddmm_b200_engine *e, int enabled);
int sddmm_b200_get_plan(sddmm_b200_engine *e, sddmm_b200_plan_info *info);
/* Tuning knobs of the planner (the thread-grid command-line options of the reference's driver, src/main.cpp:326-348, and
 * the density threshold of GPUDynamic, src/competitors/gpu/gpu_dynamic.hpp:72-73, play this role there).  A negative
 * value hands the decision back to the planner; a knob takes effect at the next upload ("b_fraction" at the next run).  Defaults come from the environment variables SDDMM_B200_<NAME IN CAPITALS> at create.
 *   "panels"        column panels of the row-segment path (1..64)
 *   "panel_mb"      target size of one panel of B in MiB
 *   "rowseg"        0: never take the row-segment kernel, 1: take it whenever it applies
 *   "b_fraction"    with column panels the gathers of B carry an L2 evict_last hint: share of the lines it applies to, (0, 1]
 *   "group_units"   0: rows with identical column lists run the warp-per-group kernel instead of shared segments
 *   "offset_tiles"  0: dense tiles only on the 64-grid, 1: always also look for half-full 64x64 windows at arbitrary offsets
 *   "k_slices"      fp32 storage, K >= 128 and a multiple of 64: 1 = take K in slices of 64 columns (one launch each over the same
 *                   segment list, adding to P.val; default when B is larger than four times the L2), 0 = never
 *   "long_rows"     rows too short for column panels on average but B far larger than L2: column panels for the rows of at
 *                   least this many nonzeros only, the shorter rows follow whole (default: 64 or 128, chosen with the number
 *                   of panels, when such rows hold at least 40 % of the nonzeros); 0 = never
 *   "dense_split3"  fp32-grade mode on dense tiles: 1 = operands through three shared-memory slots and two accumulators in
 *                   tensor memory (default for K >= 64), 0 = one A block + one B block like the other modes */
int sddmm_b200_set_knob(sddmm_b200_engine *e, const char *name, double value);
/* compulsory traffic e*K*(M+ + N+) + 12*nnz + 4*(M+1) with e = bytes per stored
 * element of A/B; extends the read-only model of plots/plot_roofline.py:30 */
int64_t sddmm_b200_algorithmic_bytes(sddmm_b200_engine *e);
int64_t sddmm_b200_flops(sddmm_b200_engine *e); /* 2*nnz*K (plots/plot_roofline.py:29 without the +nnz) */
const char *sddmm_b200_last_error(sddmm_b200_engine *e);
/* raw CUDA stream (cudaStream_t) the engine launches on, for external event timing */
void *sddmm_b200_stream(sddmm_b200_engine *e);
int sddmm_b200_device_count(void);
const char *sddmm_b200_version(void);

/* ---- allocation-free call ---------------------------------------------------------
 * No counterpart in the reference (every competitor there allocates in init_*).
 *
 * For callers that must not reach the CUDA allocator when they need an SDDMM: code running
 * inside a framework that owns all device memory through its own pool and forbids foreign
 * cudaMalloc calls, a real-time loop that cannot take the allocator's lock or its implicit
 * device synchronisation, a process whose memory is already fully committed.  Everything is
 * caller-owned DEVICE memory on `device`; the work-item table and the error word the row-tile
 * kernel needs live in a fixed 512.25 KiB array inside the library image (every GPU that loads
 * the library holds it until the process exits), so the call performs no cudaMalloc, cudaFree
 * or other allocating call.
 *
 *   - fp32, CSR, K % 4 == 0 and K <= 256, nnz <= 2^27 (134 217 728); anything else returns
 *     SDDMM_B200_ERR_UNSUPPORTED and touches nothing.  row_ptr/col_idx are trusted (not validated).
 *   - alignment: d_col_idx, d_A and d_B must be 16-byte aligned (the kernel reads them with 128-bit
 *     accesses), d_row_ptr, d_s_val and d_p_val 4-byte aligned; a row-shard slice such as
 *     d_col_idx + offset qualifies only when offset % 4 == 0.  Anything else returns
 *     SDDMM_B200_ERR_ARG before any launch.
 *   - synchronous: work is enqueued on `cuda_stream` (a cudaStream_t, may be 0) and the call
 *     returns after that stream has drained.
 *   - the first call on a device looks up the array's device address; make that call outside
 *     any stream capture.
 *   - all calls on one device share the array and it keeps the last call's contents (the parts
 *     that must start clean are reset by each call): two calls that overlap on the same GPU
 *     race on it -- serialise them. */
int sddmm_b200_sddmm_csr_prealloc(int device, void *cuda_stream, int64_t M, int64_t N, int64_t K, int64_t nnz,
                                  const int32_t *d_row_ptr, const int32_t *d_col_idx, const float *d_s_val,
                                  const float *d_A, const float *d_B, float *d_p_val);

/* ---- chunked host-to-host call ------------------------------------------------------
 * The one-shot sequence of the reference's harness -- init_csr, run_csr, cleanup_csr
 * (src/benchmark/benchmark.hpp:81-83) -- as ONE call on host buffers, with the three phases
 * of consecutive row chunks overlapped: the rows of S are cut into up to `chunks` contiguous
 * ranges with equal shares of the nonzeros; while one range is planned, computed and copied
 * back, the next one's inputs are already crossing the (full-duplex) host link.  B crosses
 * the link once.  The result is the same as upload_csr + run + download on one engine
 * (every nonzero is computed by the same kernels; which rows reach the tensor-core tiles is
 * decided per range).  The number of ranges is the host-link traffic (12 bytes per nonzero + A + B)
 * divided by 64 MB, rounded, at most `chunks` (sddmm_b200_pipeline_set_min_chunk_bytes changes the
 * 64 MB), so small inputs run as one range.  One call at a time per pipeline object.  For full overlap the host buffers should be pinned
 * (sddmm_b200_host_alloc); pageable buffers work, with less overlap.
 * Errors: the status codes above; sddmm_b200_pipeline_last_error names the row range. */
typedef struct sddmm_b200_pipeline sddmm_b200_pipeline;
int sddmm_b200_pipeline_create(sddmm_b200_pipeline **out, int device, int mode, uint32_t flags, int chunks /* 1..64 */);
int sddmm_b200_pipeline_destroy(sddmm_b200_pipeline *p);
int sddmm_b200_pipeline_sddmm_csr(sddmm_b200_pipeline *p, int64_t M, int64_t N, int64_t K, const int32_t *row_ptr,
                                  const int32_t *col_idx, const float *s_val, const float *A, const float *B,
                                  float *p_val /* nnz, out */);
/* COO form (Competitor<T>::init_coo / run_coo / cleanup_coo, src/benchmark/competitor.hpp:28-34): rows sorted as COO<T>
 * keeps them (src/matrices/COO.hpp:39), otherwise SDDMM_B200_ERR_INDEX.  The row indices are not rewritten on the host:
 * every range is re-based on the device. */
int sddmm_b200_pipeline_sddmm_coo(sddmm_b200_pipeline *p, int64_t M, int64_t N, int64_t K, int64_t nnz, const int32_t *row_idx,
                                  const int32_t *col_idx, const float *s_val, const float *A, const float *B,
                                  float *p_val /* nnz, out */);
/* The pattern of the last successful sddmm_b200_pipeline_sddmm_csr / _coo call with new S.val, A and B (iterative
 * callers: no counterpart in the reference, which re-uploads everything): only the numbers cross the link,
 * plans are kept, ranges overlap in the same way.  SDDMM_B200_ERR_STATE without such a call. */
int sddmm_b200_pipeline_update_csr(sddmm_b200_pipeline *p, const float *s_val, const float *A, const float *B,
                                   float *p_val /* nnz, out */);
int sddmm_b200_pipeline_last_chunks(sddmm_b200_pipeline *p); /* ranges the last call used */
int sddmm_b200_pipeline_set_min_chunk_bytes(sddmm_b200_pipeline *p, int64_t bytes);
const char *sddmm_b200_pipeline_last_error(sddmm_b200_pipeline *p);

/* ---- several GPUs of one box from one process -----------------------------------------
 * SDDMM shards by rows with no exchange in the compute step; what the devices share is B.
 *
 * sddmm_b200_row_cuts: parts + 1 row indices (cuts[0] = 0, cuts[parts] = M) that give every part an equal share of the
 * nonzeros -- the row boundary closest to g * nnz / parts, moved to a multiple of `align` rows when align > 1 (64 keeps
 * the 64 x 64 tile grid of the tensor-core path in every shard).  The goal of the reference's CSR<T>::_dispatch
 * (src/matrices/CSR.hpp:196-264: equal nonzeros per worker), by one binary search per cut.  Host only.
 * sddmm_b200_coo_cuts does the same from a COO row array sorted by row (no row_ptr is built): cuts[g] is the row and
 * offsets[g] the position in row_idx where part g starts (offsets[parts] = nnz).  SDDMM_B200_ERR_INDEX when the
 * entries it looks at are out of range or not sorted (the upload of every part validates its whole slice).
 *
 * sddmm_b200_stage_b: B crosses the host link ONCE, to engines[0]'s device, and is then copied device to device in
 * log2(n) rounds (every device that holds B serves one that does not; NVLink where the devices are peers).  After it
 * every listed engine accepts B = NULL in its next sddmm_b200_upload_csr / _coo with the same N and K and takes its
 * staged copy.  Engines may sit on the same device.  SDDMM_B200_ERR_COMM when a device-to-device copy fails (the reason
 * is in the engine's last_error); no engine keeps a staged B then.  No reference counterpart (the reference is
 * single-GPU: every competitor uploads B itself, e.g. src/competitors/gpu/gpu_basic.hpp:33-60). */
int sddmm_b200_row_cuts(const int32_t *row_ptr, int64_t M, int parts, int64_t align, int64_t *cuts);
int sddmm_b200_coo_cuts(const int32_t *row_idx, int64_t nnz, int64_t M, int parts, int64_t align, int64_t *cuts,
                        int64_t *offsets);
int sddmm_b200_stage_b(sddmm_b200_engine **engines, int n, int64_t N, int64_t K, const float *B);

/* ---- self-test of the failure path ------------------------------------------------------------
 * Every wait inside the kernels (on an mbarrier fed by a TMA copy or by the tensor cores) gives up after a bounded
 * number of probes, records that in a device error word and lets the kernel return; sync() then reports
 * SDDMM_B200_ERR_DEVICE_WAIT.  This call exercises exactly that path without any fault: a one-thread kernel waits
 * `probes` (1..65536) times on a barrier nothing completes.  Returns SDDMM_B200_ERR_DEVICE_WAIT when the mechanism
 * works (the time-out was seen, recorded and read back), SDDMM_B200_OK if the wait unexpectedly succeeded.  The engine
 * stays usable: the next run() clears the error word.  No reference counterpart (its kernels do not wait on anything). */
int sddmm_b200_selftest_wait_timeout(sddmm_b200_engine *e, int probes);

/* pinned host memory helpers (so callers without a CUDA toolchain can stage
 * inputs for full-rate copies) */
int sddmm_b200_host_alloc(void **ptr, int64_t bytes);
int sddmm_b200_host_free(void *ptr);

#ifdef __cplusplus
}
#endif
#endif /* SDDMM_B200_H */
