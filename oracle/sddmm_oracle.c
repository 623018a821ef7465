/*
 * sddmm_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the CPU algorithms of francois141/dphpc that define
 * "the right answer" for the SDDMM path.  Only tests/, __graft_entry__.smoke()
 * and bench.py's cpu_baseline / --impl reference legs may load this library, and
 * only as the checker or as the timed CPU baseline.  The CUDA engine never
 * calls it.
 *
 * Parity of this restatement is pinned two ways (see tests/test_oracle.py):
 *   - against the reference's own golden vectors (dispatcher start indices,
 *     DummyDataset, format-conversion identities of tests/matrix_test.cc);
 *   - bit for bit against oracle/_ref/libsddmm_ref.so, the reference's own
 *     headers compiled unmodified, whenever that library has been built, and
 *     against fixtures generated from it (tests/golden/).
 *
 * Build: gcc -O2 -ffp-contract=off (no FMA contraction: the reference's
 * Release build multiplies, then adds, in fp32).
 * Paths below are relative to the reference project's root.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* CPUBasic<T>::run_csr, src/competitors/cpu/cpu_basic.hpp:18-36.
 * Pass 1: P[j] = sum_k A[i,k] * B[col[j],k], accumulated in fp32 in k order
 * through the output element; pass 2: P[j] *= S[j]. */
void oracle_sddmm_csr(int32_t M, int32_t K, const int32_t *row_ptr, const int32_t *col_idx, const float *s_val,
                      const float *A, const float *B, float *p_val) {
    for (int32_t i = 0; i < M; i++) {
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; j++) {
            const float *a = A + (size_t)i * K;
            const float *b = B + (size_t)col_idx[j] * K;
            float acc = 0.0f;
            for (int32_t k = 0; k < K; k++) acc += a[k] * b[k]; /* fp32 mul, then fp32 add, in k order */
            p_val[j] = acc;
        }
    }
    for (int32_t i = 0; i < M; i++)
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; j++) p_val[j] *= s_val[j];
}

/* CPUBasic<T>::run_coo, src/competitors/cpu/cpu_basic.hpp:38-51 */
void oracle_sddmm_coo(int64_t nnz, int32_t K, const int32_t *row_idx, const int32_t *col_idx, const float *s_val,
                      const float *A, const float *B, float *p_val) {
    for (int64_t i = 0; i < nnz; i++) {
        const float *a = A + (size_t)row_idx[i] * K;
        const float *b = B + (size_t)col_idx[i] * K;
        float acc = 0.0f;
        for (int32_t k = 0; k < K; k++) acc += a[k] * b[k];
        p_val[i] = acc;
    }
    for (int64_t i = 0; i < nnz; i++) p_val[i] *= s_val[i];
}

/* Same loops, rows [row_begin, row_end) only: the bounded sample bench.py times. */
void oracle_sddmm_csr_rows(int32_t row_begin, int32_t row_end, int32_t K, const int32_t *row_ptr, const int32_t *col_idx,
                           const float *s_val, const float *A, const float *B, float *p_val) {
    for (int32_t i = row_begin; i < row_end; i++) {
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; j++) {
            const float *a = A + (size_t)i * K;
            const float *b = B + (size_t)col_idx[j] * K;
            float acc = 0.0f;
            for (int32_t k = 0; k < K; k++) acc += a[k] * b[k];
            p_val[j] = acc;
        }
    }
    for (int32_t i = row_begin; i < row_end; i++)
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; j++) p_val[j] *= s_val[j];
}

/* ---- triplets -> CSR / COO ------------------------------------------------
 * CSR<T>::init_csr (src/matrices/CSR.hpp:169-194) and the COO<T> constructor
 * (src/matrices/COO.hpp:27-49): sort by (row, col) with operator< of
 * src/matrices/triplet.h:16-19, then std::unique with operator== of
 * triplet.h:11-14 -- which treats two neighbours as equal only when row and col
 * match AND both values are non-zero -- then emit; CSR keeps empty rows. */
typedef struct { int32_t row, col; float val; int64_t seq; } trip_t;

static int trip_cmp(const void *x, const void *y) {
    const trip_t *a = (const trip_t *)x, *b = (const trip_t *)y;
    if (a->row != b->row) return a->row < b->row ? -1 : 1;
    if (a->col != b->col) return a->col < b->col ? -1 : 1;
    /* std::sort is not stable; ties are only distinguishable by value, and the
     * generators used with this oracle never emit duplicate positions with
     * different values.  Input order is kept to make the result deterministic. */
    return a->seq < b->seq ? -1 : (a->seq > b->seq ? 1 : 0);
}

/* returns the number of entries kept; out arrays need room for n entries */
int64_t oracle_sort_unique_triplets(int64_t n, const int32_t *rows, const int32_t *cols, const float *vals,
                                    int32_t *out_rows, int32_t *out_cols, float *out_vals) {
    trip_t *t = (trip_t *)malloc((size_t)(n > 0 ? n : 1) * sizeof(trip_t));
    if (!t) return -1;
    for (int64_t i = 0; i < n; i++) { t[i].row = rows[i]; t[i].col = cols[i]; t[i].val = vals[i]; t[i].seq = i; }
    qsort(t, (size_t)n, sizeof(trip_t), trip_cmp);
    int64_t m = 0;
    for (int64_t i = 0; i < n; i++) {
        if (m > 0) {
            const trip_t *p = &t[m - 1];
            const int same = p->row == t[i].row && p->col == t[i].col && p->val != 0.0f && t[i].val != 0.0f;
            if (same) continue; /* std::unique keeps the first of a run */
        }
        t[m++] = t[i];
    }
    for (int64_t i = 0; i < m; i++) { out_rows[i] = t[i].row; out_cols[i] = t[i].col; out_vals[i] = t[i].val; }
    free(t);
    return m;
}

/* sorted COO rows -> row_ptr with empty rows kept (CSR.hpp:183-193) */
void oracle_coo_rows_to_row_ptr(int32_t M, int64_t nnz, const int32_t *rows, int32_t *row_ptr) {
    int64_t idx = 0;
    for (int32_t i = 0; i < M; i++) {
        row_ptr[i] = (int32_t)idx;
        while (idx < nnz && rows[idx] == i) idx++;
    }
    row_ptr[M] = (int32_t)idx;
}

/* COO<T>(CSR<T>&), src/matrices/COO.hpp:55-74 */
void oracle_row_ptr_to_coo_rows(int32_t M, const int32_t *row_ptr, int32_t *rows) {
    for (int32_t i = 0; i < M; i++)
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; j++) rows[j] = i;
}

/* ---- nnz-balanced row dispatcher ---------------------------------------------
 * CSR<T>::testValue / _dispatch, src/matrices/CSR.hpp:196-264: sizes are the
 * nnz of `stride` consecutive rows; binary search the smallest segment capacity
 * for which a greedy left-to-right cut needs <= parts segments; cut greedily;
 * pad start_idx with `rows` up to parts+1 entries.
 * out_start needs max(parts, nsizes) + 1 entries.  Returns the entry count. */
static int fits(const int32_t *sizes, int64_t n, int64_t cap, int64_t parts) {
    int64_t mx = 0;
    for (int64_t i = 0; i < n; i++) if (sizes[i] > mx) mx = sizes[i];
    if (mx > cap) return 0;
    int64_t cnt = 1, sum = 0;
    for (int64_t i = 0; i < n; i++) {
        sum += sizes[i];
        if (sum > cap) { cnt++; sum = sizes[i]; }
    }
    return cnt <= parts;
}

int64_t oracle_dispatch(int32_t M, const int32_t *row_ptr, int32_t parts, int32_t stride, int32_t *out_start) {
    const int64_t nnz = row_ptr[M];
    int64_t n = 0;
    int32_t *sizes = (int32_t *)malloc((size_t)(M / stride + 2) * sizeof(int32_t));
    if (!sizes) return -1;
    for (int32_t i = 0; i < M; i += stride) {
        const int32_t hi = i + stride; /* the reference reads row_ptr[i+stride]; callers keep M % stride == 0 */
        sizes[n++] = row_ptr[hi <= M ? hi : M] - row_ptr[i];
    }
    int64_t lo = 1, hi = nnz, seg = 0;
    while (lo <= hi) {
        const int64_t mid = (lo + hi) / 2;
        if (fits(sizes, n, mid, parts)) { seg = mid; hi = mid - 1; } else { lo = mid + 1; }
    }
    int64_t cnt = 0, cur = 0;
    out_start[cnt++] = 0;
    for (int64_t i = 0; i < n; i++) {
        cur += sizes[i];
        if (cur > seg) { out_start[cnt++] = (int32_t)(i * stride); cur = sizes[i]; }
    }
    while (cnt <= parts) out_start[cnt++] = M;
    free(sizes);
    return cnt;
}

/* operator== of CSR<T>/COO<T> on float values (src/matrices/CSR.hpp:86-96):
 * one-sided, signed: |rhs - lhs| / rhs <= 1e-3 for every entry. */
int oracle_values_equal_reference_rule(int64_t n, const float *lhs, const float *rhs) {
    int ok = 1;
    for (int64_t i = 0; i < n; i++) {
        float d = rhs[i] - lhs[i];
        if (d < 0) d = -d;
        const float diff = d / rhs[i];
        ok &= ((double)diff <= 1e-3);
    }
    return ok;
}

/* ---- the consumer of P: Y = P X (CSR SpMM) --------------------------------
 * No counterpart in the reference's sources (its report names SpMM / ALS-style consumers of the SDDMM result as the
 * motivation, but ships none): a plain row-by-row loop, y_i = sum_j p_ij * x_col(j), fp32, in CSR order.  Used to check
 * the engine's device-side consumer; rows [row_begin, row_end). */
void oracle_spmm_csr_rows(int32_t row_begin, int32_t row_end, int32_t K2, const int32_t *row_ptr, const int32_t *col_idx,
                          const float *p_val, const float *X, float *Y) {
    for (int32_t i = row_begin; i < row_end; i++) {
        float *y = Y + (size_t)i * K2;
        for (int32_t k = 0; k < K2; k++) y[k] = 0.0f;
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; j++) {
            const float *x = X + (size_t)col_idx[j] * K2;
            const float p = p_val[j];
            for (int32_t k = 0; k < K2; k++) y[k] += p * x[k];
        }
    }
}
