// ref_shim.cpp -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// extern "C" doors into the UNMODIFIED reference headers (francois141/dphpc),
// compiled where they lie (-I<reference>/src) by oracle/build.py into
// oracle/_ref/libsddmm_ref.so.  Nothing of the reference is copied here: this
// file only constructs the reference's own Dense/CSR/COO objects from raw
// arrays and calls its CPUBasic competitor and its CSR dispatcher.
//
// Used to (a) validate oracle/sddmm_oracle.c bit for bit, (b) generate the
// fixtures under tests/golden/, (c) time the reference CPU path in bench.py.
#include <cassert>
#include <cmath>
#include <cstdint>
#include <chrono>
#include <vector>

#include "competitors/cpu/cpu_basic.hpp"

namespace {

Dense<float> make_dense(int64_t rows, int64_t cols, const float *data) {
    std::vector<std::vector<float>> v(static_cast<size_t>(rows), std::vector<float>(static_cast<size_t>(cols)));
    for (int64_t i = 0; i < rows; ++i)
        for (int64_t k = 0; k < cols; ++k) v[i][k] = data[i * cols + k];
    return Dense<float>(v);
}

std::vector<Triplet<float>> make_triplets(int64_t n, const int32_t *rows, const int32_t *cols, const float *vals) {
    std::vector<Triplet<float>> t(static_cast<size_t>(n));
    for (int64_t i = 0; i < n; ++i) t[i] = Triplet<float>{rows[i], cols[i], vals[i]};
    return t;
}

}  // namespace

extern "C" {

// CSR<float>(M, N, triplets) -> arrays. Returns nnz kept. row_ptr needs M+1 entries, the others n.
int64_t ref_csr_from_triplets(int32_t M, int32_t N, int64_t n, const int32_t *rows, const int32_t *cols, const float *vals,
                              int32_t *row_ptr, int32_t *col_idx, float *out_vals) {
    CSR<float> S(M, N, make_triplets(n, rows, cols, vals));
    const auto &rp = S.getRowPositions();
    const auto &cp = S.getColPositions();
    const auto &v = S.getValues();
    for (size_t i = 0; i < rp.size(); ++i) row_ptr[i] = rp[i];
    for (size_t i = 0; i < cp.size(); ++i) { col_idx[i] = cp[i]; out_vals[i] = v[i]; }
    return static_cast<int64_t>(v.size());
}

// COO<float>(M, N, triplets) -> arrays. Returns nnz kept.
int64_t ref_coo_from_triplets(int32_t M, int32_t N, int64_t n, const int32_t *rows, const int32_t *cols, const float *vals,
                              int32_t *out_rows, int32_t *out_cols, float *out_vals) {
    COO<float> S(M, N, make_triplets(n, rows, cols, vals));
    const auto &r = S.getRowPositions();
    const auto &c = S.getColPositions();
    const auto &v = S.getValues();
    for (size_t i = 0; i < v.size(); ++i) { out_rows[i] = r[i]; out_cols[i] = c[i]; out_vals[i] = v[i]; }
    return static_cast<int64_t>(v.size());
}

// CPUBasic<float>::run_csr on a CSR given as (sorted, duplicate-free) arrays.
// Returns the wall time of run_csr alone in nanoseconds (std::chrono, the
// reference's own clock for CPU competitors).
int64_t ref_cpu_basic_csr(int32_t M, int32_t N, int32_t K, const int32_t *row_ptr, const int32_t *col_idx, const float *s_val,
                          const float *A, const float *B, float *p_val) {
    const int64_t nnz = row_ptr[M];
    std::vector<Triplet<float>> t(static_cast<size_t>(nnz));
    for (int32_t i = 0; i < M; ++i)
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; ++j) t[j] = Triplet<float>{i, col_idx[j], s_val[j]};
    Dense<float> dA = make_dense(M, K, A), dB = make_dense(N, K, B);
    CSR<float> S(M, N, t);
    if (static_cast<int64_t>(S.getValues().size()) != nnz) return -1;  // input had duplicates the reference drops
    // exact zeros would defeat the reference's dedup rule but never reorder entries; put values back verbatim
    std::vector<float> sv(s_val, s_val + nnz);
    S.setValues(sv);
    CSR<float> P(S);
    P.clearValues();
    Competitors::CPUBasic<float> cpu;
    cpu.init_csr(dA, dB, S, P);
    const auto t0 = std::chrono::high_resolution_clock::now();
    cpu.run_csr(dA, dB, S, P);
    const auto t1 = std::chrono::high_resolution_clock::now();
    cpu.cleanup_csr(dA, dB, S, P);
    for (int64_t j = 0; j < nnz; ++j) p_val[j] = P.getValues()[j];
    return std::chrono::duration_cast<std::chrono::nanoseconds>(t1 - t0).count();
}

int64_t ref_cpu_basic_coo(int32_t M, int32_t N, int32_t K, int64_t nnz, const int32_t *row_idx, const int32_t *col_idx,
                          const float *s_val, const float *A, const float *B, float *p_val) {
    Dense<float> dA = make_dense(M, K, A), dB = make_dense(N, K, B);
    COO<float> S(M, N, make_triplets(nnz, row_idx, col_idx, s_val));
    if (static_cast<int64_t>(S.getValues().size()) != nnz) return -1;
    std::vector<float> sv(s_val, s_val + nnz);
    S.setValues(sv);
    COO<float> P(S);
    P.clearValues();
    Competitors::CPUBasic<float> cpu;
    const auto t0 = std::chrono::high_resolution_clock::now();
    cpu.run_coo(dA, dB, S, P);
    const auto t1 = std::chrono::high_resolution_clock::now();
    for (int64_t j = 0; j < nnz; ++j) p_val[j] = P.getValues()[j];
    return std::chrono::duration_cast<std::chrono::nanoseconds>(t1 - t0).count();
}

// CSR<float>::computeDispatcher / computeDispatcherTensorCores -> start_idx. Returns its length.
int64_t ref_dispatch(int32_t M, int32_t N, const int32_t *row_ptr, const int32_t *col_idx, int32_t parts, int32_t tensor,
                     int32_t *out_start, int64_t out_cap) {
    const int64_t nnz = row_ptr[M];
    std::vector<Triplet<float>> t(static_cast<size_t>(nnz));
    for (int32_t i = 0; i < M; ++i)
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; ++j) t[j] = Triplet<float>{i, col_idx[j], 1.0f};
    CSR<float> S(M, N, t);
    if (tensor) S.computeDispatcherTensorCores(parts); else S.computeDispatcher(parts);
    const auto &s = S.getStartIdx();
    for (size_t i = 0; i < s.size() && static_cast<int64_t>(i) < out_cap; ++i) out_start[i] = s[i];
    return static_cast<int64_t>(s.size());
}

// Persistent problem for repeated timing (bench.py --impl reference): the
// reference objects are built once, every run() is one CPUBasic::run_csr.
struct ref_problem {
    Dense<float> A, B;
    CSR<float> S, P;
    Competitors::CPUBasic<float> cpu;
};

void *ref_problem_create(int32_t M, int32_t N, int32_t K, const int32_t *row_ptr, const int32_t *col_idx, const float *s_val,
                         const float *A, const float *B) {
    const int64_t nnz = row_ptr[M];
    std::vector<Triplet<float>> t(static_cast<size_t>(nnz));
    for (int32_t i = 0; i < M; ++i)
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; ++j) t[j] = Triplet<float>{i, col_idx[j], s_val[j]};
    ref_problem *p = new ref_problem{make_dense(M, K, A), make_dense(N, K, B), CSR<float>(M, N, t), CSR<float>(), {}};
    if (static_cast<int64_t>(p->S.getValues().size()) != nnz) { delete p; return nullptr; }
    p->S.setValues(std::vector<float>(s_val, s_val + nnz));
    p->P = CSR<float>(p->S);
    p->P.clearValues();
    return p;
}

int64_t ref_problem_run(void *h) {
    ref_problem *p = static_cast<ref_problem *>(h);
    const auto t0 = std::chrono::high_resolution_clock::now();
    p->cpu.run_csr(p->A, p->B, p->S, p->P);
    const auto t1 = std::chrono::high_resolution_clock::now();
    return std::chrono::duration_cast<std::chrono::nanoseconds>(t1 - t0).count();
}

void ref_problem_result(void *h, float *p_val) {
    ref_problem *p = static_cast<ref_problem *>(h);
    const auto &v = p->P.getValues();
    for (size_t j = 0; j < v.size(); ++j) p_val[j] = v[j];
}

void ref_problem_destroy(void *h) { delete static_cast<ref_problem *>(h); }

// the reference's operator== on CSR<float> (pattern equal, values by its 1e-3 rule)
int ref_csr_equal(int32_t M, int32_t N, const int32_t *row_ptr, const int32_t *col_idx, const float *lhs, const float *rhs) {
    const int64_t nnz = row_ptr[M];
    std::vector<Triplet<float>> t(static_cast<size_t>(nnz));
    for (int32_t i = 0; i < M; ++i)
        for (int32_t j = row_ptr[i]; j < row_ptr[i + 1]; ++j) t[j] = Triplet<float>{i, col_idx[j], 1.0f};
    CSR<float> L(M, N, t), R(M, N, t);
    L.setValues(std::vector<float>(lhs, lhs + nnz));
    R.setValues(std::vector<float>(rhs, rhs + nnz));
    return (L == R) ? 1 : 0;
}

}  // extern "C"
