// CPU-Basic: the correctness baseline of the benchmark driver, registered FIRST so that every GPU row's
// `correctness` column is a comparison with an independent host computation (the reference's driver does the same:
// src/main.cpp:18-20 registers CPU-Basic first, src/benchmark/benchmark.hpp:50-61 takes competitors[0] as the
// expected result).  Same arithmetic as the reference's CPUBasic (src/competitors/cpu/cpu_basic.hpp:18-51): per
// nonzero a sequential fp32 sum over k, then one multiplication by S's value -- so the values are the reference's
// bit for bit -- but the rows (CSR) or entries (COO) are spread over the host threads, one writer per nonzero.
// This is a comparator, not a fallback: no GPU competitor ever routes through it.
#pragma once
#include <algorithm>
#include <cstdint>
#include <thread>
#include <vector>

#include "benchmark/competitor.hpp"
#include "matrices/matrices.h"

namespace Competitors {

class CPUCheck : public SDDMM::Competitor<float> {
public:
    explicit CPUCheck(unsigned threads = 0) : SDDMM::Competitor<float>("CPU-Basic"), threads_(threads) {}

    void run_csr(Dense<float> &A, Dense<float> &B, CSR<float> &S, CSR<float> &P) override {
        const int64_t M = S.getRows(), K = A.getCols();
        const int *rp = S.getRowPositions().data(), *col = S.getColPositions().data();
        const float *sv = S.getValues().data(), *a = A.get_pointer(), *b = B.get_pointer();
        if (P.getValues().size() != S.getValues().size()) P.setValues(S.getValues());
        float *out = P.getValues().data();
        const int64_t nnz = rp[M];
        parallel(M, nnz, [=](int64_t part, int64_t parts) {
            // rows whose first nonzero falls into this part's share of the nonzeros
            const int64_t lo = nnz * part / parts, hi = nnz * (part + 1) / parts;
            int64_t r0 = std::lower_bound(rp, rp + M, lo) - rp, r1 = std::lower_bound(rp, rp + M, hi) - rp;
            if (part == 0) r0 = 0;
            if (part == parts - 1) r1 = M;
            for (int64_t i = r0; i < r1; ++i)
                for (int64_t j = rp[i]; j < rp[i + 1]; ++j) out[j] = one(a + i * K, b + static_cast<int64_t>(col[j]) * K, K) * sv[j];
        });
    }

    void run_coo(Dense<float> &A, Dense<float> &B, COO<float> &S, COO<float> &P) override {
        const int64_t K = A.getCols(), nnz = static_cast<int64_t>(S.getValues().size());
        const int *row = S.getRowPositions().data(), *col = S.getColPositions().data();
        const float *sv = S.getValues().data(), *a = A.get_pointer(), *b = B.get_pointer();
        if (P.getValues().size() != S.getValues().size()) P.setValues(S.getValues());
        float *out = P.getValues().data();
        parallel(nnz, nnz, [=](int64_t part, int64_t parts) {
            for (int64_t j = nnz * part / parts; j < nnz * (part + 1) / parts; ++j)
                out[j] = one(a + static_cast<int64_t>(row[j]) * K, b + static_cast<int64_t>(col[j]) * K, K) * sv[j];
        });
    }

    bool csr_supported() override { return true; }
    bool coo_supported() override { return true; }

private:
    unsigned threads_;

    static float one(const float *x, const float *y, int64_t K) {
        float acc = 0.0f;
        for (int64_t k = 0; k < K; ++k) acc += x[k] * y[k];   // (built without FMA contraction: see the build recipe)
        return acc;
    }

    template <typename F>
    void parallel(int64_t units, int64_t work, F fn) {
        unsigned n = threads_ ? threads_ : std::max(1u, std::min(std::thread::hardware_concurrency(), 64u));
        if (work < (1 << 16) || units < 2) n = 1;
        if (n == 1) {
            fn(0, 1);
            return;
        }
        std::vector<std::thread> pool;
        for (unsigned t = 0; t < n; ++t) pool.emplace_back(fn, static_cast<int64_t>(t), static_cast<int64_t>(n));
        for (auto &t : pool) t.join();
    }
};

}  // namespace Competitors
