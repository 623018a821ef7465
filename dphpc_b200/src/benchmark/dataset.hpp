// Inputs of one benchmark: A, B, S in CSR and COO form, and optionally the expected P.
// Dataset<T> keeps the public getters of the reference's SDDMM::Dataset<T>
// (src/benchmark/dataset.hpp:79-119).  SyntheticDataset wraps the seeded generators of
// include/sddmm_datasets.h (the reference's RandomWithDensityDataset, :331-356, is unseeded);
// DummyDataset is the reference's built-in known-answer case (:183-204).
#pragma once
#include <stdexcept>
#include <string>
#include <vector>

#include "matrices/matrices.h"
#include "sddmm_datasets.h"

namespace SDDMM {

template <typename T>
class Dataset {
public:
    Dataset(const std::string &name, Dense<T> A, Dense<T> B, CSR<T> S) : name_(name), A_(std::move(A)), B_(std::move(B)), S_csr_(std::move(S)), S_coo_(S_csr_) {}
    virtual ~Dataset() = default;

    const std::string getName() { return name_; }
    Dense<T> &getA() { return A_; }
    Dense<T> &getB() { return B_; }
    CSR<T> &getS_CSR() { return S_csr_; }
    COO<T> &getS_COO() { return S_coo_; }

    bool hasExpected() { return P_csr_.getRows() > 0 && P_coo_.getRows() > 0; }
    CSR<T> &getExpected_CSR() { return P_csr_; }
    COO<T> &getExpected_COO() { return P_coo_; }
    void setExpected_CSR(CSR<T> &P) { P_csr_ = P; P_coo_ = COO<T>(P); }
    void setExpected_COO(COO<T> &P) { P_coo_ = P; P_csr_ = CSR<T>(P); }

protected:
    std::string name_;
    Dense<T> A_, B_;
    CSR<T> S_csr_;
    COO<T> S_coo_;
    CSR<T> P_csr_;
    COO<T> P_coo_;
};

// A = B = ones(2x2), S = ones(2x2)  ->  P = 2 everywhere
class DummyDataset : public Dataset<float> {
public:
    DummyDataset() : Dataset<float>("Dummy", ones(), ones(), full(1.0f)) {
        CSR<float> P = full(2.0f);
        setExpected_CSR(P);
    }

private:
    static Dense<float> ones() { return Dense<float>(2, 2, std::vector<float>(4, 1.0f)); }
    static CSR<float> full(float v) { return CSR<float>(2, 2, {0, 2, 4}, {0, 1, 0, 1}, std::vector<float>(4, v)); }
};

// one of the five seeded configurations (or a uniform pattern) from libsddmm_datasets
class SyntheticDataset : public Dataset<float> {
public:
    SyntheticDataset(int config, int K, double scale = 1.0, uint64_t seed = 0, int variant = 0)
        : Dataset<float>(make(config, K, scale, seed ? seed : 0x5DD0 + static_cast<uint64_t>(config), variant)) {}

    static SyntheticDataset uniform(int M, int N, int K, int64_t nnz, uint64_t seed) {
        sddmm_dataset *ds = nullptr;
        if (sddmm_dataset_create_uniform(&ds, M, N, K, nnz, seed) != 0) throw std::runtime_error("dataset generation failed");
        return SyntheticDataset(adopt(ds));
    }

private:
    explicit SyntheticDataset(Dataset<float> base) : Dataset<float>(std::move(base)) {}

    static Dataset<float> make(int config, int K, double scale, uint64_t seed, int variant) {
        sddmm_dataset *ds = nullptr;
        if (sddmm_dataset_create(&ds, config, K, scale, seed, variant) != 0) throw std::runtime_error("dataset generation failed");
        return adopt(ds);
    }

    static Dataset<float> adopt(sddmm_dataset *ds) {
        int64_t M, N, K, nnz;
        sddmm_dataset_dims(ds, &M, &N, &K, &nnz);
        const float *a = sddmm_dataset_A(ds), *b = sddmm_dataset_B(ds), *v = sddmm_dataset_s_val(ds);
        const int32_t *rp = sddmm_dataset_row_ptr(ds), *ci = sddmm_dataset_col_idx(ds);
        Dataset<float> out(sddmm_dataset_name(ds), Dense<float>(static_cast<unsigned>(M), static_cast<unsigned>(K), std::vector<float>(a, a + M * K)),
                           Dense<float>(static_cast<unsigned>(N), static_cast<unsigned>(K), std::vector<float>(b, b + N * K)),
                           CSR<float>(static_cast<int>(M), static_cast<int>(N), std::vector<int>(rp, rp + M + 1), std::vector<int>(ci, ci + nnz),
                                      std::vector<float>(v, v + nnz)));
        sddmm_dataset_destroy(ds);
        return out;
    }
};

}  // namespace SDDMM
