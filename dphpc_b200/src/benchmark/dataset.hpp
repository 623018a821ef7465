// Inputs of one benchmark: A, B, S in CSR and COO form, and optionally the expected P.
// Dataset<T> keeps the public getters of the reference's SDDMM::Dataset<T>
// (src/benchmark/dataset.hpp:79-119).  SyntheticDataset wraps the seeded generators of
// include/sddmm_datasets.h (the reference's RandomWithDensityDataset, :331-356, is unseeded);
// DummyDataset is the reference's built-in known-answer case (:183-204).  MatrixMarketDataset and
// EdgeListDataset read the two file formats the reference loads (:122-181 and :270-313) with its
// semantics: 1-based MatrixMarket coordinates, no mirroring of symmetric files, entries with
// |value| < 1e-7 dropped; SNAP edge lists take the ids as they are and the value 1.  Unlike the
// reference they fill A and B from a seed, accept pattern files, and report bad input by exception
// instead of assert.
#pragma once
#include <cmath>
#include <cstdint>
#include <fstream>
#include <sstream>
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

// A and B for inputs that come without dense operands: uniform [-1, 1), reproducible from the seed
inline Dense<float> seeded_dense(unsigned rows, unsigned cols, uint64_t seed) {
    std::vector<float> v(static_cast<size_t>(rows) * cols);
    uint64_t x = seed;
    for (float &f : v) {
        x += 0x9E3779B97F4A7C15ull;   // splitmix64 step
        uint64_t z = x;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        f = static_cast<float>(static_cast<double>(z >> 40) * (2.0 / 16777216.0) - 1.0);
    }
    return Dense<float>(rows, cols, std::move(v));
}

// MatrixMarket coordinate file (https://math.nist.gov/MatrixMarket/formats.html), real, integer or pattern.
class MatrixMarketDataset : public Dataset<float> {
public:
    MatrixMarketDataset(const std::string &name, const std::string &path, int K, uint64_t seed = 0x5DD0)
        : Dataset<float>(load(name, path, K, seed)) {}

private:
    static Dataset<float> load(const std::string &name, const std::string &path, int K, uint64_t seed) {
        std::ifstream in(path);
        if (!in) throw std::runtime_error("cannot open " + path);
        std::string line;
        bool pattern = false;
        long long M = -1, N = -1, declared = -1;
        while (std::getline(in, line)) {
            if (line.empty()) continue;
            if (line[0] == '%') {
                if (line.rfind("%%MatrixMarket", 0) == 0 && line.find("pattern") != std::string::npos) pattern = true;
                continue;
            }
            std::istringstream size_line(line);
            if (!(size_line >> M >> N >> declared) || M < 1 || N < 1 || declared < 0) throw std::runtime_error("bad size line in " + path);
            break;
        }
        if (M < 0) throw std::runtime_error("no size line in " + path);
        std::vector<Triplet<float>> triplets;
        triplets.reserve(static_cast<size_t>(declared));
        long long seen = 0;
        while (std::getline(in, line)) {
            if (line.empty() || line[0] == '%') continue;
            std::istringstream entry(line);
            long long r, c;
            double v = 1.0;
            if (!(entry >> r >> c) || (!pattern && !(entry >> v))) throw std::runtime_error("bad entry in " + path + ": " + line);
            if (r < 1 || r > M || c < 1 || c > N) throw std::runtime_error("coordinate out of range in " + path + ": " + line);
            ++seen;
            if (std::fabs(v) < 1e-7) continue;   // the reference drops (numerically) zero entries
            triplets.push_back({static_cast<int>(r - 1), static_cast<int>(c - 1), static_cast<float>(v)});
        }
        if (seen != declared) throw std::runtime_error(path + ": " + std::to_string(seen) + " entries, size line says " + std::to_string(declared));
        return Dataset<float>(name, seeded_dense(static_cast<unsigned>(M), static_cast<unsigned>(K), seed),
                              seeded_dense(static_cast<unsigned>(N), static_cast<unsigned>(K), seed + 1),
                              CSR<float>(static_cast<int>(M), static_cast<int>(N), triplets));
    }
};

// SNAP-style edge list: '#' comment lines, then "row<TAB or space>col" pairs used as they are (0-based), value 1.
class EdgeListDataset : public Dataset<float> {
public:
    EdgeListDataset(const std::string &name, const std::string &path, int M, int N, int K, uint64_t seed = 0x5DD0)
        : Dataset<float>(load(name, path, M, N, K, seed)) {}

private:
    static Dataset<float> load(const std::string &name, const std::string &path, int M, int N, int K, uint64_t seed) {
        std::ifstream in(path);
        if (!in) throw std::runtime_error("cannot open " + path);
        std::vector<Triplet<float>> triplets;
        std::string line;
        while (std::getline(in, line)) {
            if (line.empty() || line[0] == '#') continue;
            std::istringstream entry(line);
            long long r, c;
            if (!(entry >> r >> c)) throw std::runtime_error("bad edge in " + path + ": " + line);
            if (r < 0 || r >= M || c < 0 || c >= N) throw std::runtime_error("edge out of range in " + path + ": " + line);
            triplets.push_back({static_cast<int>(r), static_cast<int>(c), 1.0f});
        }
        return Dataset<float>(name, seeded_dense(static_cast<unsigned>(M), static_cast<unsigned>(K), seed),
                              seeded_dense(static_cast<unsigned>(N), static_cast<unsigned>(K), seed + 1), CSR<float>(M, N, triplets));
    }
};

}  // namespace SDDMM
