// GPU-B200 behind the competitor interface, checked like the reference checks its competitors
// (tests/matrix_test.cc:40-82: run init/run/cleanup into a P that still holds S's values, compare with
// CPU-Basic).  CPU-Basic here is the C oracle (oracle/sddmm_oracle.c), linked into this test binary only.
// Cases: sddmm_coo1..4 (:124-182), random suites (:184-246), DummyDataset, csr-vs-coo agreement, and
// reuse of one competitor object across datasets (the harness does that, src/benchmark/benchmark.hpp:64-137).
#include <algorithm>
#include <cmath>
#include <memory>

#include "benchmark/benchmark.hpp"
#include "check.hpp"
#include "competitors/cpu/cpu_check.hpp"
#include "competitors/gpu/gpu_b200.hpp"
#include "competitors/gpu/gpu_b200_multi.hpp"

extern "C" {
void oracle_sddmm_csr(int32_t M, int32_t K, const int32_t *row_ptr, const int32_t *col_idx, const float *s_val, const float *A,
                      const float *B, float *p_val);
void oracle_sddmm_coo(int64_t nnz, int32_t K, const int32_t *row_idx, const int32_t *col_idx, const float *s_val, const float *A,
                      const float *B, float *p_val);
}

namespace {

// the oracle dressed as a competitor, so the harness and the helpers below can use it as "competitors[0]"
class CPUOracle : public SDDMM::Competitor<float> {
public:
    CPUOracle() : SDDMM::Competitor<float>("CPU-Basic(oracle)") {}
    void run_csr(Dense<float> &A, Dense<float> &B, CSR<float> &S, CSR<float> &P) override {
        P.setValues(S.getValues());
        oracle_sddmm_csr(S.getRows(), static_cast<int>(A.getCols()), S.getRowPositions().data(), S.getColPositions().data(),
                         S.getValues().data(), A.get_pointer(), B.get_pointer(), P.getValues().data());
    }
    void run_coo(Dense<float> &A, Dense<float> &B, COO<float> &S, COO<float> &P) override {
        P.setValues(S.getValues());
        oracle_sddmm_coo(static_cast<int64_t>(S.getValues().size()), static_cast<int>(A.getCols()), S.getRowPositions().data(),
                         S.getColPositions().data(), S.getValues().data(), A.get_pointer(), B.get_pointer(), P.getValues().data());
    }
    bool csr_supported() override { return true; }
    bool coo_supported() override { return true; }
};

std::vector<std::shared_ptr<SDDMM::Competitor<float>>> &competitors() {
    static std::vector<std::shared_ptr<SDDMM::Competitor<float>>> c{
        std::make_shared<CPUOracle>(), std::make_shared<Competitors::GPUB200>(SDDMM_B200_FP32, 0, "GPU-B200"),
        std::make_shared<Competitors::GPUB200>(SDDMM_B200_FP32_TC, 0, "GPU-B200-fp32_tc"),
        // row shards over several engines: every visible device; two and three engines on device 0 (the sharding
        // logic is the same, so it is also covered on a single-GPU machine)
        std::make_shared<Competitors::GPUB200Multi>(std::vector<int>{}, SDDMM_B200_FP32, "GPU-B200-all"),
        std::make_shared<Competitors::GPUB200Multi>(std::vector<int>{0, 0}, SDDMM_B200_FP32, "GPU-B200-2shards"),
        std::make_shared<Competitors::GPUB200Multi>(std::vector<int>{0, 0, 0}, SDDMM_B200_FP32_TC, "GPU-B200-3shards-fp32_tc")};
    return c;
}

// |p - ref| <= tol * |s| * sum_k |a b|  (relative error that survives cancellation)
template <typename Sparse>
bool close_enough(Dense<float> &A, Dense<float> &B, Sparse &S, const std::vector<int> &rows, Sparse &P, Sparse &ref, double tol) {
    const int K = static_cast<int>(A.getCols());
    for (size_t j = 0; j < ref.getValues().size(); ++j) {
        double bound = 0;
        for (int k = 0; k < K; ++k) bound += std::fabs(double(A.getValue(rows[j], k)) * double(B.getValue(S.getColPositions()[j], k)));
        bound *= std::fabs(double(S.getValues()[j]));
        if (std::fabs(double(P.getValues()[j]) - double(ref.getValues()[j])) > tol * bound + 1e-30) return false;
    }
    return true;
}

COO<float> all_competitors_coo(Dense<float> &A, Dense<float> &B, COO<float> &S) {
    COO<float> P1(S), P2(S);  // P2 starts with S's values and is reused, as in the reference helper
    competitors()[0]->run_coo(A, B, S, P1);
    for (auto &c : competitors()) {
        c->init_coo(A, B, S, P2);
        c->run_coo(A, B, S, P2);
        c->cleanup_coo(A, B, S, P2);
        CHECK(P1.getRowPositions() == P2.getRowPositions() && P1.getColPositions() == P2.getColPositions());
        CHECK(close_enough(A, B, S, S.getRowPositions(), P2, P1, 1e-5));
    }
    return P1;
}

CSR<float> all_competitors_csr(Dense<float> &A, Dense<float> &B, CSR<float> &S) {
    CSR<float> P1(S), P2(S);
    competitors()[0]->run_csr(A, B, S, P1);
    COO<float> coo(S);
    for (auto &c : competitors()) {
        c->init_csr(A, B, S, P2);
        c->run_csr(A, B, S, P2);
        c->cleanup_csr(A, B, S, P2);
        CHECK(P1.getRowPositions() == P2.getRowPositions() && P1.getColPositions() == P2.getColPositions());
        CHECK(close_enough(A, B, S, coo.getRowPositions(), P2, P1, 1e-5));
    }
    return P1;
}

Dense<float> dense(std::vector<std::vector<float>> v) { return Dense<float>(v); }

}  // namespace

TEST_CASE(sddmm_coo1) {
    auto A = dense({{1, 2}, {3, 4}}), B = dense({{-1, 2}, {-3, 4}});
    COO<float> S(2, 2, {{0, 0, 1.0f}, {0, 1, 1.0f}, {1, 0, 1.0f}, {1, 1, 1.0f}});
    CHECK_EQ(all_competitors_coo(A, B, S).getValues(), (std::vector<float>{3, 5, 5, 7}));
}
TEST_CASE(sddmm_coo2) {
    auto A = dense({{1, 2, 3}, {4, 5, 6}}), B = dense({{-1, -3, 5}, {2, 4, -6}});
    COO<float> S(2, 2, {{0, 0, 1.0f}, {1, 0, 1.0f}, {1, 1, 1.0f}});
    CHECK_EQ(all_competitors_coo(A, B, S).getValues(), (std::vector<float>{8, 11, -8}));
}
TEST_CASE(sddmm_coo3) {
    auto A = dense({{1, 2, 3}, {4, 5, 6}}), B = dense({{-1, -3, 5}});
    COO<float> S(2, 2, {{0, 0, 1.0f}, {1, 0, -1.0f}});
    CHECK_EQ(all_competitors_coo(A, B, S).getValues(), (std::vector<float>{8, -11}));
}
TEST_CASE(sddmm_coo4) {
    auto A = dense({{1, 2}, {3, 4}, {5, 6}}), B = dense({{-1, -3}, {2, 2}, {3, 1}});
    COO<float> S(3, 3, {{0, 0, 1.0f}, {1, 0, -1.0f}, {2, 0, 1.0f}, {2, 2, 1.0f}});
    CHECK_EQ(all_competitors_coo(A, B, S).getValues(), (std::vector<float>{-7, 15, -23, 21}));
}
TEST_CASE(sddmm_random_coo) {
    auto d = SDDMM::SyntheticDataset::uniform(500, 500, 32, 75000, 1);
    all_competitors_coo(d.getA(), d.getB(), d.getS_COO());
}
TEST_CASE(sddmm_random_dense_coo) {
    auto d = SDDMM::SyntheticDataset::uniform(250, 250, 32, 43750, 2);
    all_competitors_coo(d.getA(), d.getB(), d.getS_COO());
}
TEST_CASE(sddmm_random_sparse_coo) {
    auto d = SDDMM::SyntheticDataset::uniform(10000, 10000, 32, 100000, 3);
    all_competitors_coo(d.getA(), d.getB(), d.getS_COO());
}
TEST_CASE(sddmm_csr_coo) {
    auto d = SDDMM::SyntheticDataset::uniform(500, 500, 32, 75000, 4);
    CSR<float> p_csr = all_competitors_csr(d.getA(), d.getB(), d.getS_CSR());
    COO<float> p_coo = all_competitors_coo(d.getA(), d.getB(), d.getS_COO());
    CHECK(p_coo == COO<float>(p_csr));
}
TEST_CASE(harness_dummy_and_synthetic) {
    SDDMM::DummyDataset dummy;
    SDDMM::Benchmark<float> b1(dummy, competitors(), 1);
    CHECK_EQ(b1.benchmark(), 0);   // expected P = 2.0 comes with the dataset
    SDDMM::SyntheticDataset blocks(2, 32, 0.08);
    SDDMM::Benchmark<float> b2(blocks, competitors(), 2);   // expected P from competitors[0] = the oracle
    CHECK_EQ(b2.benchmark(), 0);
    SDDMM::SyntheticDataset power(4, 32, 0.004);
    SDDMM::Benchmark<float> b3(power, competitors(), 1);
    CHECK_EQ(b3.benchmark(), 0);
}
TEST_CASE(row_cuts_balance_nonzeros) {
    // 6 rows with 0, 10, 0, 10, 30, 10 nonzeros: halves cut after row 4 would be 20 | 40, after row 5 50 | 10 -> the closer
    // boundary to 30 is row_ptr = 20 (cut at row 4)
    const std::vector<int> rp{0, 0, 10, 10, 20, 50, 60};
    CHECK(Competitors::GPUB200Multi::row_cuts(rp, 2) == std::vector<int64_t>({0, 4, 6}));
    CHECK(Competitors::GPUB200Multi::row_cuts(rp, 1) == std::vector<int64_t>({0, 6}));
    const std::vector<int64_t> c3 = Competitors::GPUB200Multi::row_cuts(rp, 3);
    CHECK(c3.front() == 0 && c3.back() == 6 && std::is_sorted(c3.begin(), c3.end()));
    // more shards than rows: cuts stay monotone, some shards are empty
    const std::vector<int64_t> c8 = Competitors::GPUB200Multi::row_cuts(rp, 8);
    CHECK(c8.size() == 9 && c8.front() == 0 && c8.back() == 6 && std::is_sorted(c8.begin(), c8.end()));
    // aligned cuts land on multiples of 64
    std::vector<int> big(1025);
    for (int i = 0; i <= 1024; ++i) big[static_cast<size_t>(i)] = 7 * i;
    for (int64_t c : Competitors::GPUB200Multi::row_cuts(big, 4, 64)) CHECK(c % 64 == 0);
}

TEST_CASE(multi_device_shards_and_reuse) {
    // a matrix big enough for aligned cuts and dense tiles, run twice through the same object with different inputs
    auto multi = std::make_shared<Competitors::GPUB200Multi>(std::vector<int>{0, 0, 0}, SDDMM_B200_FP32_TC, "GPU-B200-3shards");
    for (int round = 0; round < 2; ++round) {
        SDDMM::SyntheticDataset d(round == 0 ? 2 : 3, round == 0 ? 32 : 64, round == 0 ? 0.15 : 0.01);
        CSR<float> ref(d.getS_CSR()), P(d.getS_CSR());
        competitors()[0]->run_csr(d.getA(), d.getB(), d.getS_CSR(), ref);
        multi->init_csr(d.getA(), d.getB(), d.getS_CSR(), P);
        multi->run_csr(d.getA(), d.getB(), d.getS_CSR(), P);
        multi->cleanup_csr(d.getA(), d.getB(), d.getS_CSR(), P);
        CHECK(multi->shards() == 3 && multi->cuts().size() == 4 && multi->last_kernel_ms() > 0.f);
        std::vector<int> rows;
        for (int i = 0; i < d.getS_CSR().getRows(); ++i)
            rows.insert(rows.end(), static_cast<size_t>(d.getS_CSR().getRowPositions()[static_cast<size_t>(i) + 1] - d.getS_CSR().getRowPositions()[static_cast<size_t>(i)]), i);
        CHECK(close_enough(d.getA(), d.getB(), d.getS_CSR(), rows, P, ref, 1e-5));
    }
}

TEST_CASE(launch_shape_is_reported) {
    auto d = SDDMM::SyntheticDataset::uniform(300, 300, 32, 9000, 5);
    auto &gpu = *competitors()[1];
    CSR<float> P(d.getS_CSR());
    gpu.init_csr(d.getA(), d.getB(), d.getS_CSR(), P);
    CHECK(gpu.get_num_thread_blocks() >= 1 && gpu.get_num_threads_per_block() == 256);
    gpu.run_csr(d.getA(), d.getB(), d.getS_CSR(), P);
    gpu.cleanup_csr(d.getA(), d.getB(), d.getS_CSR(), P);
}

int main(int argc, char **argv) {
    if (sddmm_b200_device_count() < 1) { std::printf("no CUDA device\n"); return 77; }
    return tiny_test::run_all(argc > 1 ? argv[1] : nullptr);
}
