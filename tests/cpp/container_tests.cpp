// Host containers and dispatcher: the cases of the reference's tests/matrix_test.cc that need no GPU
// (BasicTest.COO :84-91, RepresentationConversion :93-106, BiggerConversion :108-122, dispatcher_* :354-425,
// test_dispatch_tensor :460-477, DummyDataset known answer), run against this repository's interface mirror.
#include <numeric>

#include "benchmark/dataset.hpp"
#include "check.hpp"
#include "matrices/matrices.h"

TEST_CASE(coo_sizes) {
    std::vector<Triplet<float>> t{{0, 0, 1.0f}, {0, 1, 1.0f}, {1, 0, 1.0f}, {1, 1, 1.0f}};
    COO<float> coo(2, 2, t);
    CHECK_EQ(coo.getValues().size(), size_t(4));
    CHECK_EQ(coo.getRowPositions().size(), size_t(4));
    CHECK_EQ(coo.getColPositions().size(), size_t(4));
}

TEST_CASE(representation_conversion) {
    std::vector<Triplet<float>> unsorted{{0, 0, 1.0f}, {1, 0, 1.0f}, {0, 1, 1.0f}, {1, 1, 1.0f}};
    CSR<float> csr(2, 2, unsorted);
    std::vector<Triplet<float>> sorted{{0, 0, 1.0f}, {0, 1, 1.0f}, {1, 0, 1.0f}, {1, 1, 1.0f}};
    COO<float> coo(2, 2, sorted);
    CHECK(csr == CSR<float>(coo));
    CHECK(coo == COO<float>(csr));
}

TEST_CASE(bigger_conversion) {
    for (int i = 100; i <= 1500; i += 25) {
        SDDMM::SyntheticDataset d = SDDMM::SyntheticDataset::uniform(2 * i, i, 4, i, 1000 + i);
        CHECK(d.getS_CSR() == CSR<float>(d.getS_COO()));
        CHECK(d.getS_COO() == COO<float>(d.getS_CSR()));
        CHECK_EQ(d.getS_CSR().getRowPositions().size(), size_t(2 * i + 1));
    }
}

TEST_CASE(duplicates_follow_the_reference_rule) {
    // (0,1) twice with non-zero values collapses to the first; a zero value keeps both entries
    std::vector<Triplet<float>> t{{0, 1, 1.0f}, {0, 1, 2.0f}, {0, 2, 0.0f}, {0, 2, 3.0f}};
    CSR<float> csr(1, 3, t);
    CHECK_EQ(csr.getColPositions(), (std::vector<int>{1, 2, 2}));
}

static std::vector<int> dispatch(CSR<float> m, int parts, bool tensor = false) {
    if (tensor) m.computeDispatcherTensorCores(parts); else m.computeDispatcher(parts);
    return m.getStartIdx();
}

TEST_CASE(dispatcher_golden_vectors) {
    std::vector<Triplet<float>> full{{0, 0, 1.0f}, {1, 0, 1.0f}, {0, 1, 1.0f}, {1, 1, 1.0f}};
    CHECK_EQ(dispatch(CSR<float>(2, 2, full), 4), (std::vector<int>{0, 1, 2, 2, 2}));
    CHECK_EQ(dispatch(CSR<float>(2, 2, full), 2), (std::vector<int>{0, 1, 2}));
    std::vector<Triplet<float>> four{{0, 0, 1.0f}, {1, 0, 1.0f}, {2, 1, 1.0f}, {3, 1, 1.0f}};
    CHECK_EQ(dispatch(CSR<float>(4, 2, four), 2), (std::vector<int>{0, 2, 4}));
    std::vector<Triplet<float>> one{{1, 0, 1.0f}};
    CHECK_EQ(dispatch(CSR<float>(4, 2, one), 2), (std::vector<int>{0, 4, 4}));
}

TEST_CASE(dispatcher_large_regular_input) {
    const int n = 150000;
    std::vector<Triplet<float>> t;
    for (int i = 0; i < n; ++i) t.push_back({i, i, 4.0f});
    std::vector<int> expected(n / 2 + 1);
    for (int i = 0; i <= n / 2; ++i) expected[i] = 2 * i;
    CHECK_EQ(dispatch(CSR<float>(n, n, t), n / 2), expected);
}

TEST_CASE(dispatcher_tensor_stride) {
    std::vector<Triplet<float>> t;
    for (int i = 0; i < 64; ++i) t.push_back({i, i, 1.0f});
    CHECK_EQ(dispatch(CSR<float>(64, 64, t), 4, true), (std::vector<int>{0, 16, 32, 48, 64}));
}

TEST_CASE(dummy_dataset_expected) {
    SDDMM::DummyDataset d;
    CHECK(d.hasExpected());
    CHECK_EQ(d.getExpected_CSR().getValues(), std::vector<float>(4, 2.0f));
    CHECK_EQ(d.getS_COO().getRowPositions(), (std::vector<int>{0, 0, 1, 1}));
}

TEST_CASE(density_does_not_overflow) {
    CSR<float> big(503712, 503712, std::vector<int>(503713, 0), {}, {});
    CHECK(big.getDensity() == 0.0);
    SDDMM::SyntheticDataset d(1, 4);
    CHECK(d.getS_CSR().getDensity() > 0.04 && d.getS_CSR().getDensity() < 0.05);
}

int main(int argc, char **argv) { return tiny_test::run_all(argc > 1 ? argv[1] : nullptr); }
