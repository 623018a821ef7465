// Host containers and dispatcher: the cases of the reference's tests/matrix_test.cc that need no GPU
// (BasicTest.COO :84-91, RepresentationConversion :93-106, BiggerConversion :108-122, dispatcher_* :354-425,
// test_dispatch_tensor :460-477, DummyDataset known answer), run against this repository's interface mirror.
#include <algorithm>
#include <cstdlib>
#include <fstream>
#include <numeric>

#include "benchmark/dataset.hpp"
#include "check.hpp"
#include "competitors/gpu/pattern_copy.hpp"
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

namespace {
std::string write_temp(const char *name, const char *text) {
    const char *dir = std::getenv("TMPDIR");
    const std::string path = std::string(dir ? dir : "/tmp") + "/sddmm_b200_" + name;
    std::ofstream(path) << text;
    return path;
}
template <typename F>
bool throws(F f) {
    try { f(); } catch (const std::runtime_error &) { return true; }
    return false;
}
}  // namespace

TEST_CASE(matrix_market_reader_follows_the_reference_rules) {
    // comments, 1-based coordinates, a numerically zero entry (dropped), unsorted input, a duplicate coordinate,
    // a symmetric header that is NOT mirrored (src/benchmark/dataset.hpp:150-180 of the reference)
    const std::string path = write_temp("a.mtx",
        "%%MatrixMarket matrix coordinate real symmetric\n% a comment\n4 5 6\n3 2 1.5\n1 1 2.0\n4 5 -3.0\n2 3 1e-9\n1 4 0.5\n3 2 7.0\n");
    SDDMM::MatrixMarketDataset d("tiny", path, 8);
    CSR<float> &S = d.getS_CSR();
    CHECK_EQ(S.getRows(), 4);
    CHECK_EQ(S.getCols(), 5);
    CHECK(S.getRowPositions() == std::vector<int>({0, 2, 2, 3, 4}));      // row 2 lost its only (zero) entry
    CHECK(S.getColPositions() == std::vector<int>({0, 3, 1, 4}));
    CHECK_EQ(S.getValues()[0], 2.0f);
    CHECK_EQ(S.getValues()[3], -3.0f);
    CHECK_EQ(static_cast<int>(d.getA().getRows()), 4);
    CHECK_EQ(static_cast<int>(d.getB().getRows()), 5);
    CHECK_EQ(static_cast<int>(d.getA().getCols()), 8);
    CHECK(d.getS_COO() == COO<float>(S));
    // the dense operands depend on the seed only
    SDDMM::MatrixMarketDataset again("tiny", path, 8);
    const size_t na = static_cast<size_t>(d.getA().getRows()) * d.getA().getCols();
    CHECK(std::equal(d.getA().get_pointer(), d.getA().get_pointer() + na, again.getA().get_pointer()));
    float lo = 1.f, hi = -1.f;
    const size_t nb = static_cast<size_t>(d.getB().getRows()) * d.getB().getCols();
    for (size_t i = 0; i < nb; ++i) { lo = std::min(lo, d.getB().get_pointer()[i]); hi = std::max(hi, d.getB().get_pointer()[i]); }
    CHECK(lo >= -1.f && hi < 1.f && lo < 0.f && hi > 0.f);
}

TEST_CASE(matrix_market_pattern_files_and_bad_input) {
    const std::string pat = write_temp("p.mtx", "%%MatrixMarket matrix coordinate pattern general\n3 3 2\n1 3\n3 1\n");
    SDDMM::MatrixMarketDataset d("pattern", pat, 4);
    CHECK(d.getS_CSR().getColPositions() == std::vector<int>({2, 0}));
    CHECK(d.getS_CSR().getValues() == std::vector<float>({1.0f, 1.0f}));
    CHECK(throws([] { SDDMM::MatrixMarketDataset x("missing", "/nonexistent/file.mtx", 4); }));
    const std::string short_file = write_temp("s.mtx", "3 3 4\n1 1 1.0\n");
    CHECK(throws([&] { SDDMM::MatrixMarketDataset x("short", short_file, 4); }));
    const std::string range = write_temp("r.mtx", "3 3 1\n4 1 1.0\n");
    CHECK(throws([&] { SDDMM::MatrixMarketDataset x("range", range, 4); }));
}

TEST_CASE(edge_list_reader) {
    const std::string path = write_temp("e.txt", "# Directed graph\n# Nodes: 4 Edges: 4\n# FromNodeId\tToNodeId\n0\t1\n2\t3\n2\t0\n0\t1\n");
    SDDMM::EdgeListDataset d("edges", path, 4, 4, 4);
    CHECK(d.getS_CSR().getRowPositions() == std::vector<int>({0, 1, 1, 3, 3}));
    CHECK(d.getS_CSR().getColPositions() == std::vector<int>({1, 0, 3}));
    CHECK(d.getS_CSR().getValues() == std::vector<float>({1.0f, 1.0f, 1.0f}));
    CHECK(throws([&] { SDDMM::EdgeListDataset x("small", path, 2, 2, 4); }));
}

// cleanup_* of the GPU competitors: P takes S's pattern on helper threads while the download fills the values
// (the reference's convention for what P holds afterwards: src/competitors/gpu/gpu_convert.hpp:58-64)
TEST_CASE(cleanup_hands_back_the_pattern_of_s_with_the_downloaded_values) {
    std::vector<Triplet<float>> t = {{0, 1, 0.5f}, {0, 3, 1.5f}, {2, 0, 2.5f}, {3, 3, 3.5f}};
    CSR<float> S(4, 4, t);
    CSR<float> P;   // empty: values are sized, the pattern copied
    SDDMM::finish_into(S, P, [](float *v) { for (int i = 0; i < 4; ++i) v[i] = 10.f * static_cast<float>(i); });
    CHECK(P.getRowPositions() == S.getRowPositions());
    CHECK(P.getColPositions() == S.getColPositions());
    CHECK(P.getValues() == std::vector<float>({0.f, 10.f, 20.f, 30.f}));
    CSR<float> stale(4, 4, t);   // same size, stale values: everything is overwritten, nothing reallocated
    const float *before = stale.getValues().data();
    SDDMM::finish_into(S, stale, [](float *v) { for (int i = 0; i < 4; ++i) v[i] = -1.f; });
    CHECK(stale.getValues().data() == before);
    CHECK(stale.getValues() == std::vector<float>(4, -1.f));
    COO<float> Sc(S), Pc;
    SDDMM::finish_into(Sc, Pc, [](float *v) { for (int i = 0; i < 4; ++i) v[i] = 1.f; });
    CHECK(Pc.getRowPositions() == Sc.getRowPositions());
    CHECK(Pc.getColPositions() == Sc.getColPositions());
    CHECK(Pc.getValues() == std::vector<float>(4, 1.f));
}

int main(int argc, char **argv) { return tiny_test::run_all(argc > 1 ? argv[1] : nullptr); }
