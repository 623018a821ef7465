// Host side of the pageable-memory staging (dphpc_b200/csrc/host_staging.cuh): the thread pool, the sliced copy and the
// cache-bypassing copy are plain host code and are checked here without a device.
#include <cstdint>
#include <numeric>
#include <thread>
#include <vector>

#include "check.hpp"
#include "host_staging.cuh"

TEST_CASE(pool_runs_every_slice_once_and_takes_callers_in_turn) {
    sddmm::HostPool &pool = sddmm::HostPool::instance();
    CHECK(pool.width() >= 1);
    std::vector<int> hits(1000, 0);
    pool.run(static_cast<int>(hits.size()), [&](int k) { ++hits[static_cast<size_t>(k)]; });
    CHECK(std::all_of(hits.begin(), hits.end(), [](int h) { return h == 1; }));
    // several host threads (one per device in the multi-device competitor) share the pool
    std::vector<std::vector<int>> per(4, std::vector<int>(257, 0));
    std::vector<std::thread> callers;
    for (int t = 0; t < 4; ++t)
        callers.emplace_back([&, t] {
            for (int rep = 0; rep < 20; ++rep) pool.run(257, [&](int k) { ++per[static_cast<size_t>(t)][static_cast<size_t>(k)]; });
        });
    for (std::thread &c : callers) c.join();
    for (const auto &v : per) CHECK(std::all_of(v.begin(), v.end(), [](int h) { return h == 20; }));
}

TEST_CASE(sliced_and_streaming_copies_move_every_byte) {
    for (size_t bytes : {size_t(0), size_t(1), size_t(63), size_t(4096), size_t(4097), (size_t(5) << 20) + 13, (size_t(33) << 20) + 7}) {
        std::vector<unsigned char> src(bytes + 64), dst(bytes + 128, 0xEE);
        for (size_t i = 0; i < src.size(); ++i) src[i] = static_cast<unsigned char>((i * 131u + 7u) & 0xFF);
        for (size_t shift : {size_t(0), size_t(3)}) {   // source alignment is free, the destination here is 64-byte aligned + 64
            unsigned char *d = dst.data() + 64 - (reinterpret_cast<uintptr_t>(dst.data()) & 63);
            std::fill(dst.begin(), dst.end(), 0xEE);
            sddmm::parallel_memcpy(d, src.data() + shift, bytes, /*stream_stores=*/true);
            CHECK(std::equal(d, d + bytes, src.data() + shift));
            CHECK(d[bytes] == 0xEE && (d == dst.data() || d[-1] == 0xEE));
            std::fill(dst.begin(), dst.end(), 0xEE);
            sddmm::parallel_memcpy(d, src.data() + shift, bytes);
            CHECK(std::equal(d, d + bytes, src.data() + shift));
            CHECK(d[bytes] == 0xEE);
        }
    }
    // a destination that is not 16-byte aligned falls back to memcpy
    std::vector<unsigned char> a(10000), b(10016, 0);
    std::iota(a.begin(), a.end(), static_cast<unsigned char>(1));
    sddmm::stream_copy(b.data() + 1, a.data(), a.size());
    CHECK(std::equal(a.begin(), a.end(), b.begin() + 1));
}

int main(int argc, char **argv) { return tiny_test::run_all(argc > 1 ? argv[1] : nullptr); }
