// cleanup_* of a GPU competitor hands P back with S's pattern (the reference's convention, e.g.
// src/competitors/gpu/gpu_convert.hpp:58-64).  The containers only offer copying setters for the index arrays
// (src/matrices/CSR.hpp:125-139, src/matrices/COO.hpp:149-163), 150 MB each on the largest configuration, and one
// thread copies at about a fifth of what the host memory gives: here the copies run on helper threads, several per
// array, beside the device-to-host copy of the values instead of after it.
#pragma once
#include <algorithm>
#include <cstring>
#include <thread>
#include <vector>

namespace SDDMM {

namespace detail {
// dst = src, the bytes moved by the calling thread and up to `helpers` more (the getters hand out const references to
// plain, non-const members: writing through them is the setter's effect without its single-threaded copy)
inline void copy_index_array(const std::vector<int> &dst_ref, const std::vector<int> &src, int helpers) {
    std::vector<int> &dst = const_cast<std::vector<int> &>(dst_ref);
    if (&dst == &src) return;
    dst.resize(src.size());
    const size_t n = src.size();
    const int parts = static_cast<int>(std::min<size_t>(static_cast<size_t>(helpers) + 1, std::max<size_t>(1, n >> 20)));   // >= 4 MB per thread
    const size_t per = (n + parts - 1) / parts;
    std::vector<std::thread> th;
    for (int k = 1; k < parts; ++k) {
        const size_t a = std::min(n, per * static_cast<size_t>(k)), b = std::min(n, a + per);
        if (a < b) th.emplace_back([&dst, &src, a, b] { std::memcpy(dst.data() + a, src.data() + a, (b - a) * sizeof(int)); });
    }
    if (n) std::memcpy(dst.data(), src.data(), std::min(n, per) * sizeof(int));
    for (std::thread &t : th) t.join();
}
}  // namespace detail

// P takes S's index arrays on helper threads while `download` (which fills P's values) runs on the caller's.
template <class Sparse, class Download>
void finish_into(Sparse &S, Sparse &P, Download &&download) {
    if (P.getValues().size() != S.getValues().size()) P.getValues().resize(S.getValues().size());
    std::thread cols([&] { detail::copy_index_array(P.getColPositions(), S.getColPositions(), 3); });
    std::thread rows([&] { detail::copy_index_array(P.getRowPositions(), S.getRowPositions(), 3); });
    download(P.getValues().data());
    cols.join();
    rows.join();
}

}  // namespace SDDMM
