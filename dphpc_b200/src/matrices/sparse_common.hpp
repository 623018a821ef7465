// Helpers shared by the CSR and COO containers.
#pragma once
#include <algorithm>
#include <cmath>
#include <type_traits>
#include <vector>

#include "triplet.h"

namespace sparse_detail {

// sort by (row, col), then drop neighbours that compare equal (see triplet.h)
template <typename T>
inline void canonicalise(std::vector<Triplet<T>> &t) {
    std::sort(t.begin(), t.end());
    t.erase(std::unique(t.begin(), t.end()), t.end());
}

// Value comparison used by operator== of the containers.  The reference accepts
// |rhs - lhs| / rhs <= 1e-3 with a signed denominator (src/matrices/CSR.hpp:91-95), which only
// works for positive data without cancellation.  Here an entry matches when
//   |rhs - lhs| <= 1e-3 * |rhs| + 1e-5 * max_i |rhs_i|
// i.e. the same relative bar, plus an absolute floor scaled by the largest entry so that
// outputs that cancel to (nearly) zero are not held to an impossible relative error.
template <typename T>
inline bool values_match(const std::vector<T> &lhs, const std::vector<T> &rhs) {
    if (lhs.size() != rhs.size()) return false;
    if (std::is_integral<T>::value) return lhs == rhs;
    double scale = 0.0;
    for (const T &v : rhs) scale = std::max(scale, std::fabs(static_cast<double>(v)));
    for (size_t i = 0; i < lhs.size(); ++i) {
        const double d = std::fabs(static_cast<double>(rhs[i]) - static_cast<double>(lhs[i]));
        if (!(d <= 1e-3 * std::fabs(static_cast<double>(rhs[i])) + 1e-5 * scale)) return false;
    }
    return true;
}

}  // namespace sparse_detail
