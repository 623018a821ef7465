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
// |rhs - lhs| / rhs <= 1e-3 with a signed denominator (src/matrices/CSR.hpp:91-95),
// which only works for positive data; here the denominator is |rhs| and exact
// zeros must match exactly, so signed SDDMM outputs compare sensibly.
template <typename T>
inline bool values_match(const std::vector<T> &lhs, const std::vector<T> &rhs) {
    if (lhs.size() != rhs.size()) return false;
    if (std::is_integral<T>::value) return lhs == rhs;
    for (size_t i = 0; i < lhs.size(); ++i) {
        const double d = std::fabs(static_cast<double>(rhs[i]) - static_cast<double>(lhs[i]));
        const double ref = std::fabs(static_cast<double>(rhs[i]));
        if (ref == 0.0 ? d != 0.0 : d / ref > 1e-3) return false;
    }
    return true;
}

}  // namespace sparse_detail
