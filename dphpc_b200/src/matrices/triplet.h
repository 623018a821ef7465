// (row, col, value) entry used to build sparse containers.
// Same public shape and comparison semantics as the reference's Triplet<T>
// (src/matrices/triplet.h): ordering is by (row, col); two triplets compare equal
// only when position matches AND both values are non-zero -- the rule its
// std::unique based de-duplication relies on.
#pragma once
#include <ostream>

template <typename T>
struct Triplet {
    int row;
    int col;
    T value;
};

template <typename T>
inline bool operator<(const Triplet<T> &a, const Triplet<T> &b) {
    return (a.row != b.row) ? (a.row < b.row) : (a.col < b.col);
}

template <typename T>
inline bool operator==(const Triplet<T> &a, const Triplet<T> &b) {
    const bool same_cell = (a.row == b.row) && (a.col == b.col);
    return same_cell && (a.value != T(0)) && (b.value != T(0));
}

template <typename T>
inline std::ostream &operator<<(std::ostream &os, const Triplet<T> &t) {
    return os << t.row << ' ' << t.col << ' ' << t.value;
}
