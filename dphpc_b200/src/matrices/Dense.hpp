// Row-major dense matrix on the host.  Public interface of the reference's
// Dense<T> (src/matrices/Dense.hpp): construct from vector-of-rows, getValue,
// get_pointer, getRows, getCols.  A flat constructor is added so large synthetic
// operands need no vector-of-vectors detour.
#pragma once
#include <cassert>
#include <cstddef>
#include <ostream>
#include <utility>
#include <vector>

template <class T>
class Dense {
public:
    Dense() = default;

    explicit Dense(std::vector<std::vector<T>> &rows_in) {
        assert(!rows_in.empty());
        n_rows = static_cast<unsigned>(rows_in.size());
        n_cols = static_cast<unsigned>(rows_in.front().size());
        data.reserve(static_cast<size_t>(n_rows) * n_cols);
        for (const auto &r : rows_in) data.insert(data.end(), r.begin(), r.end());
    }

    // extension: adopt a flat row-major buffer
    Dense(unsigned rows, unsigned cols, std::vector<T> flat) : n_rows(rows), n_cols(cols), data(std::move(flat)) {
        assert(data.size() == static_cast<size_t>(rows) * cols);
    }

    T &getValue(int row, int col) { return data[static_cast<size_t>(row) * n_cols + col]; }
    T *get_pointer() { return data.data(); }
    unsigned int getRows() const { return n_rows; }
    unsigned int getCols() const { return n_cols; }

    friend std::ostream &operator<<(std::ostream &os, const Dense &m) {
        for (unsigned i = 0; i < m.n_rows; ++i) {
            for (unsigned j = 0; j < m.n_cols; ++j) os << m.data[static_cast<size_t>(i) * m.n_cols + j] << ' ';
            os << '\n';
        }
        return os;
    }

private:
    unsigned n_rows = 0, n_cols = 0;
    std::vector<T> data;
};
