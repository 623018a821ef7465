// Coordinate-format container on the host with the public interface of the
// reference's COO<T> (src/matrices/COO.hpp): entries sorted by (row, col),
// de-duplicated; conversion from CSR expands row_ptr.
#pragma once
#include <cassert>
#include <iostream>
#include <ostream>
#include <vector>

#include "sparse_common.hpp"
#include "triplet.h"

template <class T>
class CSR;

template <class T>
class COO {
public:
    COO() = default;

    COO(int rows, int cols, std::vector<Triplet<T>> t) : n_rows(rows), n_cols(cols) {
        assert(!t.empty());
        sparse_detail::canonicalise(t);
        reserve(t.size());
        for (const auto &e : t) {
            assert(e.row >= 0 && e.row < n_rows && e.col >= 0 && e.col < n_cols);
            row_idx.push_back(e.row);
            col_idx.push_back(e.col);
            vals.push_back(e.value);
        }
    }

    COO(const COO &) = default;
    COO &operator=(const COO &) = default;

    explicit COO(CSR<T> &csr) : n_rows(csr.getRows()), n_cols(csr.getCols()) {
        reserve(csr.getValues().size());
        const auto &rp = csr.getRowPositions();
        for (int r = 0; r < n_rows; ++r)
            for (int j = rp[r]; j < rp[r + 1]; ++j) {
                row_idx.push_back(r);
                col_idx.push_back(csr.getColPositions()[j]);
                vals.push_back(csr.getValues()[j]);
            }
    }

    int getRows() const { return n_rows; }
    int getCols() const { return n_cols; }
    void clearValues() { std::fill(vals.begin(), vals.end(), T(0)); }
    std::vector<T> &getValues() { return vals; }
    void setValues(const std::vector<T> &v) { vals = v; }
    const std::vector<int> &getColPositions() { return col_idx; }
    void setColPositions(const std::vector<int> &c) { col_idx = c; }
    const std::vector<int> &getRowPositions() { return row_idx; }
    void setRowPositions(const std::vector<int> &r) { row_idx = r; }
    T *getValue(int j) { return &vals[j]; }

    friend bool operator==(const COO &lhs, const COO &rhs) {
        const bool pattern = lhs.n_rows == rhs.n_rows && lhs.n_cols == rhs.n_cols && lhs.row_idx == rhs.row_idx && lhs.col_idx == rhs.col_idx;
        if (!pattern) std::cout << "Cols and Rows don't match" << std::endl;
        return pattern && sparse_detail::values_match(lhs.vals, rhs.vals);
    }

    friend std::ostream &operator<<(std::ostream &os, const COO &m) {
        for (int r : m.row_idx) os << r << ' ';
        os << '\n';
        for (int c : m.col_idx) os << c << ' ';
        os << '\n';
        for (const T &v : m.vals) os << v << ' ';
        return os << '\n';
    }

private:
    int n_rows = 0, n_cols = 0;
    std::vector<int> row_idx, col_idx;
    std::vector<T> vals;

    void reserve(size_t n) {
        row_idx.reserve(n);
        col_idx.reserve(n);
        vals.reserve(n);
    }
};

#include "CSR.hpp"
