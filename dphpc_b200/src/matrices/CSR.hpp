// Compressed sparse row container on the host with the public interface of the
// reference's CSR<T> (src/matrices/CSR.hpp): construction from triplets (sorted,
// de-duplicated, empty rows kept) or from a COO, accessors/setters, clearValues,
// the nnz-balanced row dispatcher (computeDispatcher / computeDispatcherTensorCores
// -> getStartIdx) and getDensity.
// Deviations, on purpose: getDensity() multiplies in double (the reference's int
// product overflows from 46 341 rows on); operator== compares against |rhs|.
#pragma once
#include <cassert>
#include <cstdint>
#include <iostream>
#include <ostream>
#include <vector>

#include "sparse_common.hpp"
#include "triplet.h"

template <class T>
class COO;

template <class T>
class CSR {
public:
    CSR() = default;

    CSR(int rows, int cols, std::vector<Triplet<T>> triplets) : n_rows(rows), n_cols(cols) { build(triplets); }

    CSR(const CSR &) = default;
    CSR &operator=(const CSR &) = default;

    explicit CSR(COO<T> &coo) : n_rows(coo.getRows()), n_cols(coo.getCols()) {
        const size_t n = coo.getValues().size();
        std::vector<Triplet<T>> t(n);
        for (size_t i = 0; i < n; ++i) t[i] = Triplet<T>{coo.getRowPositions()[i], coo.getColPositions()[i], coo.getValues()[i]};
        build(t);
    }

    // extension: adopt arrays that are already in canonical CSR form
    CSR(int rows, int cols, std::vector<int> row_ptr, std::vector<int> col_idx, std::vector<T> vals)
        : n_rows(rows), n_cols(cols), row_ptr(std::move(row_ptr)), col_idx(std::move(col_idx)), vals(std::move(vals)) {
        assert(static_cast<int>(this->row_ptr.size()) == rows + 1 && this->col_idx.size() == this->vals.size());
    }

    int getRows() const { return n_rows; }
    int getCols() const { return n_cols; }

    void clearValues() { std::fill(vals.begin(), vals.end(), T(0)); }
    std::vector<T> &getValues() { return vals; }
    void setValues(const std::vector<T> &v) { vals = v; }
    const std::vector<int> &getColPositions() { return col_idx; }
    void setColPositions(const std::vector<int> &c) { col_idx = c; }
    const std::vector<int> &getRowPositions() { return row_ptr; }
    void setRowPositions(const std::vector<int> &r) { row_ptr = r; }
    T *getValue(int j) { return &vals[j]; }

    const std::vector<int> &getStartIdx() { return start_idx; }
    void computeDispatcher(int parts) { dispatch(parts, 1); }
    void computeDispatcherTensorCores(int parts) { dispatch(parts, 16); }

    double getDensity() const { return static_cast<double>(vals.size()) / (static_cast<double>(n_rows) * static_cast<double>(n_cols)); }

    friend bool operator==(const CSR &lhs, const CSR &rhs) {
        const bool pattern = lhs.n_rows == rhs.n_rows && lhs.n_cols == rhs.n_cols && lhs.row_ptr == rhs.row_ptr && lhs.col_idx == rhs.col_idx;
        if (!pattern) std::cout << "Cols and Rows don't match" << std::endl;
        return pattern && sparse_detail::values_match(lhs.vals, rhs.vals);
    }

    friend std::ostream &operator<<(std::ostream &os, const CSR &m) {
        for (const T &v : m.vals) os << v << ' ';
        os << '\n';
        for (int c : m.col_idx) os << c << ' ';
        os << '\n';
        for (int r : m.row_ptr) os << r << ' ';
        return os << '\n';
    }

private:
    int n_rows = 0, n_cols = 0;
    std::vector<int> row_ptr, col_idx;
    std::vector<T> vals;
    std::vector<int> start_idx;

    void build(std::vector<Triplet<T>> &t) {
        assert(!t.empty());
        sparse_detail::canonicalise(t);
        row_ptr.assign(static_cast<size_t>(n_rows) + 1, 0);
        col_idx.resize(t.size());
        vals.resize(t.size());
        for (size_t i = 0; i < t.size(); ++i) {
            assert(t[i].row >= 0 && t[i].row < n_rows);
            ++row_ptr[static_cast<size_t>(t[i].row) + 1];
            col_idx[i] = t[i].col;
            vals[i] = t[i].value;
        }
        for (int r = 0; r < n_rows; ++r) row_ptr[r + 1] += row_ptr[r];
    }

    // Split the rows (in groups of `stride`) into at most `parts` contiguous ranges whose largest
    // nnz is minimal: smallest feasible capacity by bisection, then a greedy left-to-right cut;
    // the list is padded with n_rows so that it always has parts + 1 entries (the contract the
    // reference's tests pin, tests/matrix_test.cc:354-425, 460-477).
    void dispatch(int parts, int stride) {
        std::vector<int64_t> load;
        for (int r = 0; r < n_rows; r += stride) load.push_back(row_ptr[std::min(n_rows, r + stride)] - row_ptr[r]);
        const auto segments_needed = [&](int64_t cap) -> int64_t {
            int64_t segs = 1, acc = 0;
            for (int64_t w : load) {
                if (w > cap) return INT64_MAX;
                acc += w;
                if (acc > cap) { ++segs; acc = w; }
            }
            return segs;
        };
        int64_t lo = 1, hi = static_cast<int64_t>(vals.size()), cap = 0;
        while (lo <= hi) {
            const int64_t mid = lo + (hi - lo) / 2;
            if (segments_needed(mid) <= parts) { cap = mid; hi = mid - 1; } else { lo = mid + 1; }
        }
        start_idx.assign(1, 0);
        int64_t acc = 0;
        for (size_t g = 0; g < load.size(); ++g) {
            acc += load[g];
            if (acc > cap) { start_idx.push_back(static_cast<int>(g) * stride); acc = load[g]; }
        }
        while (static_cast<int>(start_idx.size()) <= parts) start_idx.push_back(n_rows);
    }
};

#include "COO.hpp"
