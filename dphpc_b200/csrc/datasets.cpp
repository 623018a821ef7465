// Seeded synthetic SDDMM inputs (see include/sddmm_datasets.h).  Host only.
//
// Every random decision is a pure function of (seed, stream, index) through a
// splitmix64 finaliser, so rows can be generated in parallel and the result
// does not depend on the number of threads.
#include "../../include/sddmm_datasets.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <new>
#include <string>
#include <thread>
#include <unordered_set>
#include <vector>

namespace {

inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// sequential generator for one (seed, stream, index) cell
struct Rng {
    uint64_t s;
    Rng(uint64_t seed, uint64_t stream, uint64_t index) : s(mix64(seed ^ mix64(stream * 0xD1B54A32D192ED03ull + index))) {}
    uint64_t next() {
        s += 0x9E3779B97F4A7C15ull;
        uint64_t z = s;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    double u01() { return static_cast<double>(next() >> 11) * (1.0 / 9007199254740992.0); }      // [0,1)
    float f01() { return static_cast<float>(next() >> 40) * (1.0f / 16777216.0f); }                // [0,1), 24 bits
    uint64_t below(uint64_t n) { return static_cast<uint64_t>((static_cast<unsigned __int128>(next()) * n) >> 64); }
};

// exact Zipf(2) on {1..kmax}: propose k with P(k) = 1/(k(k+1)) (k = floor(1/u)),
// accept with probability (k+1)/(2k)  ->  P(k) proportional to k^-2
inline int64_t zipf2(Rng &r, int64_t kmax) {
    for (;;) {
        double u = 1.0 - r.u01();  // (0,1]
        double kd = std::floor(1.0 / u);
        if (kd > static_cast<double>(kmax)) continue;
        int64_t k = static_cast<int64_t>(kd);
        if (r.u01() * 2.0 * static_cast<double>(k) < static_cast<double>(k + 1)) return k;
    }
}

inline int poisson(Rng &r, double lambda) {
    const double limit = std::exp(-lambda);
    double p = 1.0;
    int k = 0;
    do {
        ++k;
        p *= r.u01();
    } while (p > limit);
    return k - 1;
}

void parallel_for(int64_t n, const std::function<void(int64_t, int64_t, int)> &fn) {
    unsigned hw = std::thread::hardware_concurrency();
    int nt = static_cast<int>(std::max(1u, std::min(hw ? hw : 1u, 32u)));
    if (n < 4096) nt = 1;
    if (nt == 1) {
        fn(0, n, 0);
        return;
    }
    std::vector<std::thread> th;
    const int64_t per = (n + nt - 1) / nt;
    for (int t = 0; t < nt; ++t) {
        const int64_t a = t * per, b = std::min(n, a + per);
        if (a >= b) break;
        th.emplace_back(fn, a, b, t);
    }
    for (auto &x : th) x.join();
}

enum Stream : uint64_t { ST_A = 1, ST_B = 2, ST_VAL = 3, ST_LEN = 4, ST_COL = 5, ST_PERM = 6, ST_BLOCK = 7, ST_POS = 8 };

}  // namespace

// resize() without the value-initialising pass: the dense operands (gigabytes at K = 256) are first touched by the
// threads that fill them
template <class T>
struct NoInit : std::allocator<T> {
    template <class U>
    struct rebind {
        using other = NoInit<U>;
    };
    template <class U>
    void construct(U *p) noexcept {
        ::new (static_cast<void *>(p)) U;
    }
    template <class U, class... Args>
    void construct(U *p, Args &&...args) {
        ::new (static_cast<void *>(p)) U(std::forward<Args>(args)...);
    }
};
using DenseVec = std::vector<float, NoInit<float>>;

struct sddmm_dataset {
    std::string name;
    int64_t M = 0, N = 0, K = 0;
    std::vector<int32_t> row_ptr, col;
    std::vector<float> val;
    DenseVec A, B;
};

namespace {

void fill_dense(sddmm_dataset &d, uint64_t seed) {
    d.A.resize(static_cast<size_t>(d.M * d.K));
    d.B.resize(static_cast<size_t>(d.N * d.K));
    auto fill = [&](DenseVec &v, uint64_t stream) {
        parallel_for(static_cast<int64_t>(v.size()), [&](int64_t a, int64_t b, int) {
            for (int64_t i = a; i < b; ++i) {
                const uint64_t z = mix64(seed ^ mix64(stream * 0xD1B54A32D192ED03ull + static_cast<uint64_t>(i)));
                v[static_cast<size_t>(i)] = static_cast<float>(z >> 40) * (2.0f / 16777216.0f) - 1.0f;  // [-1,1)
            }
        });
    };
    fill(d.A, ST_A);
    fill(d.B, ST_B);
}

void fill_values(sddmm_dataset &d, uint64_t seed, bool ones) {
    d.val.resize(d.col.size());
    parallel_for(static_cast<int64_t>(d.val.size()), [&](int64_t a, int64_t b, int) {
        for (int64_t i = a; i < b; ++i) {
            if (ones) {
                d.val[static_cast<size_t>(i)] = 1.0f;
            } else {
                const uint64_t z = mix64(seed ^ mix64(ST_VAL * 0xD1B54A32D192ED03ull + static_cast<uint64_t>(i)));
                d.val[static_cast<size_t>(i)] = static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
            }
        }
    });
}

// row lengths -> row_ptr (exclusive scan); returns nnz
int64_t scan_lengths(const std::vector<int32_t> &len, std::vector<int32_t> &row_ptr) {
    row_ptr.resize(len.size() + 1);
    int64_t acc = 0;
    for (size_t i = 0; i < len.size(); ++i) {
        row_ptr[i] = static_cast<int32_t>(acc);
        acc += len[i];
    }
    row_ptr[len.size()] = static_cast<int32_t>(acc);
    return acc;
}

// Fill every row with `len` distinct columns drawn by `draw(rng, row)`; after
// `4*len + 64` failed attempts per row the remainder is filled uniformly.
template <typename Draw>
void fill_rows_distinct(sddmm_dataset &d, const std::vector<int32_t> &len, uint64_t seed, Draw draw) {
    const int64_t N = d.N;
    d.col.resize(static_cast<size_t>(d.row_ptr.back()));
    parallel_for(d.M, [&](int64_t a, int64_t b, int) {
        std::vector<int32_t> mark(static_cast<size_t>(N), -1);
        for (int64_t i = a; i < b; ++i) {
            const int L = len[static_cast<size_t>(i)];
            if (L == 0) continue;
            int32_t *out = d.col.data() + d.row_ptr[static_cast<size_t>(i)];
            Rng r(seed, ST_COL, static_cast<uint64_t>(i));
            int got = 0;
            int64_t budget = 4ll * L + 64;
            while (got < L && budget-- > 0) {
                const int64_t c = draw(r, i);
                if (c < 0 || c >= N) continue;
                if (mark[static_cast<size_t>(c)] == static_cast<int32_t>(i)) continue;
                mark[static_cast<size_t>(c)] = static_cast<int32_t>(i);
                out[got++] = static_cast<int32_t>(c);
            }
            while (got < L) {
                const int64_t c = static_cast<int64_t>(r.below(static_cast<uint64_t>(N)));
                if (mark[static_cast<size_t>(c)] == static_cast<int32_t>(i)) continue;
                mark[static_cast<size_t>(c)] = static_cast<int32_t>(i);
                out[got++] = static_cast<int32_t>(c);
            }
            std::sort(out, out + L);
        }
    });
}

int64_t scaled(int64_t full, double scale, int64_t lo) {
    int64_t v = static_cast<int64_t>(std::llround(static_cast<double>(full) * scale));
    return std::max(lo, std::min(full, v));
}

// ---- config 1 / uniform --------------------------------------------------------
void gen_uniform(sddmm_dataset &d, int64_t nnz, uint64_t seed) {
    const int64_t M = d.M, N = d.N;
    nnz = std::min(nnz, M * N);
    std::vector<uint64_t> keys;
    keys.reserve(static_cast<size_t>(nnz));
    if (nnz * 2 > M * N) {
        // dense-ish: choose the complement instead (partial Fisher-Yates over all cells)
        std::vector<uint64_t> all(static_cast<size_t>(M * N));
        for (size_t i = 0; i < all.size(); ++i) all[i] = i;
        Rng r(seed, ST_POS, 0);
        for (int64_t i = 0; i < nnz; ++i) {
            const uint64_t j = static_cast<uint64_t>(i) + r.below(static_cast<uint64_t>(M * N - i));
            std::swap(all[static_cast<size_t>(i)], all[static_cast<size_t>(j)]);
        }
        keys.assign(all.begin(), all.begin() + nnz);
    } else {
        std::unordered_set<uint64_t> seen;
        seen.reserve(static_cast<size_t>(nnz) * 2);
        Rng r(seed, ST_POS, 0);
        while (static_cast<int64_t>(keys.size()) < nnz) {
            const uint64_t k = r.below(static_cast<uint64_t>(M * N));
            if (seen.insert(k).second) keys.push_back(k);
        }
    }
    std::sort(keys.begin(), keys.end());
    d.row_ptr.assign(static_cast<size_t>(M + 1), 0);
    d.col.resize(keys.size());
    for (size_t i = 0; i < keys.size(); ++i) {
        const int64_t rrow = static_cast<int64_t>(keys[i] / static_cast<uint64_t>(N));
        d.col[i] = static_cast<int32_t>(keys[i] % static_cast<uint64_t>(N));
        d.row_ptr[static_cast<size_t>(rrow + 1)]++;
    }
    for (int64_t i = 0; i < M; ++i) d.row_ptr[static_cast<size_t>(i + 1)] += d.row_ptr[static_cast<size_t>(i)];
    fill_values(d, seed, false);
}

// ---- config 2: randomly placed 64x64 blocks, 70 % full ---------------------------
void gen_blocks(sddmm_dataset &d, int64_t target_nnz, uint64_t seed, bool unaligned) {
    const int64_t M = d.M, N = d.N;
    const int BS = 64;
    struct Block { int64_t r0, c0; uint64_t rows[64]; int64_t cnt; };
    const int64_t gr = M / BS, gc = N / BS;  // last partial block row / column excluded
    if (gr < 1 || gc < 1) { gen_uniform(d, target_nnz, seed); return; }
    const int64_t max_blocks = unaligned ? (gr * gc) / 2 : gr * gc;
    std::vector<Block> blocks;
    std::unordered_set<uint64_t> used;
    Rng pos(seed, ST_POS, 1);
    int64_t total = 0;
    // occupancy grid for the unaligned variant: reject overlapping placements
    auto overlaps = [&](int64_t r0, int64_t c0) {
        for (const Block &b : blocks)
            if (std::llabs(b.r0 - r0) < BS && std::llabs(b.c0 - c0) < BS) return true;
        return false;
    };
    int64_t attempts = 0;
    while (total < target_nnz && static_cast<int64_t>(blocks.size()) < max_blocks && attempts < 64 * max_blocks + 1024) {
        ++attempts;
        int64_t r0, c0;
        if (unaligned) {
            r0 = static_cast<int64_t>(pos.below(static_cast<uint64_t>(M - BS + 1)));
            c0 = static_cast<int64_t>(pos.below(static_cast<uint64_t>(N - BS + 1)));
            if (overlaps(r0, c0)) continue;
        } else {
            const uint64_t cell = pos.below(static_cast<uint64_t>(gr * gc));
            if (!used.insert(cell).second) continue;
            r0 = static_cast<int64_t>(cell / static_cast<uint64_t>(gc)) * BS;
            c0 = static_cast<int64_t>(cell % static_cast<uint64_t>(gc)) * BS;
        }
        Block b;
        b.r0 = r0; b.c0 = c0; b.cnt = 0;
        Rng r(seed, ST_BLOCK, static_cast<uint64_t>(blocks.size()));
        for (int i = 0; i < BS; ++i) {
            uint64_t m = 0;
            for (int j = 0; j < BS; ++j)
                if (r.u01() < 0.70) m |= (1ull << j);
            b.rows[i] = m;
            b.cnt += __builtin_popcountll(m);
        }
        if (total + b.cnt > target_nnz) {  // trim the block that crosses the target (row-major order)
            int64_t keep = target_nnz - total, seen = 0;
            for (int i = 0; i < BS; ++i) {
                uint64_t m = b.rows[i], out = 0;
                for (int j = 0; j < BS; ++j)
                    if ((m >> j) & 1ull) {
                        if (seen < keep) { out |= (1ull << j); ++seen; }
                    }
                b.rows[i] = out;
            }
            b.cnt = keep;
        }
        total += b.cnt;
        blocks.push_back(b);
    }
    // assemble CSR: per row, blocks ordered by column origin
    std::vector<std::vector<int32_t>> by_row(static_cast<size_t>(M));  // block ids touching each row
    for (size_t bi = 0; bi < blocks.size(); ++bi)
        for (int i = 0; i < BS; ++i) by_row[static_cast<size_t>(blocks[bi].r0 + i)].push_back(static_cast<int32_t>(bi));
    std::vector<int32_t> len(static_cast<size_t>(M), 0);
    for (int64_t i = 0; i < M; ++i) {
        auto &v = by_row[static_cast<size_t>(i)];
        std::sort(v.begin(), v.end(), [&](int32_t x, int32_t y) { return blocks[static_cast<size_t>(x)].c0 < blocks[static_cast<size_t>(y)].c0; });
        int64_t n = 0;
        for (int32_t bi : v) n += __builtin_popcountll(blocks[static_cast<size_t>(bi)].rows[i - blocks[static_cast<size_t>(bi)].r0]);
        len[static_cast<size_t>(i)] = static_cast<int32_t>(n);
    }
    scan_lengths(len, d.row_ptr);
    d.col.resize(static_cast<size_t>(d.row_ptr.back()));
    parallel_for(M, [&](int64_t a, int64_t b, int) {
        for (int64_t i = a; i < b; ++i) {
            int32_t *out = d.col.data() + d.row_ptr[static_cast<size_t>(i)];
            for (int32_t bi : by_row[static_cast<size_t>(i)]) {
                const Block &blk = blocks[static_cast<size_t>(bi)];
                const uint64_t m = blk.rows[i - blk.r0];
                for (int j = 0; j < BS; ++j)
                    if ((m >> j) & 1ull) *out++ = static_cast<int32_t>(blk.c0 + j);
            }
        }
    });
    fill_values(d, seed, false);
}

// ---- config 3: dense 3x3 blocks inside a band -------------------------------------
void gen_banded(sddmm_dataset &d, double blocks_per_row, int64_t half_width, uint64_t seed) {
    const int64_t M = d.M, N = d.N;
    const int64_t nbr = (M + 2) / 3, nbc = (N + 2) / 3;
    const int64_t hw = std::max<int64_t>(1, half_width / 3);
    const int base = static_cast<int>(std::floor(blocks_per_row));
    const double frac = blocks_per_row - base;
    // block columns of every block row
    std::vector<int32_t> bptr(static_cast<size_t>(nbr + 1), 0);
    std::vector<int32_t> blen(static_cast<size_t>(nbr));
    for (int64_t bi = 0; bi < nbr; ++bi) {
        Rng r(seed, ST_LEN, static_cast<uint64_t>(bi));
        const int64_t lo = std::max<int64_t>(0, bi - hw), hi = std::min<int64_t>(nbc - 1, bi + hw);
        int want = base + (r.u01() < frac ? 1 : 0);
        want = static_cast<int>(std::min<int64_t>(want, hi - lo + 1));
        blen[static_cast<size_t>(bi)] = want;
    }
    for (int64_t bi = 0; bi < nbr; ++bi) bptr[static_cast<size_t>(bi + 1)] = bptr[static_cast<size_t>(bi)] + blen[static_cast<size_t>(bi)];
    std::vector<int32_t> bcol(static_cast<size_t>(bptr.back()));
    parallel_for(nbr, [&](int64_t a, int64_t b, int) {
        std::vector<int32_t> mark(static_cast<size_t>(nbc), -1);
        for (int64_t bi = a; bi < b; ++bi) {
            Rng r(seed, ST_COL, static_cast<uint64_t>(bi));
            const int64_t lo = std::max<int64_t>(0, bi - hw), hi = std::min<int64_t>(nbc - 1, bi + hw);
            int32_t *out = bcol.data() + bptr[static_cast<size_t>(bi)];
            int got = 0;
            const int want = blen[static_cast<size_t>(bi)];
            while (got < want) {
                const int64_t c = lo + static_cast<int64_t>(r.below(static_cast<uint64_t>(hi - lo + 1)));
                if (mark[static_cast<size_t>(c)] == static_cast<int32_t>(bi)) continue;
                mark[static_cast<size_t>(c)] = static_cast<int32_t>(bi);
                out[got++] = static_cast<int32_t>(c);
            }
            std::sort(out, out + want);
        }
    });
    std::vector<int32_t> len(static_cast<size_t>(M));
    for (int64_t i = 0; i < M; ++i) {
        const int64_t bi = i / 3;
        int64_t n = 0;
        for (int32_t t = bptr[static_cast<size_t>(bi)]; t < bptr[static_cast<size_t>(bi + 1)]; ++t) {
            const int64_t c0 = static_cast<int64_t>(bcol[static_cast<size_t>(t)]) * 3;
            n += std::min<int64_t>(3, N - c0);
        }
        len[static_cast<size_t>(i)] = static_cast<int32_t>(n);
    }
    scan_lengths(len, d.row_ptr);
    d.col.resize(static_cast<size_t>(d.row_ptr.back()));
    parallel_for(M, [&](int64_t a, int64_t b, int) {
        for (int64_t i = a; i < b; ++i) {
            const int64_t bi = i / 3;
            int32_t *out = d.col.data() + d.row_ptr[static_cast<size_t>(i)];
            for (int32_t t = bptr[static_cast<size_t>(bi)]; t < bptr[static_cast<size_t>(bi + 1)]; ++t) {
                const int64_t c0 = static_cast<int64_t>(bcol[static_cast<size_t>(t)]) * 3;
                for (int64_t c = c0; c < std::min<int64_t>(c0 + 3, N); ++c) *out++ = static_cast<int32_t>(c);
            }
        }
    });
    fill_values(d, seed, false);
}

// ---- config 4: Zipf(2) row lengths and Zipf(2) column popularity -------------------
void gen_powerlaw(sddmm_dataset &d, int64_t target_nnz, int64_t max_len, uint64_t seed) {
    const int64_t M = d.M, N = d.N;
    max_len = std::min(max_len, N);
    std::vector<int32_t> raw(static_cast<size_t>(M));
    parallel_for(M, [&](int64_t a, int64_t b, int) {
        for (int64_t i = a; i < b; ++i) {
            Rng r(seed, ST_LEN, static_cast<uint64_t>(i));
            raw[static_cast<size_t>(i)] = static_cast<int32_t>(zipf2(r, max_len));
        }
    });
    // The truncated Zipf(2) mean (~6.9 at max 50 000) is below the target mean
    // (~13.9): lengths are multiplied by the constant c that makes the total hit
    // the target, found by bisection; len = clamp(floor(c*raw + 0.5), 1, max_len).
    auto total_for = [&](double c) {
        int64_t t = 0;
        for (int64_t i = 0; i < M; ++i) {
            int64_t l = static_cast<int64_t>(c * raw[static_cast<size_t>(i)] + 0.5);
            t += std::max<int64_t>(1, std::min<int64_t>(max_len, l));
        }
        return t;
    };
    double lo = 0.0, hi = 64.0;
    for (int it = 0; it < 60; ++it) {
        const double mid = 0.5 * (lo + hi);
        if (total_for(mid) < target_nnz) lo = mid; else hi = mid;
    }
    const double c = hi;
    std::vector<int32_t> len(static_cast<size_t>(M));
    for (int64_t i = 0; i < M; ++i) {
        int64_t l = static_cast<int64_t>(c * raw[static_cast<size_t>(i)] + 0.5);
        len[static_cast<size_t>(i)] = static_cast<int32_t>(std::max<int64_t>(1, std::min<int64_t>(max_len, l)));
    }
    scan_lengths(len, d.row_ptr);
    // random permutation of the columns: popularity rank -> column id
    std::vector<int32_t> perm(static_cast<size_t>(N));
    for (int64_t i = 0; i < N; ++i) perm[static_cast<size_t>(i)] = static_cast<int32_t>(i);
    {
        Rng r(seed, ST_PERM, 0);
        for (int64_t i = N - 1; i > 0; --i) std::swap(perm[static_cast<size_t>(i)], perm[static_cast<size_t>(r.below(static_cast<uint64_t>(i + 1)))]);
    }
    fill_rows_distinct(d, len, seed, [&](Rng &r, int64_t) { return static_cast<int64_t>(perm[static_cast<size_t>(zipf2(r, N) - 1)]); });
    fill_values(d, seed, true);
}

// ---- config 5: Poisson row lengths, uniform columns ---------------------------------
void gen_poisson(sddmm_dataset &d, double lambda, uint64_t seed) {
    const int64_t M = d.M, N = d.N;
    std::vector<int32_t> len(static_cast<size_t>(M));
    parallel_for(M, [&](int64_t a, int64_t b, int) {
        for (int64_t i = a; i < b; ++i) {
            Rng r(seed, ST_LEN, static_cast<uint64_t>(i));
            len[static_cast<size_t>(i)] = static_cast<int32_t>(std::min<int64_t>(N, poisson(r, lambda)));
        }
    });
    scan_lengths(len, d.row_ptr);
    fill_rows_distinct(d, len, seed, [&](Rng &r, int64_t) { return static_cast<int64_t>(r.below(static_cast<uint64_t>(N))); });
    fill_values(d, seed, false);
}

}  // namespace

extern "C" {

int sddmm_dataset_create(sddmm_dataset **out, int config, int64_t K, double scale, uint64_t seed, int variant) {
    if (!out) return 1;
    *out = nullptr;
    if (config < 1 || config > 5 || K < 1 || !(scale > 0.0) || scale > 1.0) return 1;
    sddmm_dataset *d = new (std::nothrow) sddmm_dataset();
    if (!d) return 3;
    try {
        d->K = K;
        switch (config) {
            case 1:
                d->name = "small-uniform";
                d->M = d->N = scaled(656, scale, 8);
                gen_uniform(*d, static_cast<int64_t>(std::llround(18964.0 * (double(d->M) / 656.0) * (double(d->N) / 656.0))), seed);
                break;
            case 2: {
                d->name = variant == 1 ? "clustered-blocks-unaligned" : "clustered-blocks";
                d->M = d->N = scaled(14340, scale, 128);
                const double dens = 18.07e6 / (14340.0 * 14340.0);
                gen_blocks(*d, static_cast<int64_t>(std::llround(dens * double(d->M) * double(d->N))), seed, variant == 1);
                break;
            }
            case 3:
                d->name = "banded-3x3";
                d->M = d->N = scaled(503712, scale, 96) / 3 * 3;
                gen_banded(*d, 36.8e6 / 9.0 / (503712.0 / 3.0), 2000, seed);
                break;
            case 4:
                d->name = "power-law";
                d->M = d->N = scaled(2601977, scale, 64);
                gen_powerlaw(*d, static_cast<int64_t>(std::llround(36.2e6 * double(d->M) / 2601977.0)), 50000, seed);
                break;
            case 5:
                d->name = "poisson-rows";
                d->M = d->N = scaled(1453908, scale, 64);
                gen_poisson(*d, 37.5e6 / 1453908.0, seed);
                break;
        }
        fill_dense(*d, seed);
    } catch (const std::bad_alloc &) {
        delete d;
        return 3;
    }
    *out = d;
    return 0;
}

int sddmm_dataset_create_uniform(sddmm_dataset **out, int64_t M, int64_t N, int64_t K, int64_t nnz, uint64_t seed) {
    if (!out) return 1;
    *out = nullptr;
    if (M < 1 || N < 1 || K < 1 || nnz < 0) return 1;
    sddmm_dataset *d = new (std::nothrow) sddmm_dataset();
    if (!d) return 3;
    try {
        d->name = "uniform";
        d->M = M; d->N = N; d->K = K;
        gen_uniform(*d, nnz, seed);
        fill_dense(*d, seed);
    } catch (const std::bad_alloc &) {
        delete d;
        return 3;
    }
    *out = d;
    return 0;
}

void sddmm_dataset_destroy(sddmm_dataset *ds) { delete ds; }

void sddmm_dataset_dims(const sddmm_dataset *ds, int64_t *M, int64_t *N, int64_t *K, int64_t *nnz) {
    if (M) *M = ds->M;
    if (N) *N = ds->N;
    if (K) *K = ds->K;
    if (nnz) *nnz = static_cast<int64_t>(ds->col.size());
}
const char *sddmm_dataset_name(const sddmm_dataset *ds) { return ds->name.c_str(); }
const int32_t *sddmm_dataset_row_ptr(const sddmm_dataset *ds) { return ds->row_ptr.data(); }
const int32_t *sddmm_dataset_col_idx(const sddmm_dataset *ds) { return ds->col.data(); }
const float *sddmm_dataset_s_val(const sddmm_dataset *ds) { return ds->val.data(); }
const float *sddmm_dataset_A(const sddmm_dataset *ds) { return ds->A.data(); }
const float *sddmm_dataset_B(const sddmm_dataset *ds) { return ds->B.data(); }

}  // extern "C"
