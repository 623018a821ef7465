// GPU-B200 on several GPUs of one box, behind the same competitor interface
// (SDDMM::Competitor<float>, src/benchmark/competitor.hpp:13-60) and from ONE host process:
//
//     competitors.push_back(std::make_shared<Competitors::GPUB200Multi>());          // every visible GPU
//     competitors.push_back(std::make_shared<Competitors::GPUB200Multi>(std::vector<int>{0, 1}));
//
// SDDMM has no exchange step: every output nonzero needs one row of A, one row of B and one value of S.
// So the rows of S are cut into contiguous ranges with equal shares of the nonzeros (the cut nearest to
// g * nnz / G; rounded to 64 rows when the matrix is large, so that every shard keeps the 64x64 tile grid
// of the tensor-core path), device g gets its range of S and A and all of B, and the P slices come back
// into disjoint ranges of the host P.values.  The reference's dispatcher (`CSR::_dispatch`,
// src/matrices/CSR.hpp:214-264) balances nonzeros over thread blocks the same way.
//
// One engine (include/sddmm_b200.h) per device.  B crosses the host link once and is then copied device to
// device (sddmm_b200_stage_b: NVLink between peers, log2(G) rounds); the shards of S and A go up on one helper
// thread per device (they share the host but not a stream); the threads are joined before every member returns.
// A listed device that does not exist is left out with a message: the competitor then runs on the devices that do.
// run_* enqueues on every device, then waits for all of them; the caller's current device is left as it was.
// A device may be listed more than once (two engines on one GPU): the sharding logic is then testable
// on a single-GPU machine.
#pragma once
#include <algorithm>
#include <cstdint>
#include <iostream>
#include <string>
#include <thread>
#include <vector>

#include "benchmark/competitor.hpp"
#include "device_timed.hpp"
#include "matrices/matrices.h"
#include "pattern_copy.hpp"
#include "sddmm_b200.h"

namespace Competitors {

class GPUB200Multi : public SDDMM::Competitor<float>, public SDDMM::DeviceTimed {
    using T = float;

public:
    // devices: CUDA ordinals, one engine each; empty = every visible device
    explicit GPUB200Multi(std::vector<int> devices = {}, int mode = SDDMM_B200_FP32, const std::string &name = "GPU-B200-multi",
                          uint32_t flags = 0)
        : SDDMM::Competitor<T>(name), devices_(std::move(devices)), mode_(mode), flags_(flags) {}

    ~GPUB200Multi() {
        for (sddmm_b200_engine *e : engines_) sddmm_b200_destroy(e);
    }
    GPUB200Multi(const GPUB200Multi &) = delete;
    GPUB200Multi &operator=(const GPUB200Multi &) = delete;

    // first row of every shard (size shards + 1): sddmm_b200_row_cuts, the one definition every sharded path uses
    static std::vector<int64_t> row_cuts(const std::vector<int> &row_ptr, int parts, int64_t align = 1) {
        std::vector<int64_t> cuts(static_cast<size_t>(parts) + 1, 0);
        sddmm_b200_row_cuts(row_ptr.data(), static_cast<int64_t>(row_ptr.size()) - 1, parts, align, cuts.data());
        return cuts;
    }

    void init_csr(Dense<T> &A, Dense<T> &B, CSR<T> &S, CSR<T> &) override {
        if (!ensure_engines()) return;
        const int64_t M = A.getRows(), N = B.getRows(), K = A.getCols();
        const std::vector<int> &rp = S.getRowPositions();
        plan_shards(rp, M);
        if (!stage_b(N, K, B.get_pointer())) return;
        std::vector<int> status(shards(), SDDMM_B200_OK);
        parallel([&](int g) {
            const int64_t r0 = cuts_[static_cast<size_t>(g)], r1 = cuts_[static_cast<size_t>(g) + 1];
            const int64_t off = rp[static_cast<size_t>(r0)];
            std::vector<int32_t> local(static_cast<size_t>(r1 - r0) + 1);
            for (int64_t i = r0; i <= r1; ++i) local[static_cast<size_t>(i - r0)] = static_cast<int32_t>(rp[static_cast<size_t>(i)] - off);
            if (r1 == r0) return;   // an empty shard keeps its engine idle
            status[static_cast<size_t>(g)] = sddmm_b200_upload_csr(engines_[static_cast<size_t>(g)], r1 - r0, N, K, local.data(),
                                                                    S.getColPositions().data() + off, S.getValues().data() + off,
                                                                    A.get_pointer() + r0 * K, nullptr /* the staged B */);
        });
        after_upload(status);
    }

    void init_coo(Dense<T> &A, Dense<T> &B, COO<T> &S, COO<T> &) override {
        if (!ensure_engines()) return;
        const int64_t M = A.getRows(), N = B.getRows(), K = A.getCols();
        const std::vector<int> &rows = S.getRowPositions();   // sorted by row (src/matrices/COO.hpp:39)
        const int64_t nnz = static_cast<int64_t>(rows.size());
        // cuts and slice offsets straight from the sorted row array; every shard uploads its slice of the caller's arrays
        // as they are and its device subtracts the shard's first row (no row_ptr, no rewritten copy on the host)
        offsets_.assign(static_cast<size_t>(shards()) + 1, 0);
        cuts_.assign(static_cast<size_t>(shards()) + 1, 0);
        const int64_t align = M >= int64_t(64) * 8 * shards() ? 64 : 1;
        if (sddmm_b200_coo_cuts(rows.data(), nnz, M, shards(), align, cuts_.data(), offsets_.data()) != SDDMM_B200_OK) {
            std::cerr << "[" << name << "] COO row indices must be sorted and inside [0, M)" << std::endl;
            return;
        }
        if (!stage_b(N, K, B.get_pointer())) return;
        std::vector<int> status(shards(), SDDMM_B200_OK);
        parallel([&](int g) {
            const int64_t r0 = cuts_[static_cast<size_t>(g)], r1 = cuts_[static_cast<size_t>(g) + 1];
            const int64_t off = offsets_[static_cast<size_t>(g)], n = offsets_[static_cast<size_t>(g) + 1] - off;
            if (r1 == r0) return;
            status[static_cast<size_t>(g)] = sddmm_b200_upload_coo_rows(engines_[static_cast<size_t>(g)], r1 - r0, N, K, n, r0, rows.data() + off,
                                                                         S.getColPositions().data() + off, S.getValues().data() + off,
                                                                         A.get_pointer() + r0 * K, nullptr /* the staged B */);
        });
        after_upload(status);
    }

    void run_csr(Dense<T> &, Dense<T> &, CSR<T> &, CSR<T> &) override { run(); }
    void run_coo(Dense<T> &, Dense<T> &, COO<T> &, COO<T> &) override { run(); }

    void cleanup_csr(Dense<T> &, Dense<T> &, CSR<T> &S, CSR<T> &P) override {
        if (!ready_) return;
        SDDMM::finish_into(S, P, [&](T *values) { download(values); });
    }

    void cleanup_coo(Dense<T> &, Dense<T> &, COO<T> &S, COO<T> &P) override {
        if (!ready_) return;
        SDDMM::finish_into(S, P, [&](T *values) { download(values); });
    }

    bool csr_supported() override { return true; }
    bool coo_supported() override { return true; }
    bool is_gpu() override { return true; }

    int shards() const { return static_cast<int>(engines_.size()); }
    const std::vector<int64_t> &cuts() const { return cuts_; }        // rows of shard g: [cuts[g], cuts[g+1])
    // device time of the slowest shard in the last run_* (ms)
    float last_kernel_ms() override {
        float worst = 0.f;
        for (int g = 0; ready_ && g < shards(); ++g) {
            float ms = 0.f;
            if (active(g) && sddmm_b200_last_run_ms(engines_[static_cast<size_t>(g)], &ms) == SDDMM_B200_OK) worst = std::max(worst, ms);
        }
        return worst;
    }

private:
    std::vector<int> devices_;
    int mode_;
    uint32_t flags_;
    std::vector<sddmm_b200_engine *> engines_;
    std::vector<int64_t> cuts_;      // row cuts of the current upload
    std::vector<int64_t> offsets_;   // first nonzero of every shard (size shards + 1)
    bool ready_ = false;

    bool active(int g) const { return cuts_[static_cast<size_t>(g) + 1] > cuts_[static_cast<size_t>(g)]; }

    bool ensure_engines() {
        ready_ = false;
        if (!engines_.empty()) return true;
        if (devices_.empty()) {
            const int n = sddmm_b200_device_count();
            for (int d = 0; d < n; ++d) devices_.push_back(d);
        }
        const int present = sddmm_b200_device_count();
        for (int d : devices_) {
            if (d < 0 || d >= present) {   // fewer devices than asked for: go on with those that exist
                std::cerr << "[" << name << "] device " << d << " does not exist (" << present << " visible): left out" << std::endl;
                continue;
            }
            sddmm_b200_engine *e = nullptr;
            const int st = sddmm_b200_create(&e, d, mode_, flags_);
            if (st != SDDMM_B200_OK) {
                std::cerr << "[" << name << "] cannot create the engine on device " << d << " (status " << st << ")" << std::endl;
                for (sddmm_b200_engine *x : engines_) sddmm_b200_destroy(x);
                engines_.clear();
                return false;
            }
            engines_.push_back(e);
        }
        if (engines_.empty()) std::cerr << "[" << name << "] no CUDA device" << std::endl;
        return !engines_.empty();
    }

    // B to every device: once over the host link, then device to device
    bool stage_b(int64_t N, int64_t K, const T *B) {
        const int st = sddmm_b200_stage_b(engines_.data(), shards(), N, K, B);
        if (st == SDDMM_B200_OK) return true;
        std::cerr << "[" << name << "] distributing B failed (status " << st << ")";
        for (sddmm_b200_engine *e : engines_)
            if (*sddmm_b200_last_error(e)) { std::cerr << ": " << sddmm_b200_last_error(e); break; }
        std::cerr << std::endl;
        return false;
    }

    void plan_shards(const std::vector<int> &rp, int64_t M) {
        const int G = shards();
        cuts_ = row_cuts(rp, G, M >= int64_t(64) * 8 * G ? 64 : 1);
        offsets_.assign(static_cast<size_t>(G) + 1, 0);
        for (int g = 0; g <= G; ++g) offsets_[static_cast<size_t>(g)] = rp[static_cast<size_t>(cuts_[static_cast<size_t>(g)])];
    }

    template <typename F>
    void parallel(F f) {   // one helper thread per shard, all joined before returning
        std::vector<std::thread> threads;
        for (int g = 1; g < shards(); ++g) threads.emplace_back(f, g);
        f(0);
        for (std::thread &t : threads) t.join();
    }

    void after_upload(const std::vector<int> &status) {
        ready_ = true;
        for (int g = 0; g < shards(); ++g) ready_ = report(status[static_cast<size_t>(g)], "upload", g) && ready_;
        if (!ready_) return;
        int blocks = 0, threads = 0;
        for (int g = 0; g < shards(); ++g) {
            sddmm_b200_plan_info info;
            if (active(g) && sddmm_b200_get_plan(engines_[static_cast<size_t>(g)], &info) == SDDMM_B200_OK) {
                blocks += info.dense_tiles > 0 ? info.dense_grid : info.rowgroup_rows > 0 ? info.rowgroup_grid
                          : info.rowseg_units > 0 ? info.rowseg_grid : info.rowtile_grid;
                threads = info.dense_tiles > 0 ? info.dense_block : info.rowtile_block;
            }
        }
        set_num_thread_blocks(blocks);
        set_num_threads_per_block(threads);
    }

    void run() {
        if (!ready_) return;
        for (int g = 0; g < shards(); ++g)
            if (active(g)) report(sddmm_b200_run(engines_[static_cast<size_t>(g)]), "run", g);
        for (int g = 0; g < shards(); ++g)
            if (active(g)) report(sddmm_b200_sync(engines_[static_cast<size_t>(g)]), "sync", g);
    }

    void download(T *p_val) {
        std::vector<int> status(shards(), SDDMM_B200_OK);
        parallel([&](int g) {
            if (active(g)) status[static_cast<size_t>(g)] = sddmm_b200_download(engines_[static_cast<size_t>(g)], p_val + offsets_[static_cast<size_t>(g)]);
        });
        for (int g = 0; g < shards(); ++g) report(status[static_cast<size_t>(g)], "download", g);
    }

    bool report(int st, const char *what, int g) {
        if (st == SDDMM_B200_OK) return true;
        std::cerr << "[" << name << "] " << what << " failed on shard " << g << " (status " << st << "): "
                  << sddmm_b200_last_error(engines_[static_cast<size_t>(g)]) << std::endl;
        return false;
    }
};

}  // namespace Competitors
