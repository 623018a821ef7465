// Benchmark harness: runs every competitor on one dataset in CSR and in COO form, times the three
// phases (init / compute / cleanup), verifies against the expected P and prints one CSV row per run.
// Same flow and CSV schema as the reference's SDDMM::Benchmark<T> (src/benchmark/benchmark.hpp:45-190;
// schema: src/main.cpp:355-358) so its plot scripts read the output unchanged:
//   competitor,dataset,mat_repr,M,N,K,NZ,total_ns,init_ns,comp_ns,cleanup_ns,correctness,num_thread_blocks,num_threads_per_block
// Timing: host clock around each phase; a GPU competitor's compute phase is taken from the device
// (its own CUDA events around its kernels) when it implements SDDMM::DeviceTimed, since the
// reference's event pair on the legacy default stream (:160-164) cannot see another stream.
// The harness names no concrete competitor.
// If the dataset carries no expected result, the first competitor provides it (reference: :50-61).
#pragma once
#include <chrono>
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "competitor.hpp"
#include "competitors/gpu/device_timed.hpp"
#include "dataset.hpp"
#include "utils/util.hpp"

namespace SDDMM {

struct timing_result {
    uint64_t init_ns, comp_ns, cleanup_ns, total_ns;
};

template <typename T>
class Benchmark {
public:
    Benchmark(Dataset<T> &dataset, std::vector<std::shared_ptr<Competitor<T>>> &competitors, int num_runs)
        : dataset(dataset), competitors(competitors), num_runs(num_runs) {}

    Dataset<T> &getDataset() { return dataset; }

    static const char *csv_header() {
        return "competitor,dataset,mat_repr,M,N,K,NZ,total_ns,init_ns,comp_ns,cleanup_ns,correctness,num_thread_blocks,num_threads_per_block";
    }

    // returns the number of runs whose result did not match
    int benchmark() {
        int mismatches = 0;
        Dataset<T> &d = dataset;
        if (!d.hasExpected()) {
            auto *ref = competitors.front().get();
            CSR<T> P(d.getS_CSR());
            P.clearValues();
            ref->init_csr(d.getA(), d.getB(), d.getS_CSR(), P);
            ref->run_csr(d.getA(), d.getB(), d.getS_CSR(), P);
            ref->cleanup_csr(d.getA(), d.getB(), d.getS_CSR(), P);
            d.setExpected_CSR(P);
        }
        for (auto &cp : competitors) {
            Competitor<T> *c = cp.get();
            if (c->csr_supported()) {
                for (int run = 0; run < num_runs; ++run) {
                    CSR<T> P(d.getS_CSR());
                    P.clearValues();
                    const timing_result t = timing(c, [&] { c->init_csr(d.getA(), d.getB(), d.getS_CSR(), P); },
                                                   [&] { c->run_csr(d.getA(), d.getB(), d.getS_CSR(), P); },
                                                   [&] { c->cleanup_csr(d.getA(), d.getB(), d.getS_CSR(), P); });
                    const bool ok = (P == d.getExpected_CSR());
                    mismatches += ok ? 0 : 1;
                    row(c, "CSR", t, ok);
                }
            }
            if (c->coo_supported()) {
                for (int run = 0; run < num_runs; ++run) {
                    COO<T> P(d.getS_COO());
                    P.clearValues();
                    const timing_result t = timing(c, [&] { c->init_coo(d.getA(), d.getB(), d.getS_COO(), P); },
                                                   [&] { c->run_coo(d.getA(), d.getB(), d.getS_COO(), P); },
                                                   [&] { c->cleanup_coo(d.getA(), d.getB(), d.getS_COO(), P); });
                    const bool ok = (P == d.getExpected_COO());
                    mismatches += ok ? 0 : 1;
                    row(c, "COO", t, ok);
                }
            }
        }
        return mismatches;
    }

private:
    Dataset<T> &dataset;
    std::vector<std::shared_ptr<Competitor<T>>> &competitors;
    int num_runs;

    using clk = std::chrono::high_resolution_clock;
    static uint64_t ns(clk::time_point a, clk::time_point b) {
        return static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(b - a).count());
    }

    timing_result timing(Competitor<T> *c, const std::function<void()> &init, const std::function<void()> &comp,
                         const std::function<void()> &cleanup) {
        const auto t0 = clk::now();
        init();
        const auto t1 = clk::now();
        comp();
        const auto t2 = clk::now();
        timing_result r;
        r.comp_ns = ns(t1, t2);
        if (c->is_gpu()) {
            float ms = 0.f;   // the competitor's own device time, if it offers one, instead of the host clock around run_*
            if (auto *timed = dynamic_cast<DeviceTimed *>(c)) ms = timed->last_kernel_ms();
            if (ms > 0.f) r.comp_ns = static_cast<uint64_t>(static_cast<double>(ms) * 1e6);
        }
        cleanup();
        const auto t3 = clk::now();
        r.init_ns = ns(t0, t1);
        r.cleanup_ns = ns(t2, t3);
        r.total_ns = ns(t0, t3);
        return r;
    }

    void row(Competitor<T> *c, const char *repr, const timing_result &t, bool ok) {
        Dataset<T> &d = dataset;
        FILE_DUMP(c->name << "," << d.getName() << "," << repr << "," << d.getS_COO().getRows() << "," << d.getS_COO().getCols() << ","
                          << d.getA().getCols() << "," << d.getS_COO().getValues().size() << "," << t.total_ns << "," << t.init_ns << ","
                          << t.comp_ns << "," << t.cleanup_ns << "," << (ok ? 1 : 0) << "," << c->get_num_thread_blocks() << ","
                          << c->get_num_threads_per_block() << std::endl);
    }
};

}  // namespace SDDMM
