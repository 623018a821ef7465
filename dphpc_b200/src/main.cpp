// sddmm_bench: benchmark driver for the GPU-B200 competitor on the seeded synthetic configurations or on a matrix file.
// Command line of the reference's driver (src/main.cpp:285-349: --K/-k, --no_csv_header, --num_runs;
// --data_folder is accepted and ignored) plus --config, --scale, --mode, and --mtx FILE (MatrixMarket coordinate file) or
// --edges FILE --rows M --cols N (SNAP edge list), read with the reference's rules (src/benchmark/dataset.hpp:122-181, 270-313);
// --multi adds the row-sharded competitor that uses every visible GPU from this one process.
// The first competitor is the correctness baseline of the harness (src/benchmark/benchmark.hpp:50-61): CPU-Basic, as in
// the reference's driver (src/main.cpp:18-20), so every GPU row's `correctness` is a comparison with the host
// computation.  --no_cpu drops it (the baseline is then GPU-B200 in fp32 mode and the column only says that the
// other modes agree with it).
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <memory>
#include <string>
#include <vector>

#include "benchmark/benchmark.hpp"
#include "competitors/cpu/cpu_check.hpp"
#include "competitors/gpu/gpu_b200.hpp"
#include "competitors/gpu/gpu_b200_multi.hpp"

namespace {

struct Options {
    int K = 0, num_runs = 3, config = 0, variant = 0, rows = 0, cols = 0;
    std::string mtx, edges;
    double scale = 1.0;
    bool header = true;
    bool multi = false;   // also run the row-sharded competitor on every visible GPU
    bool cpu = true;      // CPU-Basic first: the correctness baseline
    std::vector<std::string> modes{"fp32", "fp32_tc"};   // tf32 / bf16 on request: their 1e-2 error fails the 1e-3 check
};

int mode_id(const std::string &m) {
    if (m == "fp32") return SDDMM_B200_FP32;
    if (m == "tf32") return SDDMM_B200_TF32;
    if (m == "bf16") return SDDMM_B200_BF16;
    if (m == "fp32_tc") return SDDMM_B200_FP32_TC;
    return -1;
}

void usage() {
    std::cerr << "usage: sddmm_bench [--config 1..5 (default: all) | --mtx FILE | --edges FILE --rows M --cols N] [-k K] [--num_runs R] [--scale s]"
                 " [--mode fp32,tf32,...] [--multi] [--no_cpu] [--no_csv_header]\n";
}

}  // namespace

int main(int argc, char **argv) {
    Options o;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto next = [&]() -> const char * { return (i + 1 < argc) ? argv[++i] : ""; };
        if (a == "-k" || a == "--K") o.K = std::atoi(next());
        else if (a == "--num_runs") o.num_runs = std::atoi(next());
        else if (a == "--config") o.config = std::atoi(next());
        else if (a == "--variant") o.variant = std::atoi(next());
        else if (a == "--mtx") o.mtx = next();
        else if (a == "--edges") o.edges = next();
        else if (a == "--rows") o.rows = std::atoi(next());
        else if (a == "--cols") o.cols = std::atoi(next());
        else if (a == "--scale") o.scale = std::atof(next());
        else if (a == "--no_csv_header") o.header = false;
        else if (a == "--multi") o.multi = true;
        else if (a == "--no_cpu") o.cpu = false;
        else if (a == "-d" || a == "--data_folder") next();
        else if (a == "--mode") {
            o.modes.clear();
            std::string list = next(), item;
            for (size_t p = 0; p <= list.size(); ++p) {
                if (p == list.size() || list[p] == ',') { if (!item.empty()) o.modes.push_back(item); item.clear(); }
                else item += list[p];
            }
        } else { usage(); return 2; }
    }
    if (sddmm_b200_device_count() < 1) {
        std::cerr << "sddmm_bench: no CUDA device; the engine has no CPU path" << std::endl;
        return 1;
    }
    std::vector<std::shared_ptr<SDDMM::Competitor<float>>> competitors;
    if (o.cpu) competitors.push_back(std::make_shared<Competitors::CPUCheck>());
    competitors.push_back(std::make_shared<Competitors::GPUB200>(SDDMM_B200_FP32, 0, "GPU-B200"));
    for (const std::string &m : o.modes) {
        const int id = mode_id(m);
        if (id < 0) { usage(); return 2; }
        if (id != SDDMM_B200_FP32) competitors.push_back(std::make_shared<Competitors::GPUB200>(id, 0, "GPU-B200-" + m));
    }
    if (o.multi) {
        const int n = sddmm_b200_device_count();
        for (const std::string &m : o.modes)
            competitors.push_back(std::make_shared<Competitors::GPUB200Multi>(std::vector<int>{}, mode_id(m), "GPU-B200-" + m + "-x" + std::to_string(n)));
    }
    if (o.header) FILE_DUMP(SDDMM::Benchmark<float>::csv_header() << std::endl);
    const int default_k[6] = {0, 32, 32, 64, 32, 32};
    int bad = 0;
    if (!o.mtx.empty() || !o.edges.empty()) {   // one matrix file instead of the synthetic configurations
        try {
            const int K = o.K ? o.K : 32;
            if (!o.mtx.empty()) {
                SDDMM::MatrixMarketDataset d(o.mtx, o.mtx, K);
                bad = SDDMM::Benchmark<float>(d, competitors, o.num_runs).benchmark();
            } else {
                if (o.rows < 1 || o.cols < 1) { usage(); return 2; }
                SDDMM::EdgeListDataset d(o.edges, o.edges, o.rows, o.cols, K);
                bad = SDDMM::Benchmark<float>(d, competitors, o.num_runs).benchmark();
            }
        } catch (const std::exception &e) {
            std::cerr << "sddmm_bench: " << e.what() << std::endl;
            return 2;
        }
        return bad ? 3 : 0;
    }
    for (int cfg = 1; cfg <= 5; ++cfg) {
        if (o.config && cfg != o.config) continue;
        SDDMM::SyntheticDataset d(cfg, o.K ? o.K : default_k[cfg], o.scale, 0, o.variant);
        SDDMM::Benchmark<float> b(d, competitors, o.num_runs);
        bad += b.benchmark();
    }
    return bad ? 3 : 0;
}
