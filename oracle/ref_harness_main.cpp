// Test infrastructure, never the product path: the GPU-B200 competitor run by the reference's OWN, UNMODIFIED
// benchmark harness.
//
// This file is compiled only where the reference checkout is present (recipe: oracle/build.py,
// build_ref_harness), against the reference's headers where they lie -- its SDDMM::Benchmark<T>
// (src/benchmark/benchmark.hpp:45-190), its datasets (src/benchmark/dataset.hpp: DummyDataset :183-204,
// RandomWithDensityDataset :332-356, LatinHypercubeDataset :359-378), its CPU-Basic competitor
// (src/competitors/cpu/cpu_basic.hpp) as the first competitor, i.e. the correctness baseline
// (benchmark.hpp:50-61) -- plus this repository's competitor header and C-ABI library.  Nothing of the
// reference is copied: the only sources of this repository in the translation unit are
// competitors/gpu/gpu_b200.hpp and include/sddmm_b200.h.
//
// It prints the harness' CSV rows (competitor,dataset,mat_repr,M,N,K,NZ,total_ns,init_ns,comp_ns,cleanup_ns,
// correctness,...) and, last, one line "entry_device_kept=<0|1>": the harness records its CUDA events on the
// default stream of the device that is current when it runs, so a competitor must leave that device current.
#include <memory>
#include <vector>

#include "benchmark/benchmark.hpp"
#include "competitors/cpu/cpu_basic.hpp"
#include "competitors/gpu/gpu_b200.hpp"

int main(int argc, char **argv) {
    const int runs = argc > 1 ? std::atoi(argv[1]) : 2;
    int dev_before = -1, dev_after = -2;
    cudaGetDevice(&dev_before);
    std::vector<std::shared_ptr<SDDMM::Competitor<float>>> competitors;
    competitors.push_back(std::make_shared<Competitors::CPUBasic<float>>());
    competitors.push_back(std::make_shared<Competitors::GPUB200>(SDDMM_B200_FP32, 0, "GPU-B200"));
    competitors.push_back(std::make_shared<Competitors::GPUB200>(SDDMM_B200_FP32_TC, 0, "GPU-B200-fp32_tc"));
    {
        SDDMM::DummyDataset d;
        SDDMM::Benchmark<float>(d, competitors, "", runs).benchmark();
    }
    {
        SDDMM::RandomWithDensityDataset<float> d(500, 400, 32, 0.05);
        SDDMM::Benchmark<float>(d, competitors, "", runs).benchmark();
    }
    {
        SDDMM::RandomWithDensityDataset<float> d(256, 256, 64, 0.7);   // dense enough for the tensor-core tiles
        SDDMM::Benchmark<float>(d, competitors, "", runs).benchmark();
    }
    {
        SDDMM::LatinHypercubeDataset<float> d(3000, 3000, 32);
        SDDMM::Benchmark<float>(d, competitors, "", runs).benchmark();
    }
    cudaGetDevice(&dev_after);
    std::cout << "entry_device_kept=" << (dev_before == dev_after ? 1 : 0) << std::endl;
    return 0;
}
