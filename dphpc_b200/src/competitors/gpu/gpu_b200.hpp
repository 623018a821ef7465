// GPU-B200: the B200-native SDDMM engine behind the reference's competitor
// interface (SDDMM::Competitor<float>, src/benchmark/competitor.hpp:13-60), so it
// registers next to the existing competitors exactly like e.g. GPUConvert
// (src/competitors/gpu/gpu_convert.hpp; registration: src/main.cpp:18-56):
//
//     competitors.push_back(std::make_shared<Competitors::GPUB200>());
//
// The class is host-only C++: all CUDA lives behind the C ABI of include/sddmm_b200.h
// (link with -lsddmm_b200).  It compiles unchanged against the reference's own
// headers (-I<reference>/src) or against the interface mirror shipped here.
//
//   init_*     upload S, A, B (H2D) -- validation, histogram and kernel plan are built on the device
//   run_*      enqueue the kernels and wait (synchronous, like every reference GPU competitor)
//   cleanup_*  download P.val (D2H) while helper threads copy S's pattern into P (as gpu_convert.hpp:58-64 does)
//
// Errors never throw across the harness: they are printed to std::cerr and P keeps
// whatever it held, which the harness reports as correctness = 0 -- the reference's
// own convention (e.g. src/competitors/gpu/gpu_basic.cu:77-80).
#pragma once
#include <iostream>
#include <string>

#include "benchmark/competitor.hpp"
#include "device_timed.hpp"
#include "matrices/matrices.h"
#include "pattern_copy.hpp"
#include "sddmm_b200.h"

namespace Competitors {

class GPUB200 : public SDDMM::Competitor<float>, public SDDMM::DeviceTimed {
    using T = float;

public:
    // mode: SDDMM_B200_FP32 / _TF32 / _BF16 / _FP32_TC; device: CUDA ordinal; flags: SDDMM_B200_FLAG_* (paths to switch off)
    explicit GPUB200(int mode = SDDMM_B200_FP32, int device = 0, const std::string &name = "GPU-B200", uint32_t flags = 0)
        : SDDMM::Competitor<T>(name), mode_(mode), device_(device), flags_(flags) {}

    // (the reference's base class has a non-virtual destructor: hold competitors through make_shared, as its main.cpp does)
    ~GPUB200() { sddmm_b200_destroy(engine_); }
    GPUB200(const GPUB200 &) = delete;
    GPUB200 &operator=(const GPUB200 &) = delete;

    void init_csr(Dense<T> &A, Dense<T> &B, CSR<T> &S, CSR<T> &) override {
        if (!ensure_engine()) return;
        const int st = sddmm_b200_upload_csr(engine_, A.getRows(), B.getRows(), A.getCols(), S.getRowPositions().data(),
                                             S.getColPositions().data(), S.getValues().data(), A.get_pointer(), B.get_pointer());
        after_upload(st);
    }

    void init_coo(Dense<T> &A, Dense<T> &B, COO<T> &S, COO<T> &) override {
        if (!ensure_engine()) return;
        const int st = sddmm_b200_upload_coo(engine_, A.getRows(), B.getRows(), A.getCols(), static_cast<int64_t>(S.getValues().size()),
                                             S.getRowPositions().data(), S.getColPositions().data(), S.getValues().data(),
                                             A.get_pointer(), B.get_pointer());
        after_upload(st);
    }

    void run_csr(Dense<T> &, Dense<T> &, CSR<T> &, CSR<T> &) override { run(); }
    void run_coo(Dense<T> &, Dense<T> &, COO<T> &, COO<T> &) override { run(); }

    void cleanup_csr(Dense<T> &, Dense<T> &, CSR<T> &S, CSR<T> &P) override {
        if (!ready_) return;
        SDDMM::finish_into(S, P, [&](T *values) { report(sddmm_b200_download(engine_, values), "download"); });
    }

    void cleanup_coo(Dense<T> &, Dense<T> &, COO<T> &S, COO<T> &P) override {
        if (!ready_) return;
        SDDMM::finish_into(S, P, [&](T *values) { report(sddmm_b200_download(engine_, values), "download"); });
    }

    bool csr_supported() override { return true; }
    bool coo_supported() override { return true; }
    bool is_gpu() override { return true; }

    // device time of the kernels of the last run_* (ms); the harness' own event pair also sees launch overhead
    float last_kernel_ms() override {
        float ms = 0.f;
        if (ready_) sddmm_b200_last_run_ms(engine_, &ms);
        return ms;
    }
    sddmm_b200_engine *engine() { return engine_; }

private:
    int mode_, device_;
    uint32_t flags_;
    sddmm_b200_engine *engine_ = nullptr;
    bool ready_ = false;

    bool ensure_engine() {
        ready_ = false;
        if (engine_) return true;
        const int st = sddmm_b200_create(&engine_, device_, mode_, flags_);
        if (st != SDDMM_B200_OK) {
            std::cerr << "[" << name << "] cannot create the engine (status " << st << "): no usable CUDA device?" << std::endl;
            engine_ = nullptr;
            return false;
        }
        return true;
    }

    void after_upload(int st) {
        ready_ = report(st, "upload");
        if (!ready_) return;
        sddmm_b200_plan_info info;
        if (sddmm_b200_get_plan(engine_, &info) == SDDMM_B200_OK) {
            set_num_thread_blocks(info.dense_tiles > 0 ? info.dense_grid : info.rowgroup_rows > 0 ? info.rowgroup_grid
                                  : info.rowseg_units > 0 ? info.rowseg_grid : info.rowtile_grid);
            set_num_threads_per_block(info.dense_tiles > 0 ? info.dense_block : info.rowtile_block);
        }
    }

    void run() {
        if (!ready_) return;
        if (report(sddmm_b200_run(engine_), "run")) report(sddmm_b200_sync(engine_), "sync");
    }

    bool report(int st, const char *what) {
        if (st == SDDMM_B200_OK) return true;
        std::cerr << "[" << name << "] " << what << " failed (status " << st << "): " << sddmm_b200_last_error(engine_) << std::endl;
        return false;
    }
};

}  // namespace Competitors
