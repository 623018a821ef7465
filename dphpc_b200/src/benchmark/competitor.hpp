// The plug-in interface every SDDMM implementation sits behind: the same virtual
// surface as the reference's SDDMM::Competitor<T> (src/benchmark/competitor.hpp:13-60) --
// init_* (uploads / preprocessing), run_* (the timed computation), cleanup_*
// (download / release) for CSR and COO, capability queries, is_gpu() (selects CUDA
// event timing in the harness) and the launch shape reported in the CSV.
#pragma once
#include <string>

#include "matrices/matrices.h"

namespace SDDMM {

template <typename T>
class Competitor {
public:
    const std::string name;

    explicit Competitor(const std::string &name) : name(name) {}
    Competitor(const std::string &name, int threads_per_block, int thread_blocks)
        : name(name), threads_per_block(threads_per_block), thread_blocks(thread_blocks) {}
    virtual ~Competitor() = default;

    virtual void init_csr(Dense<T> &, Dense<T> &, CSR<T> &, CSR<T> &) {}
    virtual void init_coo(Dense<T> &, Dense<T> &, COO<T> &, COO<T> &) {}
    virtual void run_csr(Dense<T> &A, Dense<T> &B, CSR<T> &S, CSR<T> &P) = 0;
    virtual void run_coo(Dense<T> &A, Dense<T> &B, COO<T> &S, COO<T> &P) = 0;
    virtual void cleanup_csr(Dense<T> &, Dense<T> &, CSR<T> &, CSR<T> &) {}
    virtual void cleanup_coo(Dense<T> &, Dense<T> &, COO<T> &, COO<T> &) {}

    virtual bool csr_supported() = 0;
    virtual bool coo_supported() = 0;
    virtual bool is_gpu() { return false; }

    void set_num_threads_per_block(int n) { threads_per_block = n; }
    int get_num_threads_per_block() { return threads_per_block; }
    void set_num_thread_blocks(int n) { thread_blocks = n; }
    int get_num_thread_blocks() { return thread_blocks; }

private:
    int threads_per_block = 1;
    int thread_blocks = 1;
};

}  // namespace SDDMM
