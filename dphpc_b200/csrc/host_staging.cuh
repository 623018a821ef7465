// Host <-> device copies of PAGEABLE host memory (the std::vector containers of the reference's harness).
//
// The driver stages such a copy through its own pinned buffer on one thread, which on this class of host moves about
// 10 GB/s -- a fifth of what the link carries from pinned memory.  Here the staging is done by a small pool of host
// threads: a copy is cut into 8 MiB pieces, the pool memcpy()s piece c+1 into one of two pinned ring buffers while the DMA
// engine moves piece c, and the other way round for downloads.  Pinned or registered host memory and device memory take
// the direct cudaMemcpyAsync path.  Like a pageable cudaMemcpyAsync, a staged call returns when the caller's buffer is
// free again (uploads) or filled (downloads).
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#if defined(__SSE2__)
#include <emmintrin.h>
#endif
#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <cstdint>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace sddmm {

// a fixed pool of host threads that runs "slice k of n" jobs; the caller takes part
class HostPool {
public:
    static HostPool &instance() {
        static HostPool pool;
        return pool;
    }
    int width() const { return static_cast<int>(workers_.size()) + 1; }
    // fn(k) for k in [0, n), spread over the pool; returns when all are done
    void run(int n, const std::function<void(int)> &fn) {
        if (n <= 1 || workers_.empty()) {
            for (int k = 0; k < n; ++k) fn(k);
            return;
        }
        std::lock_guard<std::mutex> one_at_a_time(run_mu_);   // callers on different host threads (one per device) take turns
        std::unique_lock<std::mutex> lock(mu_);
        job_ = &fn;
        next_ = 0;
        total_ = n;
        pending_ = n;
        ++generation_;
        cv_.notify_all();
        lock.unlock();
        work();   // the caller helps
        lock.lock();
        done_.wait(lock, [&] { return pending_ == 0; });
        job_ = nullptr;
    }

private:
    HostPool() {
        unsigned hw = std::thread::hardware_concurrency();
        unsigned want = std::min(hw ? hw / 2 : 2u, 8u);
        if (const char *env = std::getenv("SDDMM_B200_HOST_THREADS")) {   // override: 1 .. 64 threads including the caller
            const int v = std::atoi(env);
            if (v >= 1 && v <= 64) want = static_cast<unsigned>(v);
        }
        const int n = static_cast<int>(std::max(1u, want)) - 1;
        for (int i = 0; i < n; ++i) workers_.emplace_back([this] { loop(); });
    }
    ~HostPool() {
        {
            std::lock_guard<std::mutex> lock(mu_);
            stop_ = true;
            ++generation_;
        }
        cv_.notify_all();
        for (std::thread &t : workers_) t.join();
    }
    void work() {
        while (true) {
            int k;
            const std::function<void(int)> *fn;
            {
                std::lock_guard<std::mutex> lock(mu_);
                if (!job_ || next_ >= total_) return;
                k = next_++;
                fn = job_;
            }
            (*fn)(k);
            std::lock_guard<std::mutex> lock(mu_);
            if (--pending_ == 0) done_.notify_all();
        }
    }
    void loop() {
        unsigned long long seen = 0;
        while (true) {
            {
                std::unique_lock<std::mutex> lock(mu_);
                cv_.wait(lock, [&] { return generation_ != seen; });
                seen = generation_;
                if (stop_) return;
            }
            work();
        }
    }
    std::vector<std::thread> workers_;
    std::mutex mu_, run_mu_;
    std::condition_variable cv_, done_;
    const std::function<void(int)> *job_ = nullptr;
    int next_ = 0, total_ = 0, pending_ = 0;
    unsigned long long generation_ = 0;
    bool stop_ = false;
};

// memcpy whose stores bypass the cache (x86): the destination is a pinned staging buffer that the DMA engine reads next,
// no host thread does, so write-allocating its lines would only add a read of memory per line written.
// SDDMM_B200_STREAM_STORES=0 switches back to plain memcpy.
inline void stream_copy(void *dst, const void *src, size_t bytes) {
#if defined(__SSE2__)
    static const bool enabled = [] { const char *e = std::getenv("SDDMM_B200_STREAM_STORES"); return !(e && e[0] == '0'); }();
    char *d = static_cast<char *>(dst);
    const char *s = static_cast<const char *>(src);
    if (enabled && bytes >= 4096 && (reinterpret_cast<uintptr_t>(d) & 15) == 0) {
        size_t n = bytes / 64;
        for (; n; --n, d += 64, s += 64) {
            const __m128i a = _mm_loadu_si128(reinterpret_cast<const __m128i *>(s));
            const __m128i b = _mm_loadu_si128(reinterpret_cast<const __m128i *>(s + 16));
            const __m128i c = _mm_loadu_si128(reinterpret_cast<const __m128i *>(s + 32));
            const __m128i e = _mm_loadu_si128(reinterpret_cast<const __m128i *>(s + 48));
            _mm_stream_si128(reinterpret_cast<__m128i *>(d), a);
            _mm_stream_si128(reinterpret_cast<__m128i *>(d + 16), b);
            _mm_stream_si128(reinterpret_cast<__m128i *>(d + 32), c);
            _mm_stream_si128(reinterpret_cast<__m128i *>(d + 48), e);
        }
        _mm_sfence();
        bytes &= 63;
    }
    if (bytes) std::memcpy(d, s, bytes);
#else
    std::memcpy(dst, src, bytes);
#endif
}

inline void parallel_memcpy(void *dst, const void *src, size_t bytes, bool stream_stores = false) {
    HostPool &pool = HostPool::instance();
    const int parts = static_cast<int>(std::min<size_t>(pool.width(), std::max<size_t>(1, bytes >> 20)));   // >= 1 MiB per slice
    if (parts <= 1) {
        if (stream_stores) stream_copy(dst, src, bytes); else std::memcpy(dst, src, bytes);
        return;
    }
    const size_t per = (bytes / parts + 4095) & ~size_t(4095);
    pool.run(parts, [&](int k) {
        const size_t off = std::min(bytes, per * static_cast<size_t>(k));
        const size_t len = std::min(per, bytes - off);
        if (!len) return;
        if (stream_stores) stream_copy(static_cast<char *>(dst) + off, static_cast<const char *>(src) + off, len);
        else std::memcpy(static_cast<char *>(dst) + off, static_cast<const char *>(src) + off, len);
    });
}

// two pinned buffers of one engine, used alternately
struct HostStager {
    // bytes per piece (= size of each pinned buffer); SDDMM_B200_STAGE_MB overrides the 8 MiB default (1 .. 256).
    // Measured on a 16-core host with 8 pool threads, 678 MB up: 8 MiB 19-21 ms, 16 MiB 22-23 ms, 32 MiB 23-25 ms,
    // 4 MiB and 2 MiB 43-75 ms (the per-piece hand-over dominates); 12 or 16 threads are no faster and at times far slower.
    const size_t kPiece = [] {
        size_t mb = 8;
        if (const char *env = std::getenv("SDDMM_B200_STAGE_MB")) {
            const int v = std::atoi(env);
            if (v >= 1 && v <= 256) mb = static_cast<size_t>(v);
        }
        return mb << 20;
    }();
    static constexpr size_t kMinStaged = size_t(4) << 20;   // smaller copies are left to the driver
    char *buf[2] = {nullptr, nullptr};
    cudaEvent_t ev[2] = {nullptr, nullptr};
    bool busy[2] = {false, false};

    bool ready() {
        if (buf[0]) return true;
        for (int i = 0; i < 2; ++i) {
            if (cudaHostAlloc(reinterpret_cast<void **>(&buf[i]), kPiece, cudaHostAllocDefault) != cudaSuccess ||
                cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming) != cudaSuccess) {
                cudaGetLastError();
                release();
                return false;
            }
        }
        return true;
    }
    void release() {
        for (int i = 0; i < 2; ++i) {
            if (ev[i]) cudaEventDestroy(ev[i]);
            if (buf[i]) cudaFreeHost(buf[i]);
            ev[i] = nullptr;
            buf[i] = nullptr;
            busy[i] = false;
        }
    }
    static bool pageable(const void *p) {
        cudaPointerAttributes a;
        if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        return a.type == cudaMemoryTypeUnregistered;
    }

    // host -> device on `stream`; the caller's buffer is free when this returns if it was staged
    cudaError_t upload(void *dst, const void *src, size_t bytes, cudaStream_t stream) {
        if (bytes < kMinStaged || !pageable(src) || !ready()) return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream);
        int b = 0;
        for (size_t off = 0; off < bytes; off += kPiece, b ^= 1) {
            const size_t len = std::min(kPiece, bytes - off);
            if (busy[b]) {
                const cudaError_t st = cudaEventSynchronize(ev[b]);
                if (st != cudaSuccess) return st;
            }
            parallel_memcpy(buf[b], static_cast<const char *>(src) + off, len, /*stream_stores=*/true);
            cudaError_t st = cudaMemcpyAsync(static_cast<char *>(dst) + off, buf[b], len, cudaMemcpyHostToDevice, stream);
            if (st == cudaSuccess) st = cudaEventRecord(ev[b], stream);
            if (st != cudaSuccess) return st;
            busy[b] = true;
        }
        return cudaSuccess;
    }
    // device -> host on `stream`; returns when the caller's buffer is filled (the stream has drained up to the copy)
    cudaError_t download(void *dst, const void *src, size_t bytes, cudaStream_t stream) {
        if (bytes < kMinStaged || !pageable(dst) || !ready()) return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream);
        for (int b = 0; b < 2; ++b)
            if (busy[b]) {
                const cudaError_t st = cudaEventSynchronize(ev[b]);
                if (st != cudaSuccess) return st;
                busy[b] = false;
            }
        const size_t pieces = (bytes + kPiece - 1) / kPiece;
        auto enqueue = [&](size_t c) -> cudaError_t {
            const size_t off = c * kPiece, len = std::min(kPiece, bytes - off);
            cudaError_t st = cudaMemcpyAsync(buf[c & 1], static_cast<const char *>(src) + off, len, cudaMemcpyDeviceToHost, stream);
            if (st == cudaSuccess) st = cudaEventRecord(ev[c & 1], stream);
            return st;
        };
        cudaError_t st = enqueue(0);
        for (size_t c = 0; c < pieces && st == cudaSuccess; ++c) {
            st = cudaEventSynchronize(ev[c & 1]);          // piece c has landed in its pinned buffer
            if (st != cudaSuccess) break;
            if (c + 1 < pieces) st = enqueue(c + 1);       // the next piece crosses the link while this one is copied out
            const size_t off = c * kPiece, len = std::min(kPiece, bytes - off);
            parallel_memcpy(static_cast<char *>(dst) + off, buf[c & 1], len);
            if (st != cudaSuccess) break;
        }
        return st;
    }
};

}  // namespace sddmm
