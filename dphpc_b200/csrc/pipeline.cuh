// Chunked host-to-host SDDMM (sddmm_b200_pipeline_*, include/sddmm_b200.h): the one-shot sequence
// init_csr -> run_csr -> cleanup_csr of the reference's harness (src/benchmark/benchmark.hpp:81-83) with the
// three phases of consecutive row chunks overlapped.
//
// A one-shot call is bound by the host link, not by the kernels: 8 bytes per nonzero go to the device and
// 4 come back, one direction after the other.  The link is full duplex, so the rows of S are cut into
// `chunks` contiguous ranges with equal shares of the nonzeros, every range gets its own engine (own stream,
// own arena) on the same GPU, and while range c is being planned, computed and copied back, the inputs of
// range c+1 are already on their way in.  The host-to-device copies of the ranges are chained through events
// (range c+1 starts after range c's last copy), so the ranges do not share the inbound link and the first
// one is complete as early as possible; B crosses the link once (the first range uploads it, the others take
// a device-to-device copy of it).
//
// Included at the end of engine.cu (it reaches into the engine object for the chaining hooks).
#pragma once

#include <atomic>
#include <chrono>
#include <string>
#include <thread>

struct sddmm_b200_pipeline {
    int device = 0;
    std::vector<sddmm_b200_engine *> engines;
    std::vector<int32_t *> h_rp;        // pinned staging of every chunk's rebased row_ptr
    std::vector<int64_t> h_rp_cap;      // ... and its capacity in elements
    std::vector<int64_t> cuts;          // first row of every chunk of the last call (chunks + 1)
    std::vector<int64_t> offsets;       // ... and its first nonzero
    int64_t K = 0;
    bool ready = false;                 // the last sddmm_csr call succeeded: its pattern and plans are in the engines
    int last_chunks = 0;
    int64_t min_chunk_bytes = int64_t(64) << 20;   // a chunk costs a plan (a handful of stream round trips): about this much traffic each, or more
    std::string err;
};

namespace {

struct ChunkSignal {
    std::atomic<int> *enqueued;   // chunks whose copies are in their streams (or that gave up)
    std::atomic<const float *> *b_src;
    std::atomic<cudaEvent_t> *last_copy;   // ev_h2d of the last chunk that enqueued copies
    sddmm_b200_engine *e;
    int index;
    bool fired;
};

void chunk_copies_enqueued(void *user) {
    ChunkSignal *s = static_cast<ChunkSignal *>(user);
    if (s->fired) return;
    s->fired = true;
    const float *expected = nullptr;
    s->b_src->compare_exchange_strong(expected, s->e->d_B32);   // the first chunk that holds B serves the others
    s->last_copy->store(s->e->ev_h2d);
    s->enqueued->store(s->index + 1, std::memory_order_release);
}

// first row of every chunk: the nnz-balanced cuts every sharded path uses (sddmm_b200_row_cuts), a multiple of 64 rows
// when the matrix is large, so that every chunk keeps the 64 x 64 tile grid of the tensor-core path
std::vector<int64_t> chunk_cuts(const int32_t *row_ptr, int64_t M, int chunks) {
    std::vector<int64_t> cuts(static_cast<size_t>(chunks) + 1, 0);
    sddmm_b200_row_cuts(row_ptr, M, chunks, M >= int64_t(64) * 8 * chunks ? 64 : 1, cuts.data());
    return cuts;
}

}  // namespace

namespace {

// Chunks of the current call are in p->cuts (rows) and p->offsets (nonzeros): run them, one host thread each.
// CSR: row_ptr given (rebased per chunk into pinned staging); COO: row_idx given (rebased on the device).
int run_chunks(sddmm_b200_pipeline *p, int chunks, int64_t N, int64_t K, const int32_t *row_ptr, const int32_t *row_idx,
               const int32_t *col_idx, const float *s_val, const float *A, const float *B, float *p_val) {
    std::atomic<int> enqueued{0};
    std::atomic<const float *> b_src{nullptr};
    std::atomic<cudaEvent_t> last_copy{nullptr};
    std::vector<int> status(static_cast<size_t>(chunks), SDDMM_B200_OK);
    std::vector<ChunkSignal> signals(static_cast<size_t>(chunks));
    static const bool trace = std::getenv("SDDMM_B200_PIPELINE_TRACE") != nullptr;   // debugging knob: host times of every phase
    const auto t_start = std::chrono::steady_clock::now();
    auto since = [&]() { return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t_start).count(); };
    auto work = [&](int c) {
        sddmm_b200_engine *e = p->engines[static_cast<size_t>(c)];
        double t_go = 0, t_up = 0, t_run = 0;
        ChunkSignal &sig = signals[static_cast<size_t>(c)];
        sig = ChunkSignal{&enqueued, &b_src, &last_copy, e, c, false};
        const int64_t r0 = p->cuts[static_cast<size_t>(c)], r1 = p->cuts[static_cast<size_t>(c) + 1];
        const int64_t off = p->offsets[static_cast<size_t>(c)], n = p->offsets[static_cast<size_t>(c) + 1] - off;
        int32_t *local = row_ptr ? p->h_rp[static_cast<size_t>(c)] : nullptr;
        if (row_ptr)
            for (int64_t i = r0; i <= r1; ++i) local[i - r0] = static_cast<int32_t>(row_ptr[i] - off);
        while (enqueued.load(std::memory_order_acquire) < c) std::this_thread::yield();   // every earlier chunk signals, also when it fails
        int st = SDDMM_B200_OK;
        t_go = since();
        if (r1 > r0) {
            e->h2d_after = last_copy.load();   // null for the first chunk that copies
            e->B_on_device = b_src.load();
            e->on_copies_enqueued = chunk_copies_enqueued;
            e->on_copies_user = &sig;
            if (row_ptr) {
                st = sddmm_b200_upload_csr(e, r1 - r0, N, K, local, col_idx + off, s_val + off, A + r0 * K, B);
            } else {
                st = sddmm_b200_upload_coo_rows(e, r1 - r0, N, K, n, r0, row_idx + off, col_idx + off, s_val + off, A + r0 * K, B);
            }
            e->h2d_after = nullptr;
            e->B_on_device = nullptr;
            e->on_copies_enqueued = nullptr;
        }
        if (!sig.fired) {   // empty chunk, or the upload gave up before its copies: let the next chunk go
            sig.fired = true;
            enqueued.store(c + 1, std::memory_order_release);
        }
        t_up = since();
        if (r1 > r0 && st == SDDMM_B200_OK) st = sddmm_b200_run(e);
        t_run = since();
        if (r1 > r0 && st == SDDMM_B200_OK) st = sddmm_b200_download(e, p_val + off);
        status[static_cast<size_t>(c)] = st;
        if (trace) std::fprintf(stderr, "[pipeline] chunk %d rows [%lld, %lld): go %.3f  uploaded+planned %.3f  launched %.3f  downloaded %.3f ms\n", c,
                                static_cast<long long>(r0), static_cast<long long>(r1), t_go, t_up, t_run, since());
    };
    {
        std::vector<std::thread> threads;
        for (int c = 1; c < chunks; ++c) threads.emplace_back(work, c);
        work(0);
        for (std::thread &t : threads) t.join();
    }
    p->last_chunks = chunks;
    for (int c = 0; c < chunks; ++c) {
        if (status[static_cast<size_t>(c)] == SDDMM_B200_OK) continue;
        p->err = "rows [" + std::to_string(p->cuts[static_cast<size_t>(c)]) + ", " + std::to_string(p->cuts[static_cast<size_t>(c) + 1]) +
                 "): " + sddmm_b200_last_error(p->engines[static_cast<size_t>(c)]);
        return status[static_cast<size_t>(c)];
    }
    p->K = K;
    p->ready = true;
    return SDDMM_B200_OK;
}

}  // namespace

extern "C" {

int sddmm_b200_pipeline_create(sddmm_b200_pipeline **out, int device, int mode, uint32_t flags, int chunks) {
    if (!out) return SDDMM_B200_ERR_ARG;
    *out = nullptr;
    if (chunks < 1 || chunks > 64) return SDDMM_B200_ERR_ARG;
    sddmm_b200_pipeline *p = new (std::nothrow) sddmm_b200_pipeline();
    if (!p) return SDDMM_B200_ERR_OOM;
    p->device = device;
    for (int c = 0; c < chunks; ++c) {
        sddmm_b200_engine *e = nullptr;
        const int st = sddmm_b200_create(&e, device, mode, flags);
        if (st != SDDMM_B200_OK) {
            sddmm_b200_pipeline_destroy(p);
            return st;
        }
        p->engines.push_back(e);
    }
    p->h_rp.assign(static_cast<size_t>(chunks), nullptr);
    p->h_rp_cap.assign(static_cast<size_t>(chunks), 0);
    *out = p;
    return SDDMM_B200_OK;
}

int sddmm_b200_pipeline_destroy(sddmm_b200_pipeline *p) {
    if (!p) return SDDMM_B200_OK;
    for (sddmm_b200_engine *e : p->engines) sddmm_b200_destroy(e);
    {
        DeviceGuard g(p->device);
        for (int32_t *h : p->h_rp)
            if (h) cudaFreeHost(h);
    }
    delete p;
    return SDDMM_B200_OK;
}

const char *sddmm_b200_pipeline_last_error(sddmm_b200_pipeline *p) { return p ? p->err.c_str() : "null pipeline"; }

int sddmm_b200_pipeline_last_chunks(sddmm_b200_pipeline *p) { return p ? p->last_chunks : 0; }

int sddmm_b200_pipeline_set_min_chunk_bytes(sddmm_b200_pipeline *p, int64_t bytes) {
    if (!p || bytes < 1) return SDDMM_B200_ERR_ARG;
    p->min_chunk_bytes = bytes;
    return SDDMM_B200_OK;
}

int sddmm_b200_pipeline_sddmm_csr(sddmm_b200_pipeline *p, int64_t M, int64_t N, int64_t K, const int32_t *row_ptr,
                                  const int32_t *col_idx, const float *s_val, const float *A, const float *B, float *p_val) {
    if (!p) return SDDMM_B200_ERR_ARG;
    p->err.clear();
    p->last_chunks = 0;
    p->ready = false;
    auto bad = [&](int code, const char *msg) {
        p->err = msg;
        return code;
    };
    if (!row_ptr || !A || !B) return bad(SDDMM_B200_ERR_ARG, "null pointer argument");
    if (M < 1 || N < 1 || K < 1) return bad(SDDMM_B200_ERR_ARG, "need M, N, K >= 1");
    if (M >= (int64_t(1) << 31) - 1) return bad(SDDMM_B200_ERR_ARG, "int32 index range exceeded");
    const int64_t nnz = row_ptr[M];
    if (nnz < 0) return bad(SDDMM_B200_ERR_INDEX, "row_ptr[M] is negative");
    if (nnz > 0 && (!col_idx || !s_val || !p_val)) return bad(SDDMM_B200_ERR_ARG, "null pointer argument");

    // small inputs: fewer chunks, down to one (nothing to overlap; every chunk costs a plan)
    const int64_t bytes = nnz * 12 + (M + N) * K * 4;
    const int chunks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(static_cast<int64_t>(p->engines.size()), (bytes + p->min_chunk_bytes / 2) / p->min_chunk_bytes)));
    p->cuts = chunk_cuts(row_ptr, M, chunks);
    for (int c = 0; c <= chunks; ++c) {   // the cut rows index col_idx / s_val on the host: check them here, the rest on the device
        const int64_t at = row_ptr[p->cuts[static_cast<size_t>(c)]];
        const int64_t prev = c ? row_ptr[p->cuts[static_cast<size_t>(c) - 1]] : 0;
        if (at < prev || at > nnz || (c == 0 && at != 0)) return bad(SDDMM_B200_ERR_INDEX, "row_ptr is not monotone from 0");
    }
    p->offsets.assign(static_cast<size_t>(chunks) + 1, 0);
    for (int c = 0; c <= chunks; ++c) p->offsets[static_cast<size_t>(c)] = row_ptr[p->cuts[static_cast<size_t>(c)]];
    {   // pinned staging for the rebased row_ptr of every chunk (grows, never shrinks)
        DeviceGuard g(p->device);
        if (!g.ok) return bad(SDDMM_B200_ERR_CUDA, "cannot select the device");
        for (int c = 0; c < chunks; ++c) {
            const int64_t need = p->cuts[static_cast<size_t>(c) + 1] - p->cuts[static_cast<size_t>(c)] + 1;
            if (need <= p->h_rp_cap[static_cast<size_t>(c)]) continue;
            if (p->h_rp[static_cast<size_t>(c)]) cudaFreeHost(p->h_rp[static_cast<size_t>(c)]);
            p->h_rp[static_cast<size_t>(c)] = nullptr;
            p->h_rp_cap[static_cast<size_t>(c)] = 0;
            void *h = nullptr;
            if (cudaHostAlloc(&h, static_cast<size_t>(need) * 4, cudaHostAllocDefault) != cudaSuccess) {
                cudaGetLastError();
                return bad(SDDMM_B200_ERR_OOM, "pinned host allocation failed");
            }
            p->h_rp[static_cast<size_t>(c)] = static_cast<int32_t *>(h);
            p->h_rp_cap[static_cast<size_t>(c)] = need;
        }
    }
    return run_chunks(p, chunks, N, K, row_ptr, nullptr, col_idx, s_val, A, B, p_val);
}

// COO, rows sorted as the reference's COO<T> keeps them (src/matrices/COO.hpp:39).  The cuts are found by binary search in
// row_idx; every chunk's slice is validated on the device against its own row range, which together proves the global order.
int sddmm_b200_pipeline_sddmm_coo(sddmm_b200_pipeline *p, int64_t M, int64_t N, int64_t K, int64_t nnz, const int32_t *row_idx,
                                  const int32_t *col_idx, const float *s_val, const float *A, const float *B, float *p_val) {
    if (!p) return SDDMM_B200_ERR_ARG;
    p->err.clear();
    p->last_chunks = 0;
    p->ready = false;
    auto bad = [&](int code, const char *msg) {
        p->err = msg;
        return code;
    };
    if (!A || !B) return bad(SDDMM_B200_ERR_ARG, "null pointer argument");
    if (M < 1 || N < 1 || K < 1 || nnz < 0) return bad(SDDMM_B200_ERR_ARG, "need M, N, K >= 1 and nnz >= 0");
    if (M >= (int64_t(1) << 31) - 1) return bad(SDDMM_B200_ERR_ARG, "int32 index range exceeded");
    if (nnz > 0 && (!row_idx || !col_idx || !s_val || !p_val)) return bad(SDDMM_B200_ERR_ARG, "null pointer argument");
    const int64_t bytes = nnz * 16 + (M + N) * K * 4;
    const int chunks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(static_cast<int64_t>(p->engines.size()), (bytes + p->min_chunk_bytes / 2) / p->min_chunk_bytes)));
    const int64_t align = M >= int64_t(64) * 8 * chunks ? 64 : 1;
    p->cuts.assign(static_cast<size_t>(chunks) + 1, 0);
    p->offsets.assign(static_cast<size_t>(chunks) + 1, 0);
    if (sddmm_b200_coo_cuts(row_idx, nnz, M, chunks, align, p->cuts.data(), p->offsets.data()) != SDDMM_B200_OK)
        return bad(SDDMM_B200_ERR_INDEX, "COO row indices must be sorted and inside [0, M)");
    return run_chunks(p, chunks, N, K, nullptr, row_idx, col_idx, s_val, A, B, p_val);
}

// Same pattern, new numbers: nothing here blocks, so one host thread enqueues every chunk (copies chained as above,
// conversion, kernels, copy-back) and then waits for all of them.
int sddmm_b200_pipeline_update_csr(sddmm_b200_pipeline *p, const float *s_val, const float *A, const float *B, float *p_val) {
    if (!p) return SDDMM_B200_ERR_ARG;
    p->err.clear();
    auto bad = [&](int code, const std::string &msg) {
        p->err = msg;
        return code;
    };
    if (!p->ready) return bad(SDDMM_B200_ERR_STATE, "update before a successful sddmm_csr call");
    if (!A || !B) return bad(SDDMM_B200_ERR_ARG, "null pointer argument");
    const int chunks = p->last_chunks;
    if (p->offsets[static_cast<size_t>(chunks)] > 0 && (!s_val || !p_val)) return bad(SDDMM_B200_ERR_ARG, "null pointer argument");
    DeviceGuard g(p->device);
    if (!g.ok) return bad(SDDMM_B200_ERR_CUDA, "cannot select the device");
    const int64_t K = p->K;
    cudaEvent_t prev = nullptr;
    const float *b_src = nullptr;
    int st = SDDMM_B200_OK;
    for (int c = 0; c < chunks && st == SDDMM_B200_OK; ++c) {
        const int64_t r0 = p->cuts[static_cast<size_t>(c)], r1 = p->cuts[static_cast<size_t>(c) + 1], off = p->offsets[static_cast<size_t>(c)];
        if (r1 == r0) continue;
        sddmm_b200_engine *e = p->engines[static_cast<size_t>(c)];
        cudaStream_t s = e->stream;
        bool ok = true;
        if (prev) ok = ok && cudaStreamWaitEvent(s, prev, 0) == cudaSuccess;
        if (e->nnz) ok = ok && cudaMemcpyAsync(e->d_sval, s_val + off, static_cast<size_t>(e->nnz) * 4, cudaMemcpyHostToDevice, s) == cudaSuccess;
        ok = ok && cudaMemcpyAsync(e->d_A32, A + r0 * K, static_cast<size_t>((r1 - r0) * K) * 4, cudaMemcpyHostToDevice, s) == cudaSuccess;
        ok = ok && cudaMemcpyAsync(e->d_B32, b_src ? b_src : B, static_cast<size_t>(e->N * K) * 4,
                                   b_src ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, s) == cudaSuccess;
        ok = ok && cudaEventRecord(e->ev_h2d, s) == cudaSuccess;
        prev = e->ev_h2d;
        if (!b_src) b_src = e->d_B32;
        if (!ok) {
            st = bad(SDDMM_B200_ERR_CUDA, std::string("copy failed: ") + cudaGetErrorString(cudaGetLastError()));
            break;
        }
        st = convert_storage(e);
        if (st == SDDMM_B200_OK) st = sddmm_b200_run(e);
        if (st == SDDMM_B200_OK && e->nnz &&
            cudaMemcpyAsync(p_val + off, e->d_pval, static_cast<size_t>(e->nnz) * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess)
            st = SDDMM_B200_ERR_CUDA;
        if (st != SDDMM_B200_OK) p->err = sddmm_b200_last_error(e);
    }
    for (int c = 0; c < chunks; ++c) {   // always drain every chunk: the caller's buffers are free again when this returns
        if (p->cuts[static_cast<size_t>(c) + 1] == p->cuts[static_cast<size_t>(c)]) continue;
        sddmm_b200_engine *e = p->engines[static_cast<size_t>(c)];
        const int sc = sddmm_b200_sync(e);
        if (sc != SDDMM_B200_OK && st == SDDMM_B200_OK) {
            st = sc;
            p->err = sddmm_b200_last_error(e);
        }
    }
    return st;
}

}  // extern "C"
