// Small device-side building blocks shared by the SDDMM kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace sddmm {

constexpr unsigned kFullMask = 0xffffffffu;

// Device-visible error word values (first writer wins).
enum DeviceError : int {
    kDevOk = 0,
    kDevMbarrierTimeout = 1,   // a bounded mbarrier wait ran out
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier + bulk async copy (TMA, 1-D, non-multicast) -------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// make barrier initialisation visible to the async proxy
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kSpinLimit probes (each probe itself blocks for a
// hardware-defined time slice), returns false and lets the caller bail out.
constexpr uint32_t kSpinLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t limit = kSpinLimit) {
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
// global -> shared::cta bulk copy, completion counted on `bar`.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---- asynchronous copies global -> shared, tracked per thread in groups ------------
__device__ __forceinline__ void cp_async_4(void *dst_smem, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_8(void *dst_smem, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(void *dst_smem, const void *src) {   // both 16-byte aligned; not kept in L1
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait_group() {   // all but the N most recent groups of this thread have landed
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---- element helpers ---------------------------------------------------------
// A "chunk" is 4 consecutive K elements: a float4 for fp32 storage, 4 bf16
// (8 bytes) for bf16 storage.  dot4 accumulates one chunk pair in fp32.
struct Chunk32 {
    float4 v;
};
struct Chunk16 {
    uint2 v;
};

__device__ __forceinline__ float4 chunk_to_f4(const float4 &c) { return c; }
__device__ __forceinline__ float4 chunk_to_f4(const uint2 &c) {
    // bf16 -> fp32 is a 16-bit left shift of the bit pattern
    float4 r;
    r.x = __uint_as_float(c.x << 16);
    r.y = __uint_as_float(c.x & 0xffff0000u);
    r.z = __uint_as_float(c.y << 16);
    r.w = __uint_as_float(c.y & 0xffff0000u);
    return r;
}
__device__ __forceinline__ float dot4(const float4 &a, const float4 &b, float acc) {
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
    return acc;
}

// Wide bf16 chunks: 8 consecutive K elements (16 bytes), so that 8 lanes read a 128-byte piece of a bf16 row in ONE
// request (with 4-element chunks a lane reads 8 bytes and a 128-byte piece takes two requests of half a line each).
struct Bf16x8 {};
struct F8 {
    float4 lo, hi;
};

template <typename ET>
struct ChunkOf;
template <>
struct ChunkOf<float> {
    using type = float4;
    using areg = float4;
    static constexpr int elems = 4;
};
template <>
struct ChunkOf<__nv_bfloat16> {
    using type = uint2;
    using areg = float4;
    static constexpr int elems = 4;
};
template <>
struct ChunkOf<Bf16x8> {
    using type = uint4;
    using areg = F8;
    static constexpr int elems = 8;
};

__device__ __forceinline__ float4 ldg_chunk(const float4 *p) { return __ldg(p); }
__device__ __forceinline__ uint2 ldg_chunk(const uint2 *p) { return __ldg(p); }
__device__ __forceinline__ uint4 ldg_chunk(const uint4 *p) { return __ldg(p); }
__device__ __forceinline__ float4 zero_chunk(float4) { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ uint2 zero_chunk(uint2) { return make_uint2(0u, 0u); }

// chunk as stored -> fp32 values; dot of an unpacked chunk with a stored one; scaling (masking) of an unpacked chunk
__device__ __forceinline__ float4 unpack_chunk(const float4 &c) { return c; }
__device__ __forceinline__ float4 unpack_chunk(const uint2 &c) { return chunk_to_f4(c); }
__device__ __forceinline__ F8 unpack_chunk(const uint4 &c) {
    F8 r;
    r.lo = chunk_to_f4(make_uint2(c.x, c.y));
    r.hi = chunk_to_f4(make_uint2(c.z, c.w));
    return r;
}
__device__ __forceinline__ float dot_chunk(const float4 &a, const float4 &b, float acc) { return dot4(a, b, acc); }
__device__ __forceinline__ float dot_chunk(const F8 &a, const F8 &b, float acc) { return dot4(a.hi, b.hi, dot4(a.lo, b.lo, acc)); }
__device__ __forceinline__ void scale_chunk(float4 &a, float f) { a.x *= f; a.y *= f; a.z *= f; a.w *= f; }
__device__ __forceinline__ void scale_chunk(F8 &a, float f) { scale_chunk(a.lo, f); scale_chunk(a.hi, f); }

// Sum 8 per-lane partial values over the 8 lanes of an aligned lane group so
// that lane g (0..7) of the group ends up with the complete sum of value g.
// 7 shuffles instead of the 24 a per-value butterfly would take.
__device__ __forceinline__ float group8_transpose_reduce(const float (&acc)[8], int gl) {
    float w[4], x[2];
    const bool up4 = (gl & 4) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float send = up4 ? acc[i] : acc[i + 4];
        const float keep = up4 ? acc[i + 4] : acc[i];
        w[i] = keep + __shfl_xor_sync(kFullMask, send, 4);
    }
    const bool up2 = (gl & 2) != 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float send = up2 ? w[i] : w[i + 2];
        const float keep = up2 ? w[i + 2] : w[i];
        x[i] = keep + __shfl_xor_sync(kFullMask, send, 2);
    }
    const bool up1 = (gl & 1) != 0;
    const float send = up1 ? x[0] : x[1];
    const float keep = up1 ? x[1] : x[0];
    return keep + __shfl_xor_sync(kFullMask, send, 1);
}

}  // namespace sddmm
