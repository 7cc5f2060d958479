// Device helpers shared by the sm_100a kernels of this library.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace pk {

constexpr unsigned kFullMask = 0xffffffffu;

// ---- status codes shared by every C entry point (0 = ok; other small values are cudaError_t) ----
enum Status : int {
    kOk = 0,
    kErrBatch = 9101,       // batch outside the supported range
    kErrMaxSeq = 9102,      // context capacity outside 1..max
    kErrNull = 9103,        // a required pointer is null
    kErrCoop = 9104,        // device cannot do cooperative launches
    kErrResidency = 9105,   // grid cannot be co-resident / shared memory limit
    kErrArch = 9106,        // not an sm_100 device
    kErrAlign = 9107,       // pointer / stride alignment
    kErrScratch = 9108,     // workspace too small
    kErrBlock = 9109,       // KV block size / stride invalid
    kErrBarrierTimeout = 9110,  // a bounded device-side wait gave up
    kErrShape = 9111,       // unsupported geometry
    kErrStaticScratch = 9112,   // request does not fit the library's built-in scratch area
};

// ---- bf16 <-> fp32 bit helpers (bf16 carried as the high half of an fp32 pattern) ----
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// fp32 -> bf16 bits, round to nearest even (finite inputs; NaN maps to 0x7fff like cvt.rn.bf16.f32)
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    uint16_t r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
}
// round an fp32 value to the nearest bf16 and return it widened back to fp32
__device__ __forceinline__ float round_bf16(float f) { return __uint_as_float(f32_to_bf16_bits(f) << 16); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// ---- global memory access with cache hints ----
// streaming 16-byte read: read-only path, do not keep in L1
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream_8(void* p, uint2 v) {
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_stream_16(void* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(kFullMask, v, off);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, off));
    return v;
}

// ---- shared-memory barriers (mbarrier) ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// non-blocking probe (try_wait may suspend the warp for a while; the producer must never sleep)
__device__ __forceinline__ bool mbar_probe(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
}  // namespace pk
