// Device-side helpers for the NVFP4 kernels: number-format conversions,
// cache-hinted loads, mbarrier + bulk-copy (TMA) wrappers, programmatic
// dependent launch. sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nvfp4r {

constexpr int kWarp = 32;
constexpr int kBlockElems = 16;   // K elements that share one e4m3 scale

// --------------------------------------------------------------------------
// Number formats
// --------------------------------------------------------------------------

// One byte (two e2m1 codes; low nibble = even element) -> f16x2 (.x = even).
__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t byte) {
    uint32_t out;
    asm("{\n\t.reg .b8 t;\n\tcvt.u8.u32 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}"
        : "=r"(out) : "r"(byte));
    return out;
}

// Four bytes (eight codes) -> four f16x2, element order preserved.
__device__ __forceinline__ void e2m1x8_to_f16x8(uint32_t word, uint32_t out[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3]) : "r"(word));
}

// Two e4m3 bytes (low 16 bits) -> f16x2 (.x = low byte).
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
    uint32_t out;
    asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}"
        : "=r"(out) : "r"(two_bytes));
    return out;
}

// float -> e4m3 byte, round-to-nearest-even, saturating to +-448.
__device__ __forceinline__ uint32_t f32_to_e4m3(float v) {
    uint32_t out;
    asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %2, %1;\n\tcvt.u32.u16 %0, t;\n\t}"
        : "=r"(out) : "f"(v), "f"(0.0f));
    return out & 0xFFu;
}

// Eight floats -> eight e2m1 codes in one word (element i in nibble i), RNE,
// saturating to +-6.
__device__ __forceinline__ uint32_t f32x8_to_e2m1x8(const float v[8]) {
    uint32_t out;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
        : "=r"(out)
        : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]),
          "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return out;
}

__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
    uint32_t h2 = e4m3x2_to_f16x2(byte & 0xFFu);
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xFFFFu)));
}

__device__ __forceinline__ __half2 as_half2(uint32_t v) {
    return *reinterpret_cast<__half2*>(&v);
}
__device__ __forceinline__ uint32_t as_u32(__half2 v) {
    return *reinterpret_cast<uint32_t*>(&v);
}

// --------------------------------------------------------------------------
// Global loads with cache policy
// --------------------------------------------------------------------------

// Streaming 16-byte load: read once, keep out of L1.
__device__ __forceinline__ uint4 ldg_stream_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream_2(const void* p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.b16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
// Re-used data (activations): normal caching.
__device__ __forceinline__ uint4 ldg_keep_16(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

// --------------------------------------------------------------------------
// Shared-memory addresses, mbarriers, bulk copies
// --------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait: gives up after `limit` polls and returns false; the caller
// records the failure in a status word and leaves the kernel in an orderly way.
// A correct run never comes near the limit (each failed try_wait already
// blocks for a hardware-defined interval).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  uint32_t limit = 4000000u) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// L2 cache policies for bulk copies.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// 1-D bulk copy global -> this CTA's shared memory, completion on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;"
        :: "r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}

// Bulk prefetch of global memory into L2 (no destination, no completion signal).
// src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(src), "r"(bytes) : "memory");
}

// --------------------------------------------------------------------------
// Programmatic dependent launch
// --------------------------------------------------------------------------

// Let the next kernel in the stream begin its prologue.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// Wait until the preceding kernel's memory operations are visible.
__device__ __forceinline__ void pdl_wait_prior() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace nvfp4r
