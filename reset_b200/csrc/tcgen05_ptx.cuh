// tcgen05 / TMA / tensor-memory PTX wrappers and descriptor builders shared by the
// tensor-core kernels. sm_100a only.
#pragma once

#include <cuda.h>

#include "nvfp4_ptx.cuh"

namespace nvfp4r {
namespace tc {

// ---- PTX wrappers ------------------------------------------------------------

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z,
                                            uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3, %4}], [%5], %6;"
        :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_scales(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" :: "r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X "
        "[%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem),
           "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float v[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]),
          "=f"(v[7]), "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]),
          "=f"(v[14]), "=f"(v[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(threads) : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups
// 1024 B apart. Fields: start >> 4 in bits 0-13, stride-byte-offset >> 4 in bits 32-45,
// fixed 1 in bit 46, swizzle mode 2 (128 B) in bits 61-63.
__device__ __forceinline__ uint64_t desc_operand(uint32_t smem_addr) {
    return (static_cast<uint64_t>(smem_addr & 0x3FFFFu) >> 4) |
           (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Scale chunk (512 B = 32 rows x 16 B), no swizzle, 8-row groups 128 B apart.
__device__ __forceinline__ uint64_t desc_scales(uint32_t smem_addr) {
    return (static_cast<uint64_t>(smem_addr & 0x3FFFFu) >> 4) |
           (static_cast<uint64_t>(128 >> 4) << 32) | (1ull << 46);
}

// Byte offset of (row, byte b of the 128-byte chunk row) in a 128B-swizzled K-major tile.
__device__ __forceinline__ uint32_t swz128(int row, int b) {
    return static_cast<uint32_t>((row >> 3) * 1024 + (row & 7) * 128 +
                                 ((((b >> 4) ^ (row & 7)) << 4) | (b & 15)));
}

struct WaitFail {
    bool failed = false;
    __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity) {
        if (!failed && !mbar_wait_bounded(bar, parity, 20000000u)) failed = true;
        return !failed;
    }
};


}  // namespace tc
}  // namespace nvfp4r
