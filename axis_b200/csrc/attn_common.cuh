// Device helpers shared by the tcgen05 attention kernels (head_dim 64 and 128).
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"
#include "tc_common.cuh"

#define LOG2E 1.4426950408889634f
#define LN2 0.6931471805599453f

__device__ __forceinline__ void named_bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// max of three floats in one instruction (3-input max.f32 of sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// mbarrier wait that lets the hardware park the thread: try_wait with a suspend-time hint returns when the phase
// completes or the hint (in ns) runs out, so a waiting warp issues a handful of instructions per microsecond instead
// of spinning (a spinning warp is always eligible and takes issue slots from the warps that compute).  Bounded by
// elapsed SM cycles (about a second), then false.
__device__ __forceinline__ bool mbar_try_park(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(4000u) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_park(uint32_t bar, uint32_t parity) {
    if (mbar_try_park(bar, parity)) return true;
    const long long t0 = clock64();
    do {
        if (mbar_try_park(bar, parity)) return true;
    } while (clock64() - t0 < (1ll << 31));
    return false;
}
// Shared-memory descriptors of these kernels all use SBO = 1024 and 128-byte swizzle, so their upper
// word is one constant and the lower word is (address >> 4) | (LBO >> 4) << 16: the MMA-issuing thread
// keeps a few base words and adds tile offsets (in 16-byte units) instead of rebuilding descriptors.
#define DESC_HI ((1024u >> 4) | (1u << 14) | (2u << 29))
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
    return ((saddr & 0x3FFFF) >> 4) | ((lbo_bytes >> 4) << 16);
}
__device__ __forceinline__ uint64_t desc_of(uint32_t lo) { return ((uint64_t)DESC_HI << 32) | (uint64_t)lo; }
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, uint32_t src, int x, int y, int z, int w) {
    asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// 1-D bulk copy global -> this CTA's shared memory (16-byte aligned addresses, size a multiple of 16), completion on an mbarrier
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

