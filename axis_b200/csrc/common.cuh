// Shared device helpers: storage-type load/store, 16-byte vectors, reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

#define AX_SMS 148   // B200 streaming multiprocessors; grids are sized in multiples of it

__device__ __forceinline__ float ldf(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float ldf(const bf16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stf(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(bf16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

// 16-byte vector access: 4 floats or 8 bf16 widened to float registers.
template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void ld(const float* p, float* f) {
        float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    static __device__ __forceinline__ void st(float* p, const float* f) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    }
};
template <> struct Vec<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void ld(const bf16* p, float* f) {
        uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 t = __bfloat1622float2(h[i]);
            f[2 * i] = t.x; f[2 * i + 1] = t.y;
        }
    }
    static __device__ __forceinline__ void st(bf16* p, const float* f) {
        uint4 v;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = v;
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide sum; every thread gets the result. `sh` holds >= 33 floats.
// The combination order is fixed (warp shuffles, then warp 0 over the warp
// partials), so results do not depend on scheduling.
__device__ __forceinline__ float block_sum(float v, float* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (!lane) sh[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? sh[lane] : 0.f;
        t = warp_sum(t);
        if (!lane) sh[32] = t;
    }
    __syncthreads();
    return sh[32];
}
__device__ __forceinline__ float block_max(float v, float* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (!lane) sh[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? sh[lane] : -3.0e38f;
        t = warp_max(t);
        if (!lane) sh[32] = t;
    }
    __syncthreads();
    return sh[32];
}

static inline int ew_grid(long long work_items, int threads) {
    long long b = (work_items + threads - 1) / threads;
    long long cap = (long long)AX_SMS * 16;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Programmatic dependent launch.  A kernel of the main chain lets its successor be scheduled early and then waits
// itself until its predecessor in the stream has completed (nothing before this point may read what that kernel
// wrote); without the launch attribute both instructions are no-ops.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
extern int ax_gemm_pdl(void);
// launch with the attribute that allows the overlap (off on the side stream and with AXENG_NO_PDL=1, like the GEMMs)
template <typename... KA, typename... A>
static inline cudaError_t ax_launch_chain(void (*kern)(KA...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = ax_gemm_pdl() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KA>(args)...);
}
