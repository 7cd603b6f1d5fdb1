// RMSNorm forward/backward.  HBM-bound: each row is read once from DRAM (the
// second sweep of a row hits L1/L2) and written once; reductions are warp
// shuffles + one shared-memory hop; fp32 math on fp32 or bf16 storage.
#include <cstdio>

#include "common.cuh"
#include "kernels.h"

// y = x * rsqrt(mean(x^2) + eps) * w          (one block per row, grid-strided)
template <typename T, bool VEC>
__global__ void k_rmsnorm(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ o,
                          int rows, int dim, float eps) {
    __shared__ float sh[40];
    constexpr int N = Vec<T>::N;
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const T* xr = x + (long long)r * dim;
        T* orow = o + (long long)r * dim;
        float acc = 0.f;
        if (VEC) {
            for (int j = threadIdx.x * N; j < dim; j += blockDim.x * N) {
                float f[N];
                Vec<T>::ld(xr + j, f);
#pragma unroll
                for (int q = 0; q < N; q++) acc += f[q] * f[q];
            }
        } else {
            for (int j = threadIdx.x; j < dim; j += blockDim.x) { float v = ldf(xr, j); acc += v * v; }
        }
        const float inv = rsqrtf(block_sum(acc, sh) / dim + eps);
        if (VEC) {
            for (int j = threadIdx.x * N; j < dim; j += blockDim.x * N) {
                float f[N], g[N];
                Vec<T>::ld(xr + j, f);
                Vec<T>::ld(w + j, g);
#pragma unroll
                for (int q = 0; q < N; q++) f[q] = f[q] * inv * g[q];
                Vec<T>::st(orow + j, f);
            }
        } else {
            for (int j = threadIdx.x; j < dim; j += blockDim.x) stf(orow, j, ldf(xr, j) * inv * ldf(w, j));
        }
    }
}
// ── warp-per-row forms (dim = 32 * VPL * 16-byte vectors) ──────────────────
// A warp owns a row: every lane loads VPL 16-byte vectors (coalesced 512 B per
// warp per load), the row stays in registers between the reduction and the
// output pass, and the only synchronisation is a shuffle tree — so each row
// costs one DRAM read and one write with many loads in flight per lane.
template <typename T, int VPL>
__global__ void __launch_bounds__(256)
k_rmsnorm_warp(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ o, int rows, float eps) {
    constexpr int N = Vec<T>::N, DIM = 32 * VPL * N;
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nw = gridDim.x * (blockDim.x >> 5);
    for (int r = gw; r < rows; r += nw) {
        const T* xr = x + (long long)r * DIM;
        float xv[VPL][N];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            Vec<T>::ld(xr + (lane + 32 * i) * N, xv[i]);
#pragma unroll
            for (int q = 0; q < N; q++) ss += xv[i][q] * xv[i][q];
        }
        const float inv = rsqrtf(warp_sum(ss) / DIM + eps);
        T* orow = o + (long long)r * DIM;
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            float wv[N];
            Vec<T>::ld(w + (lane + 32 * i) * N, wv);
#pragma unroll
            for (int q = 0; q < N; q++) xv[i][q] = xv[i][q] * inv * wv[q];
            Vec<T>::st(orow + (lane + 32 * i) * N, xv[i]);
        }
    }
}

// ── wide rows: WPR warps share a row ───────────────────────────────────────
// Rows too wide for one warp's registers (the 7B-class width 4096 is 16 vectors per lane in bf16) are cut
// into WPR column spans, one warp each; the WPR warps of a row exchange their partial sums through shared
// memory around a named barrier of their own (two slots used alternately, so one barrier per row suffices).
// Blocks have 8 warps = 8 / WPR rows in flight.
__device__ __forceinline__ void row_bar(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
template <typename T, int VPL, int WPR>
__global__ void __launch_bounds__(256)
k_rmsnorm_wide(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ o, int rows, float eps) {
    constexpr int N = Vec<T>::N, SPAN = 32 * VPL * N, DIM = SPAN * WPR, G = 8 / WPR;
    __shared__ float red[2][G][WPR];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, grp = wib / WPR, part = wib % WPR;
    int it = 0;
    for (int r = blockIdx.x * G + grp; r < rows; r += gridDim.x * G, it ^= 1) {
        const T* xr = x + (long long)r * DIM + part * SPAN;
        float xv[VPL][N];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            Vec<T>::ld(xr + (lane + 32 * i) * N, xv[i]);
#pragma unroll
            for (int q = 0; q < N; q++) ss += xv[i][q] * xv[i][q];
        }
        ss = warp_sum(ss);
        if (lane == 0) red[it][grp][part] = ss;
        row_bar(1 + grp, WPR * 32);
        float tot = 0.f;
#pragma unroll
        for (int q = 0; q < WPR; q++) tot += red[it][grp][q];
        const float inv = rsqrtf(tot / DIM + eps);
        T* orow = o + (long long)r * DIM + part * SPAN;
        const T* wr = w + part * SPAN;
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            float wv[N];
            Vec<T>::ld(wr + (lane + 32 * i) * N, wv);
#pragma unroll
            for (int q = 0; q < N; q++) xv[i][q] = xv[i][q] * inv * wv[q];
            Vec<T>::st(orow + (lane + 32 * i) * N, xv[i]);
        }
    }
}

#define RBW_WARPS 8
template <typename T, int VPL>
__global__ void __launch_bounds__(RBW_WARPS * 32)
k_rmsnorm_bwd_warp(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ g, const T* res, T* dx,
                   float* __restrict__ partial, int rows, float eps) {
    constexpr int N = Vec<T>::N, DIM = 32 * VPL * N;
    __shared__ float sdw[DIM];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int gw = blockIdx.x * RBW_WARPS + wib, nw = gridDim.x * RBW_WARPS;
    float dw[VPL][N];
#pragma unroll
    for (int i = 0; i < VPL; i++)
#pragma unroll
        for (int q = 0; q < N; q++) dw[i][q] = 0.f;
    for (int r = gw; r < rows; r += nw) {
        const long long base = (long long)r * DIM;
        float xv[VPL][N], gv[VPL][N];
        float ss = 0.f, gwx = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            const int c = (lane + 32 * i) * N;
            float wv[N];
            Vec<T>::ld(x + base + c, xv[i]);
            Vec<T>::ld(g + base + c, gv[i]);
            Vec<T>::ld(w + c, wv);
#pragma unroll
            for (int q = 0; q < N; q++) {
                ss += xv[i][q] * xv[i][q];
                gwx += gv[i][q] * wv[q] * xv[i][q];
            }
        }
        ss = warp_sum(ss);
        gwx = warp_sum(gwx);
        const float inv = rsqrtf(ss / DIM + eps);
        const float coef = inv * inv * inv * (gwx / DIM);
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            const int c = (lane + 32 * i) * N;
            float ov[N], wv[N];
            Vec<T>::ld(w + c, wv);
            if (res) Vec<T>::ld(res + base + c, ov);
#pragma unroll
            for (int q = 0; q < N; q++) {
                const float d = gv[i][q] * wv[q] * inv - xv[i][q] * coef;
                ov[q] = res ? ov[q] + d : d;
                dw[i][q] += gv[i][q] * xv[i][q] * inv;
            }
            Vec<T>::st(dx + base + c, ov);
        }
    }
    if (!partial) return;
    // block partial: warps add their column sums one after another (fixed order)
    for (int j = threadIdx.x; j < DIM; j += blockDim.x) sdw[j] = 0.f;
    __syncthreads();
    for (int turn = 0; turn < RBW_WARPS; turn++) {
        if (wib == turn) {
#pragma unroll
            for (int i = 0; i < VPL; i++)
#pragma unroll
                for (int q = 0; q < N; q++) sdw[(lane + 32 * i) * N + q] += dw[i][q];
        }
        __syncthreads();
    }
    for (int j = threadIdx.x; j < DIM; j += blockDim.x) partial[(long long)blockIdx.x * DIM + j] = sdw[j];
}

// bf16 specialisation: rows stay packed (16-byte vectors) in registers and the dw partial of every warp
// accumulates in its own shared-memory row (a lane only ever touches its own columns, so no synchronisation),
// which leaves room for 8-warp blocks, two to an SM: sixteen rows with 3*VPL 16-byte loads per lane in flight
// per SM, and x, g and the residual are each read once.
#define RBP_WARPS 8
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <int VPL>
__global__ void __launch_bounds__(RBP_WARPS * 32, 2)
k_rmsnorm_bwd_packed(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ g, const bf16* res,
                     bf16* dx, float* __restrict__ partial, int rows, float eps) {
    constexpr int DIM = 32 * VPL * 8;
    extern __shared__ float sdw_all[];                     // [RBP_WARPS][DIM]
    pdl_enter();
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int gw = blockIdx.x * RBP_WARPS + wib, nw = gridDim.x * RBP_WARPS;
    float* sdw = sdw_all + wib * DIM;
#pragma unroll
    for (int i = 0; i < VPL; i++) {
        float4* p = reinterpret_cast<float4*>(sdw + (lane + 32 * i) * 8);
        p[0] = make_float4(0.f, 0.f, 0.f, 0.f); p[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int r = gw; r < rows; r += nw) {
        const long long base = (long long)r * DIM;
        uint4 xp[VPL], gp[VPL], rp[VPL];
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            const int c = (lane + 32 * i) * 8;
            xp[i] = *reinterpret_cast<const uint4*>(x + base + c);
            gp[i] = *reinterpret_cast<const uint4*>(g + base + c);
            if (res) rp[i] = *reinterpret_cast<const uint4*>(res + base + c);
        }
        float ss = 0.f, gwx = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            float xv[8], gv[8], wv[8];
            unpack8(xp[i], xv); unpack8(gp[i], gv); unpack8(__ldg(reinterpret_cast<const uint4*>(w + (lane + 32 * i) * 8)), wv);
#pragma unroll
            for (int q = 0; q < 8; q++) { ss += xv[q] * xv[q]; gwx += gv[q] * wv[q] * xv[q]; }
        }
        ss = warp_sum(ss);
        gwx = warp_sum(gwx);
        const float inv = rsqrtf(ss / DIM + eps);
        const float coef = inv * inv * inv * (gwx / DIM);
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            float xv[8], gv[8], wv[8], ov[8];
            unpack8(xp[i], xv); unpack8(gp[i], gv); unpack8(__ldg(reinterpret_cast<const uint4*>(w + (lane + 32 * i) * 8)), wv);
            if (res) unpack8(rp[i], ov);
            float4* p = reinterpret_cast<float4*>(sdw + (lane + 32 * i) * 8);
            float4 a0 = p[0], a1 = p[1];
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float d = gv[q] * wv[q] * inv - xv[q] * coef;
                ov[q] = res ? ov[q] + d : d;
            }
            a0.x += gv[0] * xv[0] * inv; a0.y += gv[1] * xv[1] * inv; a0.z += gv[2] * xv[2] * inv; a0.w += gv[3] * xv[3] * inv;
            a1.x += gv[4] * xv[4] * inv; a1.y += gv[5] * xv[5] * inv; a1.z += gv[6] * xv[6] * inv; a1.w += gv[7] * xv[7] * inv;
            p[0] = a0; p[1] = a1;
            Vec<bf16>::st(dx + base + (lane + 32 * i) * 8, ov);
        }
    }
    if (!partial) return;
    __syncthreads();
    for (int j = threadIdx.x; j < DIM; j += blockDim.x) {   // fixed order over the warps' rows
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < RBP_WARPS; q++) t += sdw_all[q * DIM + j];
        partial[(long long)blockIdx.x * DIM + j] = t;
    }
}

// The packed backward for wide rows: WPR warps per row (see k_rmsnorm_wide); every warp keeps the dw partial of
// its own column span in its own shared-memory row, and the block partial adds the rows' groups in fixed order.
template <int VPL, int WPR>
__global__ void __launch_bounds__(RBP_WARPS * 32, 2)
k_rmsnorm_bwd_packed_wide(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ g,
                          const bf16* res, bf16* dx, float* __restrict__ partial, int rows, float eps) {
    constexpr int SPAN = 32 * VPL * 8, DIM = SPAN * WPR, G = RBP_WARPS / WPR;
    extern __shared__ float sdw_all[];                     // [RBP_WARPS][SPAN]
    __shared__ float red[2][G][WPR][2];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, grp = wib / WPR, part = wib % WPR;
    float* sdw = sdw_all + wib * SPAN;
#pragma unroll
    for (int i = 0; i < VPL; i++) {
        float4* p = reinterpret_cast<float4*>(sdw + (lane + 32 * i) * 8);
        p[0] = make_float4(0.f, 0.f, 0.f, 0.f); p[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const bf16* wr = w + part * SPAN;
    int it = 0;
    for (int r = blockIdx.x * G + grp; r < rows; r += gridDim.x * G, it ^= 1) {
        const long long base = (long long)r * DIM + part * SPAN;
        uint4 xp[VPL], gp[VPL], rp[VPL];
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            const int c = (lane + 32 * i) * 8;
            xp[i] = *reinterpret_cast<const uint4*>(x + base + c);
            gp[i] = *reinterpret_cast<const uint4*>(g + base + c);
            if (res) rp[i] = *reinterpret_cast<const uint4*>(res + base + c);
        }
        float ss = 0.f, gwx = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            float xv[8], gv[8], wv[8];
            unpack8(xp[i], xv); unpack8(gp[i], gv); unpack8(__ldg(reinterpret_cast<const uint4*>(wr + (lane + 32 * i) * 8)), wv);
#pragma unroll
            for (int q = 0; q < 8; q++) { ss += xv[q] * xv[q]; gwx += gv[q] * wv[q] * xv[q]; }
        }
        ss = warp_sum(ss);
        gwx = warp_sum(gwx);
        if (lane == 0) { red[it][grp][part][0] = ss; red[it][grp][part][1] = gwx; }
        row_bar(1 + grp, WPR * 32);
        ss = 0.f; gwx = 0.f;
#pragma unroll
        for (int q = 0; q < WPR; q++) { ss += red[it][grp][q][0]; gwx += red[it][grp][q][1]; }
        const float inv = rsqrtf(ss / DIM + eps);
        const float coef = inv * inv * inv * (gwx / DIM);
#pragma unroll
        for (int i = 0; i < VPL; i++) {
            float xv[8], gv[8], wv[8], ov[8];
            unpack8(xp[i], xv); unpack8(gp[i], gv); unpack8(__ldg(reinterpret_cast<const uint4*>(wr + (lane + 32 * i) * 8)), wv);
            if (res) unpack8(rp[i], ov);
            float4* p = reinterpret_cast<float4*>(sdw + (lane + 32 * i) * 8);
            float4 a0 = p[0], a1 = p[1];
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float d = gv[q] * wv[q] * inv - xv[q] * coef;
                ov[q] = res ? ov[q] + d : d;
            }
            a0.x += gv[0] * xv[0] * inv; a0.y += gv[1] * xv[1] * inv; a0.z += gv[2] * xv[2] * inv; a0.w += gv[3] * xv[3] * inv;
            a1.x += gv[4] * xv[4] * inv; a1.y += gv[5] * xv[5] * inv; a1.z += gv[6] * xv[6] * inv; a1.w += gv[7] * xv[7] * inv;
            p[0] = a0; p[1] = a1;
            Vec<bf16>::st(dx + base + (lane + 32 * i) * 8, ov);
        }
    }
    if (!partial) return;
    __syncthreads();
    for (int j = threadIdx.x; j < DIM; j += blockDim.x) {   // fixed order over the row groups
        const int pj = j / SPAN, cj = j - pj * SPAN;
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < G; q++) t += sdw_all[(q * WPR + pj) * SPAN + cj];
        partial[(long long)blockIdx.x * DIM + j] = t;
    }
}
// warps per row (2 or 4, 0 = no wide form) such that a lane holds at most `maxv` 16-byte vectors of its span
static int wide_wpr(int dim, int per, int maxv) {
    for (int wpr = 2; wpr <= 4; wpr *= 2)
        if (dim % (32 * per * wpr) == 0 && dim / (32 * per * wpr) <= maxv) return wpr;
    return 0;
}

static int norm_threads(int dim, int per) {
    int t = (dim / per + 31) / 32 * 32;
    if (t < 32) t = 32;
    if (t > 512) t = 512;
    return t;
}
int ax_rmsnorm(int dt, const void* x, const void* w, void* o, int rows, int dim, float eps, cudaStream_t st) {
    if (rows <= 0 || dim <= 0) return 0;
    const int per = dt == 1 ? 8 : 4;
    const bool vec = dim % per == 0 && aligned16(x) && aligned16(w) && aligned16(o);
    if (vec && dim % (32 * per) == 0 && dim / (32 * per) <= 8) {
        const int vpl = dim / (32 * per);
        const int g = (rows + 7) / 8 < AX_SMS * 8 ? (rows + 7) / 8 : AX_SMS * 8;
#define NW(TT, V) case V: ax_launch_chain(k_rmsnorm_warp<TT, V>, dim3(g), dim3(256), 0, st, (const TT*)x, (const TT*)w, (TT*)o, rows, eps); return 0;
        if (dt == 1) { switch (vpl) { NW(bf16, 1) NW(bf16, 2) NW(bf16, 3) NW(bf16, 4) NW(bf16, 5) NW(bf16, 6) NW(bf16, 7) NW(bf16, 8) } }
        else { switch (vpl) { NW(float, 1) NW(float, 2) NW(float, 3) NW(float, 4) NW(float, 5) NW(float, 6) NW(float, 7) NW(float, 8) } }
#undef NW
    }
    if (const int wpr = vec ? wide_wpr(dim, per, 8) : 0) {
        const int vpl = dim / (32 * per * wpr), gr = 8 / wpr;
        const int g = (rows + gr - 1) / gr < AX_SMS * 8 ? (rows + gr - 1) / gr : AX_SMS * 8;
#define NWW(TT, V, W) case V: k_rmsnorm_wide<TT, V, W><<<g, 256, 0, st>>>((const TT*)x, (const TT*)w, (TT*)o, rows, eps); return 0;
#define NWS(TT, W) switch (vpl) { NWW(TT, 1, W) NWW(TT, 2, W) NWW(TT, 3, W) NWW(TT, 4, W) NWW(TT, 5, W) NWW(TT, 6, W) NWW(TT, 7, W) NWW(TT, 8, W) }
        if (dt == 1) { if (wpr == 2) NWS(bf16, 2) else NWS(bf16, 4) }
        else { if (wpr == 2) NWS(float, 2) else NWS(float, 4) }
#undef NWS
#undef NWW
    }
    const int thr = norm_threads(dim, vec ? per : 1);
    const int grid = rows < AX_SMS * 32 ? rows : AX_SMS * 32;
    if (dt == 1) {
        if (vec) k_rmsnorm<bf16, true><<<grid, thr, 0, st>>>((const bf16*)x, (const bf16*)w, (bf16*)o, rows, dim, eps);
        else k_rmsnorm<bf16, false><<<grid, thr, 0, st>>>((const bf16*)x, (const bf16*)w, (bf16*)o, rows, dim, eps);
    } else {
        if (vec) k_rmsnorm<float, true><<<grid, thr, 0, st>>>((const float*)x, (const float*)w, (float*)o, rows, dim, eps);
        else k_rmsnorm<float, false><<<grid, thr, 0, st>>>((const float*)x, (const float*)w, (float*)o, rows, dim, eps);
    }
    return 0;
}

// Two-kernel form of the reference ABI: dx plus tmp = g*x*inv (N x D), whose
// column sum (COLSUM) is dw.
template <typename T>
__global__ void k_rmsnorm_bwd(const T* x, const T* w, const T* g, T* dx, T* tmp, int rows, int dim, float eps) {
    __shared__ float sh[40];
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const long long base = (long long)r * dim;
        float ss = 0.f, gwx = 0.f;
        for (int j = threadIdx.x; j < dim; j += blockDim.x) {
            const float xv = ldf(x, base + j), gv = ldf(g, base + j);
            ss += xv * xv;
            gwx += gv * ldf(w, j) * xv;
        }
        ss = block_sum(ss, sh);
        gwx = block_sum(gwx, sh);
        const float inv = rsqrtf(ss / dim + eps);
        const float coef = inv * inv * inv * (gwx / dim);
        for (int j = threadIdx.x; j < dim; j += blockDim.x) {
            const float xv = ldf(x, base + j), gv = ldf(g, base + j);
            stf(dx, base + j, gv * ldf(w, j) * inv - xv * coef);
            stf(tmp, base + j, gv * xv * inv);
        }
    }
}
int ax_rmsnorm_bwd(int dt, const void* x, const void* w, const void* g, void* dx, void* tmp, int rows, int dim,
                   float eps, cudaStream_t st) {
    if (rows <= 0 || dim <= 0) return 0;
    const int thr = norm_threads(dim, 1);
    const int grid = rows < AX_SMS * 32 ? rows : AX_SMS * 32;
    if (dt == 1) k_rmsnorm_bwd<bf16><<<grid, thr, 0, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)g, (bf16*)dx, (bf16*)tmp, rows, dim, eps);
    else k_rmsnorm_bwd<float><<<grid, thr, 0, st>>>((const float*)x, (const float*)w, (const float*)g, (float*)dx, (float*)tmp, rows, dim, eps);
    return 0;
}

// Column sum: block (32 columns x 8 row lanes), rows strided over lanes, then
// a fixed-order shared-memory combine.  c[j] = sum_r a[r, j].
template <typename T>
__global__ void k_colsum(const T* __restrict__ a, float* __restrict__ c, int rows, int n) {
    __shared__ float sh[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    float acc = 0.f;
    if (col < n)
        for (int r = threadIdx.y; r < rows; r += 8) acc += ldf(a, (long long)r * n + col);
    sh[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && col < n) {
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < 8; q++) t += sh[q][threadIdx.x];
        c[col] = t;
    }
}
int ax_colsum(int dt, const void* a, float* c, int rows, int n, cudaStream_t st) {
    if (n <= 0) return 0;
    dim3 blk(32, 8);
    if (dt >= 1) k_colsum<bf16><<<(n + 31) / 32, blk, 0, st>>>((const bf16*)a, c, rows, n);
    else k_colsum<float><<<(n + 31) / 32, blk, 0, st>>>((const float*)a, c, rows, n);
    return 0;
}

// ── fused backward: dx (+ residual) and dw in one pass over x and g ────────
// Grid of NB blocks; block b owns rows b, b+NB, ...  Each thread owns fixed
// columns, so the per-block dw partial accumulates in shared memory without
// synchronisation.  A second kernel adds the NB partials per column in block
// order — no atomics, run-to-run identical.
#define RB_BLOCKS (AX_SMS * 2)
template <typename T, bool VEC>
__global__ void k_rmsnorm_bwd_acc(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ g,
                                  const T* res, T* dx, float* __restrict__ partial,
                                  int rows, int dim, float eps) {
    extern __shared__ float sdw[];            // dim floats
    __shared__ float sh[40];
    constexpr int N = Vec<T>::N;
    for (int j = threadIdx.x; j < dim; j += blockDim.x) sdw[j] = 0.f;
    __syncthreads();
    // inside the row loop each thread only touches the columns it owns
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const long long base = (long long)r * dim;
        float ss = 0.f, gwx = 0.f;
        if (VEC) {
            for (int j = threadIdx.x * N; j < dim; j += blockDim.x * N) {
                float xv[N], gv[N], wv[N];
                Vec<T>::ld(x + base + j, xv);
                Vec<T>::ld(g + base + j, gv);
                Vec<T>::ld(w + j, wv);
#pragma unroll
                for (int q = 0; q < N; q++) { ss += xv[q] * xv[q]; gwx += gv[q] * wv[q] * xv[q]; }
            }
        } else {
            for (int j = threadIdx.x; j < dim; j += blockDim.x) {
                const float xv = ldf(x, base + j), gv = ldf(g, base + j);
                ss += xv * xv; gwx += gv * ldf(w, j) * xv;
            }
        }
        ss = block_sum(ss, sh);
        gwx = block_sum(gwx, sh);
        const float inv = rsqrtf(ss / dim + eps);
        const float coef = inv * inv * inv * (gwx / dim);
        if (VEC) {
            for (int j = threadIdx.x * N; j < dim; j += blockDim.x * N) {
                float xv[N], gv[N], wv[N], o[N];
                Vec<T>::ld(x + base + j, xv);
                Vec<T>::ld(g + base + j, gv);
                Vec<T>::ld(w + j, wv);
                if (res) Vec<T>::ld(res + base + j, o);
#pragma unroll
                for (int q = 0; q < N; q++) {
                    const float d = gv[q] * wv[q] * inv - xv[q] * coef;
                    o[q] = res ? o[q] + d : d;
                    sdw[j + q] += gv[q] * xv[q] * inv;
                }
                Vec<T>::st(dx + base + j, o);
            }
        } else {
            for (int j = threadIdx.x; j < dim; j += blockDim.x) {
                const float xv = ldf(x, base + j), gv = ldf(g, base + j);
                const float d = gv * ldf(w, j) * inv - xv * coef;
                stf(dx, base + j, res ? ldf(res, base + j) + d : d);
                sdw[j] += gv * xv * inv;
            }
        }
    }
    __syncthreads();
    if (partial)
        for (int j = threadIdx.x; j < dim; j += blockDim.x) partial[(long long)blockIdx.x * dim + j] = sdw[j];
}
// dw[j] = sum over the nb block partials: 32 columns x 8 row lanes per block, then a fixed-order combine
__global__ void k_colsum_partials(const float* __restrict__ partial, float* __restrict__ dw, int nb, int dim) {
    __shared__ float sh[8][33];
    const int j = blockIdx.x * 32 + threadIdx.x;
    float acc = 0.f;
    if (j < dim)
        for (int b = threadIdx.y; b < nb; b += 8) acc += partial[(long long)b * dim + j];
    sh[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && j < dim) {
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < 8; q++) t += sh[q][threadIdx.x];
        dw[j] = t;
    }
}
long long ax_rmsnorm_bwd_acc_scratch(int dim) { return (long long)RB_BLOCKS * dim * sizeof(float); }
int ax_rmsnorm_bwd_acc(int dt, const void* x, const void* w, const void* g, const void* res, void* dx,
                       float* dw, float* scratch, int rows, int dim, float eps, cudaStream_t st, int defer) {
    // defer: leave the per-block partials in `scratch` (rows the launch does not use keep what they hold) and
    // do not sum them; ax_colsum_batch sums all RB_BLOCKS rows of several such scratch areas later
    if (rows <= 0 || dim <= 0) return 0;
    if ((size_t)dim * 4 > 200 * 1024) return 120;
    const int per = dt == 1 ? 8 : 4;
    const bool vec = dim % per == 0 && aligned16(x) && aligned16(w) && aligned16(g) && aligned16(dx) &&
                     (!res || aligned16(res));
    float* part = (dw || defer) ? scratch : nullptr;
    if (vec && dim % (32 * per) == 0 && dim / (32 * per) <= 6) {      // more vectors per lane would spill
        const int vpl = dim / (32 * per);
        if (dt == 1) {
            int nbp = (rows + RBP_WARPS - 1) / RBP_WARPS;
            if (nbp > RB_BLOCKS) nbp = RB_BLOCKS;            // 296 blocks: two per SM resident at once, one wave
#define BP(V) case V: ax_launch_chain(k_rmsnorm_bwd_packed<V>, dim3(nbp), dim3(RBP_WARPS * 32), (size_t)RBP_WARPS * dim * 4, st, (const bf16*)x, (const bf16*)w, (const bf16*)g, (const bf16*)res, (bf16*)dx, part, rows, eps); break;
            switch (vpl) { BP(1) BP(2) BP(3) BP(4) BP(5) BP(6) }
#undef BP
            if (dw && !defer) k_colsum_partials<<<(dim + 31) / 32, dim3(32, 8), 0, st>>>(scratch, dw, nbp, dim);
            return 0;
        }
        int nbw = (rows + RBW_WARPS - 1) / RBW_WARPS;
        if (nbw > RB_BLOCKS) nbw = RB_BLOCKS;
#define BW(TT, V) case V: k_rmsnorm_bwd_warp<TT, V><<<nbw, RBW_WARPS * 32, 0, st>>>((const TT*)x, (const TT*)w, (const TT*)g, (const TT*)res, (TT*)dx, part, rows, eps); break;
        if (dt == 1) { switch (vpl) { BW(bf16, 1) BW(bf16, 2) BW(bf16, 3) BW(bf16, 4) BW(bf16, 5) BW(bf16, 6) } }
        else { switch (vpl) { BW(float, 1) BW(float, 2) BW(float, 3) BW(float, 4) BW(float, 5) BW(float, 6) } }
#undef BW
        if (dw && !defer) k_colsum_partials<<<(dim + 31) / 32, dim3(32, 8), 0, st>>>(scratch, dw, nbw, dim);
        return 0;
    }
    // at most 5 vectors per lane: 8 warps x 5 KB of dw rows plus the exchange slots stay inside the 48 KB
    // that need no opt-in
    if (const int wpr = (vec && dt == 1) ? wide_wpr(dim, per, 5) : 0) {
        const int vpl = dim / (32 * per * wpr), gr = RBP_WARPS / wpr;
        int nbp = (rows + gr - 1) / gr;
        if (nbp > RB_BLOCKS) nbp = RB_BLOCKS;
        const size_t sm = (size_t)RBP_WARPS * (dim / wpr) * 4;
#define BPW(V, W) case V: k_rmsnorm_bwd_packed_wide<V, W><<<nbp, RBP_WARPS * 32, sm, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)g, (const bf16*)res, (bf16*)dx, part, rows, eps); break;
#define BPS(W) switch (vpl) { BPW(1, W) BPW(2, W) BPW(3, W) BPW(4, W) BPW(5, W) }
        if (wpr == 2) BPS(2) else BPS(4)
#undef BPS
#undef BPW
        if (dw && !defer) k_colsum_partials<<<(dim + 31) / 32, dim3(32, 8), 0, st>>>(scratch, dw, nbp, dim);
        return 0;
    }
    const int thr = norm_threads(dim, vec ? per : 1);
    const int nb = rows < RB_BLOCKS ? rows : RB_BLOCKS;
    const size_t smem = (size_t)dim * 4;
#define RB_LAUNCH(TT, VV)                                                                              \
    do {                                                                                               \
        if (smem > 48 * 1024)                                                                          \
            cudaFuncSetAttribute(k_rmsnorm_bwd_acc<TT, VV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        k_rmsnorm_bwd_acc<TT, VV><<<nb, thr, smem, st>>>((const TT*)x, (const TT*)w, (const TT*)g,      \
                                                         (const TT*)res, (TT*)dx, part, rows, dim, eps); \
    } while (0)
    if (dt == 1) { if (vec) RB_LAUNCH(bf16, true); else RB_LAUNCH(bf16, false); }
    else { if (vec) RB_LAUNCH(float, true); else RB_LAUNCH(float, false); }
#undef RB_LAUNCH
    if (dw && !defer) k_colsum_partials<<<(dim + 31) / 32, dim3(32, 8), 0, st>>>(scratch, dw, nb, dim);
    return 0;
}

// dw of `count` deferred RMSNorm backward launches in one launch: instance y has its RB_BLOCKS x dim partials at
// scratch + (first + y) * RB_BLOCKS * dim and its result goes to arena + table[first + y] * chunk.  Rows beyond those
// a launch wrote are zero (the scratch is allocated zeroed and row counts do not change between steps), so the sum
// always runs over all RB_BLOCKS rows in block order: no atomics, run-to-run identical.  A destination outside the
// arena is skipped and reported through the status word.
__global__ void k_colsum_batch(const float* __restrict__ scratch, float* __restrict__ arena, const int* __restrict__ table,
                               int first, int dim, int chunk, long long arena_elems, int* status) {
    __shared__ float sh[8][33];
    const int inst = first + blockIdx.y;
    const float* partial = scratch + (long long)inst * RB_BLOCKS * dim;
    const long long off = (long long)table[inst] * chunk;
    const int j = blockIdx.x * 32 + threadIdx.x;
    float acc = 0.f;
    if (j < dim)
        for (int b = threadIdx.y; b < RB_BLOCKS; b += 8) acc += partial[(long long)b * dim + j];
    sh[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && j < dim) {
        if (off < 0 || off + dim > arena_elems) { if (j == 0) atomicExch(status, 130); return; }
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < 8; q++) t += sh[q][threadIdx.x];
        arena[off + j] = t;
    }
}
int ax_colsum_batch(const float* scratch, float* arena, const int* table, int first, int count, int dim, int chunk,
                    long long arena_elems, int* status, cudaStream_t st) {
    if (count <= 0 || dim <= 0) return 0;
    if (count > 65535) return 121;
    k_colsum_batch<<<dim3((dim + 31) / 32, count), dim3(32, 8), 0, st>>>(scratch, arena, table, first, dim, chunk, arena_elems, status);
    return 0;
}

// ── allocation-free variant of the fused RMSNorm backward ──────────────────
// The per-block dw partials normally live in a scratch buffer that the caller
// allocates.  Some callers cannot allocate: code that runs while a stream is
// being captured into a CUDA graph (cudaMalloc is illegal there), hosts that
// hand this library a fixed memory budget carved up at start-up, and latency
// sensitive loops where an allocator call (and its implicit synchronisation)
// is not acceptable.  For them the partials live in this file-scope device
// array instead: RB_BLOCKS x AX_NOALLOC_MAX_DIM floats (about 9.7 MB), held by
// every GPU that loads the library until the process exits.
#define AX_NOALLOC_MAX_DIM 8192
#define AX_NOALLOC_MAX_DEVICES 64
static __device__ __align__(256) float g_noalloc_partials[RB_BLOCKS * AX_NOALLOC_MAX_DIM];
// Device address of the array per device ordinal.  In host code the symbol
// g_noalloc_partials is only a handle, not a pointer a kernel can follow, so
// the address is looked up once per device with that device current.
static float* g_noalloc_addr[AX_NOALLOC_MAX_DEVICES];

extern "C" __attribute__((visibility("default")))
int eng_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* g, const void* res, void* dx, float* dw,
                            int rows, int dim, int dt, float eps, void* stream) {
    if (!x || !w || !g || !dx || rows < 0 || dim <= 0 || (dt != 0 && dt != 1)) return 202;
    if (dim > AX_NOALLOC_MAX_DIM) {
        fprintf(stderr, "eng_rmsnorm_bwd_noalloc: dim %d exceeds the built-in scratch (max %d)\n", dim, AX_NOALLOC_MAX_DIM);
        return 201;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= AX_NOALLOC_MAX_DEVICES) return 203;
    if (!g_noalloc_addr[dev]) {
        // first call on this device: resolve the array's device address (not a stream operation;
        // make this first call before any stream capture starts)
        float* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, g_noalloc_partials) != cudaSuccess || !p) { cudaGetLastError(); return 203; }
        g_noalloc_addr[dev] = p;
    }
    cudaGetLastError();       // an earlier, unrelated error of this thread must not be reported as this call's (204)
    if (rows == 0) {          // an empty batch: dx has no rows and the column sums are zero
        if (dw && cudaMemsetAsync(dw, 0, (size_t)dim * sizeof(float), (cudaStream_t)stream) != cudaSuccess) { cudaGetLastError(); return 204; }
        return 0;
    }
    // Nothing in the scratch has to start at zero: the first kernel overwrites rows
    // [0, blocks) x [0, dim) of it and the second reads exactly those.
    const int rc = ax_rmsnorm_bwd_acc(dt, x, w, g, res, dx, dw, g_noalloc_addr[dev], rows, dim, eps, (cudaStream_t)stream, 0);
    if (rc) return rc;
    return cudaGetLastError() == cudaSuccess ? 0 : 204;
}
