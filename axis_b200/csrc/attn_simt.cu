// Causal grouped-query attention on CUDA cores with exact fp32 arithmetic —
// the parity-mode path (fp32 storage, any head_dim <= 256, any T) and the
// general path for shapes the tensor-core kernels do not take.  Layout is
// given by element strides, so [B,H,T,DH] and [B,T,H,DH] are both served.
// No atomics: dK/dV are accumulated per key row over the whole query group.
#include "common.cuh"
#include "kernels.h"

#define AW 8            // warps per block = rows per block
#define AKT 32          // keys (or queries) per shared-memory tile
#define ADMAX 8         // head_dim <= 32 * ADMAX

template <typename T>
__global__ void __launch_bounds__(AW * 32)
k_attn_fwd_simt(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ o,
                float* __restrict__ lse, AttnShape s) {
    extern __shared__ float smem[];
    const int DH = s.DH, LD = DH + 1;
    float* Ks = smem;                    // AKT x LD
    float* Vs = Ks + AKT * LD;           // AKT x LD
    float* Qs = Vs + AKT * LD;           // AW x DH
    const int b = blockIdx.z, h = blockIdx.y, g = h / (s.H / s.KV);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * AW + warp;
    const bool live = t < s.T;
    const T* qrow = q + b * s.qb + h * s.qh + (long long)t * s.qt;
    const T* kbase = k + b * s.kb + g * s.kh;
    const T* vbase = v + b * s.kb + g * s.kh;
    if (live) for (int d = lane; d < DH; d += 32) Qs[warp * DH + d] = ldf(qrow, d);
    float m = -3.0e38f, l = 0.f, acc[ADMAX];
#pragma unroll
    for (int i = 0; i < ADMAX; i++) acc[i] = 0.f;
    const int tmax = min(blockIdx.x * AW + AW - 1, s.T - 1);
    const int ntiles = tmax / AKT + 1;
    for (int kt = 0; kt < ntiles; kt++) {
        __syncthreads();
        for (int e = threadIdx.x; e < AKT * DH; e += blockDim.x) {
            const int r = e / DH, d = e % DH, key = kt * AKT + r;
            const bool in = key < s.T;
            Ks[r * LD + d] = in ? ldf(kbase, (long long)key * s.kt + d) : 0.f;
            Vs[r * LD + d] = in ? ldf(vbase, (long long)key * s.kt + d) : 0.f;
        }
        __syncthreads();
        if (!live || kt * AKT > t) continue;
        const int key = kt * AKT + lane;
        float sc = -3.0e38f;
        if (key <= t) {
            float dot = 0.f;
            for (int d = 0; d < DH; d++) dot = fmaf(Qs[warp * DH + d], Ks[lane * LD + d], dot);
            sc = dot * s.scale;
        }
        const float mn = fmaxf(m, warp_max(sc));
        const float p = key <= t ? expf(sc - mn) : 0.f;
        const float corr = expf(m - mn);
        l = l * corr + warp_sum(p);
        m = mn;
#pragma unroll
        for (int i = 0; i < ADMAX; i++) acc[i] *= corr;
        for (int j = 0; j < AKT; j++) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
            for (int i = 0; i < ADMAX; i++) {
                const int d = lane + 32 * i;
                if (d < DH) acc[i] = fmaf(pj, Vs[j * LD + d], acc[i]);
            }
        }
    }
    if (live) {
        T* orow = o + b * s.qb + h * s.qh + (long long)t * s.qt;
        const float il = 1.f / l;
#pragma unroll
        for (int i = 0; i < ADMAX; i++) {
            const int d = lane + 32 * i;
            if (d < DH) stf(orow, d, acc[i] * il);
        }
        if (lse && lane == 0) lse[((long long)b * s.H + h) * s.T + t] = m + logf(l);
    }
}

// dQ: one warp per query row.
template <typename T, typename TO>
__global__ void __launch_bounds__(AW * 32)
k_attn_bwd_dq_simt(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const T* __restrict__ dO, const float* __restrict__ lse, const float* __restrict__ Dv,
                   TO* __restrict__ dq, AttnShape s) {
    extern __shared__ float smem[];
    const int DH = s.DH, LD = DH + 1;
    float* Ks = smem;
    float* Vs = Ks + AKT * LD;
    float* Qs = Vs + AKT * LD;           // AW x DH
    float* Gs = Qs + AW * DH;            // AW x DH  (dO rows)
    const int b = blockIdx.z, h = blockIdx.y, g = h / (s.H / s.KV);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * AW + warp;
    const bool live = t < s.T;
    const long long roff = b * s.qb + h * s.qh + (long long)t * s.qt;
    const T* kbase = k + b * s.kb + g * s.kh;
    const T* vbase = v + b * s.kb + g * s.kh;
    float L = 0.f, Dr = 0.f;
    if (live) {
        for (int d = lane; d < DH; d += 32) { Qs[warp * DH + d] = ldf(q, roff + d); Gs[warp * DH + d] = ldf(dO, roff + d); }
        L = lse[((long long)b * s.H + h) * s.T + t];
        Dr = Dv[b * s.db + h * s.dh_ + (long long)t * s.dtk];
    }
    float acc[ADMAX];
#pragma unroll
    for (int i = 0; i < ADMAX; i++) acc[i] = 0.f;
    const int tmax = min(blockIdx.x * AW + AW - 1, s.T - 1);
    const int ntiles = tmax / AKT + 1;
    for (int kt = 0; kt < ntiles; kt++) {
        __syncthreads();
        for (int e = threadIdx.x; e < AKT * DH; e += blockDim.x) {
            const int r = e / DH, d = e % DH, key = kt * AKT + r;
            const bool in = key < s.T;
            Ks[r * LD + d] = in ? ldf(kbase, (long long)key * s.kt + d) : 0.f;
            Vs[r * LD + d] = in ? ldf(vbase, (long long)key * s.kt + d) : 0.f;
        }
        __syncthreads();
        if (!live || kt * AKT > t) continue;
        const int key = kt * AKT + lane;
        float ds = 0.f;
        if (key <= t) {
            float dot = 0.f, dp = 0.f;
            for (int d = 0; d < DH; d++) {
                dot = fmaf(Qs[warp * DH + d], Ks[lane * LD + d], dot);
                dp = fmaf(Gs[warp * DH + d], Vs[lane * LD + d], dp);
            }
            const float p = expf(dot * s.scale - L);
            ds = p * (dp - Dr) * s.scale;
        }
        for (int j = 0; j < AKT; j++) {
            const float dj = __shfl_sync(0xffffffffu, ds, j);
#pragma unroll
            for (int i = 0; i < ADMAX; i++) {
                const int d = lane + 32 * i;
                if (d < DH) acc[i] = fmaf(dj, Ks[j * LD + d], acc[i]);
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < ADMAX; i++) {
            const int d = lane + 32 * i;
            if (d < DH) stf(dq, roff + d, acc[i]);
        }
    }
}

// dK, dV: one warp per key row of a kv head; loops over the group's query
// heads and the causal query tiles — this is where the GQA sum happens.
template <typename T, typename TO>
__global__ void __launch_bounds__(AW * 32)
k_attn_bwd_dkv_simt(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                    const T* __restrict__ dO, const float* __restrict__ lse, const float* __restrict__ Dv,
                    TO* __restrict__ dk, TO* __restrict__ dv, AttnShape s) {
    extern __shared__ float smem[];
    const int DH = s.DH, LD = DH + 1;
    float* Qs = smem;                    // AKT x LD
    float* Gs = Qs + AKT * LD;           // AKT x LD
    float* Kr = Gs + AKT * LD;           // AW x DH
    float* Vr = Kr + AW * DH;            // AW x DH
    float* Ls = Vr + AW * DH;            // AKT
    float* Ds = Ls + AKT;                // AKT
    const int b = blockIdx.z, g = blockIdx.y, rep = s.H / s.KV;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x * AW + warp;            // key row
    const bool live = j < s.T;
    const long long koff = b * s.kb + g * s.kh + (long long)j * s.kt;
    if (live) for (int d = lane; d < DH; d += 32) { Kr[warp * DH + d] = ldf(k, koff + d); Vr[warp * DH + d] = ldf(v, koff + d); }
    float ak[ADMAX], av[ADMAX];
#pragma unroll
    for (int i = 0; i < ADMAX; i++) { ak[i] = 0.f; av[i] = 0.f; }
    const int qt0 = (blockIdx.x * AW) / AKT;
    const int nqt = (s.T + AKT - 1) / AKT;
    for (int hh = 0; hh < rep; hh++) {
        const int h = g * rep + hh;
        const long long hb = b * s.qb + h * s.qh;
        for (int qt = qt0; qt < nqt; qt++) {
            __syncthreads();
            for (int e = threadIdx.x; e < AKT * DH; e += blockDim.x) {
                const int r = e / DH, d = e % DH, t = qt * AKT + r;
                const bool in = t < s.T;
                Qs[r * LD + d] = in ? ldf(q, hb + (long long)t * s.qt + d) : 0.f;
                Gs[r * LD + d] = in ? ldf(dO, hb + (long long)t * s.qt + d) : 0.f;
            }
            if (threadIdx.x < AKT) {
                const int t = qt * AKT + threadIdx.x;
                const bool in = t < s.T;
                Ls[threadIdx.x] = in ? lse[((long long)b * s.H + h) * s.T + t] : 0.f;
                Ds[threadIdx.x] = in ? Dv[b * s.db + h * s.dh_ + (long long)t * s.dtk] : 0.f;
            }
            __syncthreads();
            if (!live) continue;
            const int t = qt * AKT + lane;
            float p = 0.f, ds = 0.f;
            if (t < s.T && t >= j) {
                float dot = 0.f, dp = 0.f;
                for (int d = 0; d < DH; d++) {
                    dot = fmaf(Qs[lane * LD + d], Kr[warp * DH + d], dot);
                    dp = fmaf(Gs[lane * LD + d], Vr[warp * DH + d], dp);
                }
                p = expf(dot * s.scale - Ls[lane]);
                ds = p * (dp - Ds[lane]) * s.scale;
            }
            for (int i2 = 0; i2 < AKT; i2++) {
                const float pj = __shfl_sync(0xffffffffu, p, i2);
                const float dj = __shfl_sync(0xffffffffu, ds, i2);
#pragma unroll
                for (int i = 0; i < ADMAX; i++) {
                    const int d = lane + 32 * i;
                    if (d < DH) { av[i] = fmaf(pj, Gs[i2 * LD + d], av[i]); ak[i] = fmaf(dj, Qs[i2 * LD + d], ak[i]); }
                }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < ADMAX; i++) {
            const int d = lane + 32 * i;
            if (d < DH) { stf(dk, koff + d, ak[i]); stf(dv, koff + d, av[i]); }
        }
    }
}

static bool attn_smem_ok(size_t bytes, const void* fn) {
    if (bytes > 200 * 1024) return false;
    if (bytes > 48 * 1024) cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    return true;
}

int ax_attn_fwd_simt(int dt, const void* q, const void* k, const void* v, void* o, float* lse,
                     const AttnShape& s, cudaStream_t st) {
    if (s.DH > 32 * ADMAX || s.DH < 1 || s.KV < 1 || s.H % s.KV) return 101;
    if (s.B <= 0 || s.T <= 0) return 0;
    const size_t smem = ((size_t)2 * AKT * (s.DH + 1) + (size_t)AW * s.DH) * 4;
    dim3 grid((s.T + AW - 1) / AW, s.H, s.B);
    if (dt == 1) {
        if (!attn_smem_ok(smem, (const void*)k_attn_fwd_simt<bf16>)) return 101;
        k_attn_fwd_simt<bf16><<<grid, AW * 32, smem, st>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, (bf16*)o, lse, s);
    } else {
        if (!attn_smem_ok(smem, (const void*)k_attn_fwd_simt<float>)) return 101;
        k_attn_fwd_simt<float><<<grid, AW * 32, smem, st>>>((const float*)q, (const float*)k, (const float*)v, (float*)o, lse, s);
    }
    return 0;
}

template <typename T, typename TO>
static int attn_bwd_launch(const void* q, const void* k, const void* v, const void* dO, const float* lse,
                           const float* Dv, void* dq, void* dk, void* dv, const AttnShape& s, cudaStream_t st) {
    const size_t sm1 = ((size_t)2 * AKT * (s.DH + 1) + (size_t)2 * AW * s.DH) * 4;
    const size_t sm2 = ((size_t)2 * AKT * (s.DH + 1) + (size_t)2 * AW * s.DH + 2 * AKT) * 4;
    if (!attn_smem_ok(sm1, (const void*)k_attn_bwd_dq_simt<T, TO>)) return 102;
    if (!attn_smem_ok(sm2, (const void*)k_attn_bwd_dkv_simt<T, TO>)) return 102;
    dim3 g1((s.T + AW - 1) / AW, s.H, s.B), g2((s.T + AW - 1) / AW, s.KV, s.B);
    k_attn_bwd_dq_simt<T, TO><<<g1, AW * 32, sm1, st>>>((const T*)q, (const T*)k, (const T*)v, (const T*)dO, lse, Dv, (TO*)dq, s);
    k_attn_bwd_dkv_simt<T, TO><<<g2, AW * 32, sm2, st>>>((const T*)q, (const T*)k, (const T*)v, (const T*)dO, lse, Dv, (TO*)dk, (TO*)dv, s);
    return 0;
}
int ax_attn_bwd_simt(int dt, int out_dt, const void* q, const void* k, const void* v, const void* dO,
                     const float* lse, const float* Dv, void* dq, void* dk, void* dv,
                     const AttnShape& s, cudaStream_t st) {
    if (s.DH > 32 * ADMAX || s.DH < 1 || s.KV < 1 || s.H % s.KV) return 102;
    if (s.B <= 0 || s.T <= 0) return 0;
    if (dt == 1 && out_dt == 1) return attn_bwd_launch<bf16, bf16>(q, k, v, dO, lse, Dv, dq, dk, dv, s, st);
    if (dt == 1) return attn_bwd_launch<bf16, float>(q, k, v, dO, lse, Dv, dq, dk, dv, s, st);
    if (out_dt == 0) return attn_bwd_launch<float, float>(q, k, v, dO, lse, Dv, dq, dk, dv, s, st);
    return 102;
}
