// Optimizer: global-norm clipping + decoupled AdamW on fp32 masters with an
// optional bf16 mirror.  Per-tensor kernels serve the reference ABI; the flat
// kernels make the whole update one bandwidth-bound pass over a parameter
// arena (g read twice, p/m/v read+written once, mirror written once).
#include "common.cuh"
#include "kernels.h"

#define B1 0.9f
#define B2 0.95f

struct AdamScalars { float step, eps, decay; };

// Bias correction folded into the step size and epsilon:
//   p -= lr*sqrt(bc2)/bc1 * m / (sqrt(v) + eps*sqrt(bc2))   ==   lr * (m/bc1) / (sqrt(v/bc2) + eps)
__device__ __forceinline__ AdamScalars adam_scalars(float lr, float wd, float eps, const float* tbuf) {
    AdamScalars s;
    if (tbuf) {
        const double t = (double)tbuf[0];
        const double bc1 = 1.0 - pow((double)B1, t), bc2 = 1.0 - pow((double)B2, t);
        s.step = (float)((double)lr * sqrt(bc2) / bc1);
        s.eps = (float)((double)eps * sqrt(bc2));
    } else { s.step = lr; s.eps = eps; }
    s.decay = 1.f - lr * wd;
    return s;
}

__global__ void k_adamw(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                        float* __restrict__ v, const float* tbuf, bf16* __restrict__ pbf,
                        const float* lrbuf, const float* gsbuf, float alpha, float beta, float gamma,
                        long long n, int vec) {
    __shared__ AdamScalars sc;
    __shared__ float s_gs;
    if (threadIdx.x == 0) {
        sc = adam_scalars(lrbuf ? lrbuf[0] : alpha, beta, gamma, tbuf);
        s_gs = gsbuf ? gsbuf[0] : 1.f;
    }
    __syncthreads();
    const float step = sc.step, eps = sc.eps, decay = sc.decay, gs = s_gs;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long start = 0;
    if (vec) {
        const long long nv = n / 4;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
            float pp[4], gg[4], mm[4], vv[4];
            Vec<float>::ld(p + i * 4, pp); Vec<float>::ld(g + i * 4, gg);
            Vec<float>::ld(m + i * 4, mm); Vec<float>::ld(v + i * 4, vv);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float gi = gg[q] * gs;
                mm[q] = B1 * mm[q] + (1.f - B1) * gi;
                vv[q] = B2 * vv[q] + (1.f - B2) * gi * gi;
                pp[q] = pp[q] * decay - step * mm[q] / (sqrtf(vv[q]) + eps);
            }
            Vec<float>::st(p + i * 4, pp); Vec<float>::st(m + i * 4, mm); Vec<float>::st(v + i * 4, vv);
            if (pbf) {
                __nv_bfloat162 h0 = __floats2bfloat162_rn(pp[0], pp[1]), h1 = __floats2bfloat162_rn(pp[2], pp[3]);
                uint2 u; u.x = *reinterpret_cast<unsigned*>(&h0); u.y = *reinterpret_cast<unsigned*>(&h1);
                *reinterpret_cast<uint2*>(pbf + i * 4) = u;
            }
        }
        start = nv * 4;
    }
    for (long long i = start + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float gi = g[i] * gs;
        const float mi = B1 * m[i] + (1.f - B1) * gi;
        const float vi = B2 * v[i] + (1.f - B2) * gi * gi;
        m[i] = mi; v[i] = vi;
        const float pi = p[i] * decay - step * mi / (sqrtf(vi) + eps);
        p[i] = pi;
        if (pbf) pbf[i] = __float2bfloat16(pi);
    }
}
int ax_adamw(float* p, const float* g, float* m, float* v, const float* tbuf, void* pbf,
             const float* lrbuf, const float* gsbuf, float alpha, float beta, float gamma, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const int vec = aligned16(p) && aligned16(g) && aligned16(m) && aligned16(v) &&
                    (!pbf || (reinterpret_cast<uintptr_t>(pbf) & 7) == 0);
    k_adamw<<<ew_grid(n / 4 + 1, 256), 256, 0, st>>>(p, g, m, v, tbuf, (bf16*)pbf, lrbuf, gsbuf, alpha, beta, gamma, n, vec);
    return 0;
}

// sum of squares -> atomicAdd(acc) (reference ABI; caller zeroes acc first)
__global__ void k_l2acc(const float* g, float* acc, long long n) {
    __shared__ float sh[40];
    float s = 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)blockDim.x * gridDim.x) s += g[i] * g[i];
    s = block_sum(s, sh);
    if (threadIdx.x == 0) atomicAdd(acc, s);
}
int ax_l2acc(const float* g, float* acc, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    long long blocks = (n + 255) / 256; if (blocks > 1024) blocks = 1024;
    k_l2acc<<<(int)blocks, 256, 0, st>>>(g, acc, n);
    return 0;
}
__global__ void k_clipscale(const float* acc, float* scale, float max_norm) {
    const float nrm = sqrtf(acc[0]);
    scale[0] = (max_norm > 0.f && nrm > max_norm) ? max_norm / (nrm + 1e-6f) : 1.f;
}
int ax_clipscale(const float* acc, float* scale, float max_norm, cudaStream_t st) {
    k_clipscale<<<1, 1, 0, st>>>(acc, scale, max_norm);
    return 0;
}
__global__ void k_tick(float* t) { t[0] += 1.f; }
int ax_tick(float* t, cudaStream_t st) { k_tick<<<1, 1, 0, st>>>(t); return 0; }

// ── flat arena ──────────────────────────────────────────────────────────────
// partials[c] = sum of g^2 over chunk c (AX_GNORM_CHUNK elements).  One block
// per chunk with a fixed in-block order, so the value of a partial depends
// only on the data, never on the grid or the scheduling.
__global__ void k_gnorm_flat(const float* __restrict__ g, float* __restrict__ partials, long long n, float* tick) {
    __shared__ float sh[40];
    const long long nchunks = (n + AX_GNORM_CHUNK - 1) / AX_GNORM_CHUNK;
    if (tick && blockIdx.x == 0 && threadIdx.x == 0) tick[0] += 1.f;
    for (long long c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const long long base = c * AX_GNORM_CHUNK;
        float s = 0.f;
#pragma unroll
        for (int it = 0; it < AX_GNORM_CHUNK / (256 * 4); it++) {
            const long long i = base + (long long)(it * 256 + threadIdx.x) * 4;
            if (i + 3 < n) {
                const float4 x = *reinterpret_cast<const float4*>(g + i);
                s += x.x * x.x; s += x.y * x.y; s += x.z * x.z; s += x.w * x.w;
            } else {
                for (long long j = i; j < n && j < i + 4; j++) s += g[j] * g[j];
            }
        }
        s = block_sum(s, sh);
        if (threadIdx.x == 0) partials[c] = s;
        __syncthreads();
    }
}
// out[0] = sum of np partials: thread t adds partials t, t+1024, ... in order,
// then a fixed tree — the result depends on the values only.
__global__ void k_sum_partials(const float* __restrict__ partials, long long np, float* out) {
    __shared__ float sh[40];
    float acc = 0.f;
    for (long long i = threadIdx.x; i < np; i += blockDim.x) acc += partials[i];
    acc = block_sum(acc, sh);
    if (threadIdx.x == 0) out[0] = acc;
}
int ax_gnorm_flat(const float* g, float* partials, long long n, float* tick, float* out, cudaStream_t st) {
    if (n <= 0) {
        if (tick) k_tick<<<1, 1, 0, st>>>(tick);
        if (out) cudaMemsetAsync(out, 0, 4, st);
        return 0;
    }
    if (!aligned16(g)) return 121;
    const long long nchunks = (n + AX_GNORM_CHUNK - 1) / AX_GNORM_CHUNK;
    const int grid = (int)(nchunks < AX_SMS * 8 ? nchunks : AX_SMS * 8);
    k_gnorm_flat<<<grid, 256, 0, st>>>(g, partials, n, tick);
    if (out) k_sum_partials<<<1, 1024, 0, st>>>(partials, nchunks, out);
    return 0;
}

// Every block first adds the np partials in index order (same value in every
// block), derives the clip factor, then updates its slice.  wdflag has one
// byte per AX_ADAMW_CHUNK elements: 1 = apply weight decay (tensors with two
// or more dimensions), 0 = exempt.
__global__ void k_adamw_flat(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, bf16* __restrict__ pbf,
                             const unsigned char* __restrict__ wdflag, const float* tbuf, const float* lrbuf,
                             const float* __restrict__ partials, int np, float* gnorm_out,
                             float max_norm, float wd, float eps, long long n) {
    __shared__ float sh[40];
    __shared__ AdamScalars sc;
    __shared__ float s_gs;
    float acc = 0.f;
    // fixed order: thread t sums partials t, t+256, ...; then the block tree
    for (int i = threadIdx.x; i < np; i += blockDim.x) acc += partials[i];
    acc = block_sum(acc, sh);
    if (threadIdx.x == 0) {
        const float nrm = sqrtf(acc);
        s_gs = (max_norm > 0.f && nrm > max_norm) ? max_norm / nrm : 1.f;
        sc = adam_scalars(lrbuf[0], wd, eps, tbuf);
        if (gnorm_out && blockIdx.x == 0) gnorm_out[0] = nrm;
    }
    __syncthreads();
    const float step = sc.step, e = sc.eps, decay_on = sc.decay, gs = s_gs;
    const long long nv = n / 4;                       // n is a multiple of AX_ADAMW_CHUNK
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
        const float decay = wdflag[(i * 4) / AX_ADAMW_CHUNK] ? decay_on : 1.f;
        float pp[4], gg[4], mm[4], vv[4];
        Vec<float>::ld(p + i * 4, pp); Vec<float>::ld(g + i * 4, gg);
        Vec<float>::ld(m + i * 4, mm); Vec<float>::ld(v + i * 4, vv);
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const float gi = gg[q] * gs;
            mm[q] = B1 * mm[q] + (1.f - B1) * gi;
            vv[q] = B2 * vv[q] + (1.f - B2) * gi * gi;
            pp[q] = pp[q] * decay - step * mm[q] / (sqrtf(vv[q]) + e);
        }
        Vec<float>::st(p + i * 4, pp); Vec<float>::st(m + i * 4, mm); Vec<float>::st(v + i * 4, vv);
        if (pbf) {
            __nv_bfloat162 h0 = __floats2bfloat162_rn(pp[0], pp[1]), h1 = __floats2bfloat162_rn(pp[2], pp[3]);
            uint2 u; u.x = *reinterpret_cast<unsigned*>(&h0); u.y = *reinterpret_cast<unsigned*>(&h1);
            *reinterpret_cast<uint2*>(pbf + i * 4) = u;
        }
    }
}
int ax_adamw_flat(float* p, const float* g, float* m, float* v, void* pbf, const unsigned char* wdflag,
                  const float* tbuf, const float* lrbuf, const float* partials, int np, float* gnorm_out,
                  float max_norm, float wd, float eps, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    if (n % AX_ADAMW_CHUNK) return 122;
    if (!(aligned16(p) && aligned16(g) && aligned16(m) && aligned16(v))) return 121;
    k_adamw_flat<<<ew_grid(n / 4, 256), 256, 0, st>>>(p, g, m, v, (bf16*)pbf, wdflag, tbuf, lrbuf, partials, np,
                                                    gnorm_out, max_norm, wd, eps, n);
    return 0;
}
