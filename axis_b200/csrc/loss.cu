// Index-based ops: embedding gather / scatter-add, valid-target count and
// token-mean cross-entropy with ignored targets (target < 0).
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

// ── embedding gather: o[r,:] = table[ids[r],:] ─────────────────────────────
// An id outside [0, rows) never reaches the table: its output row is zero-filled and the status word is set.
#define STAT_INDEX 0x400       // + 1 gather id, 2 scatter id, 3 cross-entropy target
template <typename T, typename I, int W>
__global__ void k_embed(const T* __restrict__ table, const I* __restrict__ ids, T* __restrict__ o,
                        int N, int Dw, int rows, int* status) {
    const long long total = (long long)N * Dw;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int r = (int)(i / Dw), j = (int)(i % Dw);
        const int id = (int)ids[r];
        if (id < 0 || id >= rows) {
            if (j == 0 && status) atomicExch(status, STAT_INDEX | 1);
            if (W == 1) o[i] = T(0.f);
            else reinterpret_cast<uint4*>(o)[i] = make_uint4(0, 0, 0, 0);
            continue;
        }
        const long long src = (long long)id * Dw + j;
        if (W == 1) o[i] = table[src];
        else reinterpret_cast<uint4*>(o)[i] = reinterpret_cast<const uint4*>(table)[src];
    }
}
template <typename T, typename I>
static void embed_launch(const void* table, const void* ids, void* o, int N, int D, int rows, int* status, cudaStream_t st) {
    constexpr int per = 16 / sizeof(T);
    if (D % per == 0 && aligned16(table) && aligned16(o))
        k_embed<T, I, per><<<ew_grid((long long)N * (D / per), 256), 256, 0, st>>>((const T*)table, (const I*)ids, (T*)o, N, D / per, rows, status);
    else
        k_embed<T, I, 1><<<ew_grid((long long)N * D, 256), 256, 0, st>>>((const T*)table, (const I*)ids, (T*)o, N, D, rows, status);
}
int ax_embed(int dt, const void* table, const void* ids, int ids_i32, void* o, int N, int D, int rows, int* status, cudaStream_t st) {
    if (N <= 0 || D <= 0) return 0;
    if (dt == 1) { if (ids_i32) embed_launch<bf16, int>(table, ids, o, N, D, rows, status, st); else embed_launch<bf16, float>(table, ids, o, N, D, rows, status, st); }
    else { if (ids_i32) embed_launch<float, int>(table, ids, o, N, D, rows, status, st); else embed_launch<float, float>(table, ids, o, N, D, rows, status, st); }
    return 0;
}

// ── scatter-add with fp32 atomics (reference ABI; summation order varies) ──
template <typename T>
__global__ void k_embed_bwd_atomic(const T* g, const float* ids, float* dT, int N, int D, int rows, int* status) {
    const long long total = (long long)N * D;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int r = (int)(i / D), j = (int)(i % D);
        const int id = (int)ids[r];
        if (id < 0 || id >= rows) {                     // the row is skipped, the table gradient untouched
            if (j == 0 && status) atomicExch(status, STAT_INDEX | 2);
            continue;
        }
        atomicAdd(&dT[(long long)id * D + j], ldf(g, i));
    }
}
int ax_embed_bwd_atomic(int g_bf16, const void* g, const float* ids, float* dT, int N, int D, int rows, int* status, cudaStream_t st) {
    if (N <= 0 || D <= 0) return 0;
    if (g_bf16) k_embed_bwd_atomic<bf16><<<ew_grid((long long)N * D, 256), 256, 0, st>>>((const bf16*)g, ids, dT, N, D, rows, status);
    else k_embed_bwd_atomic<float><<<ew_grid((long long)N * D, 256), 256, 0, st>>>((const float*)g, ids, dT, N, D, rows, status);
    return 0;
}

// ── ordered scatter-add without atomics ─────────────────────────────────────
// Block r acts only when row r is the first occurrence of its token; it then
// walks the later occurrences in row order and adds their gradient rows to
// dT[token] — the same order as a sequential scatter-add, every run.
template <typename T>
__global__ void k_embed_bwd_det(const T* __restrict__ g, const int* __restrict__ ids, float* dT, int N, int D, int rows, int* status) {
    __shared__ int s_flag;
    __shared__ int s_list[256];
    __shared__ int s_cnt;
    __shared__ int s_wcnt[8];
    for (int r = blockIdx.x; r < N; r += gridDim.x) {
        const int tok = ids[r];
        if (threadIdx.x == 0) s_flag = 0;
        __syncthreads();
        int seen = 0;
        for (int i = threadIdx.x; i < r; i += blockDim.x) seen |= (ids[i] == tok);
        if (seen) s_flag = 1;
        __syncthreads();
        const bool first = s_flag == 0;
        __syncthreads();
        if (tok >= rows && first && threadIdx.x == 0 && status) atomicExch(status, STAT_INDEX | 2);
        if (!first || tok < 0 || tok >= rows) continue;      // ids outside the table are skipped, nothing is written
        // gather the occurrences >= r in order, 256 at a time
        for (int base = r; base < N; base += 256) {
            if (threadIdx.x == 0) s_cnt = 0;
            __syncthreads();
            // ordered compaction of matches in [base, base+256)
            const int idx = base + (int)threadIdx.x;
            const int hit = (threadIdx.x < 256 && idx < N && ids[idx] == tok) ? 1 : 0;
            // ballot-based ordered positions (blockDim.x == 256 -> 8 warps)
            const unsigned bal = __ballot_sync(0xffffffffu, hit);
            const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
            if (!lane) s_wcnt[wp] = __popc(bal);
            __syncthreads();
            int off = 0;
            for (int q = 0; q < wp; q++) off += s_wcnt[q];
            if (hit) s_list[off + __popc(bal & ((1u << lane) - 1))] = idx;
            if (threadIdx.x == 0) { int t = 0; for (int q = 0; q < 8; q++) t += s_wcnt[q]; s_cnt = t; }
            __syncthreads();
            const int cnt = s_cnt;
            for (int j = threadIdx.x; j < D; j += blockDim.x) {
                float acc = 0.f;
                for (int q = 0; q < cnt; q++) acc += ldf(g, (long long)s_list[q] * D + j);
                if (cnt) dT[(long long)tok * D + j] += acc;
            }
            __syncthreads();
        }
    }
}
int ax_embed_bwd_det(int g_dt, const void* g, const int* ids, float* dT, int N, int D, int rows, int* status, cudaStream_t st) {
    if (N <= 0 || D <= 0) return 0;
    const int grid = N < AX_SMS * 16 ? N : AX_SMS * 16;
    if (g_dt >= 1) k_embed_bwd_det<bf16><<<grid, 256, 0, st>>>((const bf16*)g, ids, dT, N, D, rows, status);
    else k_embed_bwd_det<float><<<grid, 256, 0, st>>>((const float*)g, ids, dT, N, D, rows, status);
    return 0;
}

// ── count of valid targets (float accumulator, exact below 2^24) ───────────
__global__ void k_countvalid(const float* tgt, float* acc, int N) {
    __shared__ float sh[40];
    float s = 0.f;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += blockDim.x * gridDim.x) s += (tgt[i] >= 0.f) ? 1.f : 0.f;
    s = block_sum(s, sh);
    if (threadIdx.x == 0 && s != 0.f) atomicAdd(acc, s);
}
int ax_countvalid(const float* tgt, float* acc, int N, cudaStream_t st) {
    if (N <= 0) return 0;
    int blocks = (N + 255) / 256; if (blocks > 1024) blocks = 1024;
    k_countvalid<<<blocks, 256, 0, st>>>(tgt, acc, N);
    return 0;
}

// ── cross-entropy rows ──────────────────────────────────────────────────────
// One block per row.  Pass 1 keeps a running (max, sum) per thread — a single
// read of the row; pass 2 writes (softmax - onehot) * inv_count.  Safe in
// place (dlogits == logits): pass 2 starts after the block-wide reduction, and
// every element is re-read by the thread that overwrites it.
// Reference ABI (kind CE): fp32 targets, denom buffer optional, loss via one
// atomicAdd per row.
template <typename T, bool VEC>
__global__ void k_ce(const T* logits, const float* tgt, T* dlogits, float* loss, const float* denom, int Nrows, int V, int* status) {
    __shared__ float sh[40];
    __shared__ float s_xt;
    for (int r = blockIdx.x; r < Nrows; r += gridDim.x) {
        const T* lr = logits + (long long)r * V;
        T* dr = dlogits + (long long)r * V;
        int t = (int)tgt[r];
        if (t >= V) {                    // a target outside the vocabulary: the row counts as ignored
            if (threadIdx.x == 0 && status) atomicExch(status, STAT_INDEX | 3);
            t = -1;
        }
        if (t < 0) {
            for (int j = threadIdx.x; j < V; j += blockDim.x) stf(dr, j, 0.f);
            continue;
        }
        if (threadIdx.x == 0) s_xt = ldf(lr, t);       // before any in-place overwrite
        __syncthreads();
        const float inv = denom ? 1.f / denom[0] : 1.f / Nrows;
        constexpr int N = Vec<T>::N;
        float m = -3.0e38f, s = 0.f;
        if (VEC) {
            for (int j = threadIdx.x * N; j < V; j += blockDim.x * N) {
                float f[N];
                Vec<T>::ld(lr + j, f);
                float mx = f[0];
#pragma unroll
                for (int q = 1; q < N; q++) mx = fmaxf(mx, f[q]);
                if (mx > m) { s *= expf(m - mx); m = mx; }
#pragma unroll
                for (int q = 0; q < N; q++) s += expf(f[q] - m);
            }
        } else {
            for (int j = threadIdx.x; j < V; j += blockDim.x) {
                const float f = ldf(lr, j);
                if (f > m) { s *= expf(m - f); m = f; }
                s += expf(f - m);
            }
        }
        const float M = block_max(m, sh);
        s = (m > -3.0e38f) ? s * expf(m - M) : 0.f;
        const float S = block_sum(s, sh);
        const float invS = 1.f / S;
        if (VEC) {
            for (int j = threadIdx.x * N; j < V; j += blockDim.x * N) {
                float f[N];
                Vec<T>::ld(lr + j, f);
#pragma unroll
                for (int q = 0; q < N; q++) f[q] = (expf(f[q] - M) * invS - ((j + q) == t ? 1.f : 0.f)) * inv;
                Vec<T>::st(dr + j, f);
            }
        } else {
            for (int j = threadIdx.x; j < V; j += blockDim.x)
                stf(dr, j, (expf(ldf(lr, j) - M) * invS - (j == t ? 1.f : 0.f)) * inv);
        }
        if (threadIdx.x == 0) atomicAdd(loss, (logf(S) - (s_xt - M)) * inv);
        __syncthreads();
    }
}
int ax_ce(int dt, const void* logits, const float* tgt, void* dlogits, float* loss, const float* denom, int N, int V, int* status, cudaStream_t st) {
    if (N <= 0 || V <= 0) return 0;
    const int per = dt == 1 ? 8 : 4;
    const bool vec = V % per == 0 && aligned16(logits) && aligned16(dlogits);
    const int thr = V >= 4096 ? 512 : 256;
    const int grid = N < AX_SMS * 64 ? N : AX_SMS * 64;
    if (dt == 1) {
        if (vec) k_ce<bf16, true><<<grid, thr, 0, st>>>((const bf16*)logits, tgt, (bf16*)dlogits, loss, denom, N, V, status);
        else k_ce<bf16, false><<<grid, thr, 0, st>>>((const bf16*)logits, tgt, (bf16*)dlogits, loss, denom, N, V, status);
    } else {
        if (vec) k_ce<float, true><<<grid, thr, 0, st>>>((const float*)logits, tgt, (float*)dlogits, loss, denom, N, V, status);
        else k_ce<float, false><<<grid, thr, 0, st>>>((const float*)logits, tgt, (float*)dlogits, loss, denom, N, V, status);
    }
    return 0;
}

// ── fused, deterministic form ───────────────────────────────────────────────
// k_ce_prepare: one block counts the valid targets (integer), stores the count
// as float in denom[0], zeroes the done-counter.  k_ce_rows: as k_ce, but the
// row keeps its loss term in rowloss[r]; the last block to finish adds the N
// terms in a fixed order and writes loss[0].
__global__ void k_ce_prepare(const int* tgt, float* denom, float* loss, unsigned int* counter, int N, int V) {
    __shared__ int sh_i[32];
    int c = 0;
    for (int i = threadIdx.x; i < N; i += blockDim.x) c += tgt[i] >= 0 && tgt[i] < V;
    for (int o = 16; o; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0) sh_i[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int q = 0; q < (int)(blockDim.x >> 5); q++) t += sh_i[q];
        denom[0] = (float)t;
        loss[0] = 0.f;
        *counter = 0u;
    }
}
template <typename T, bool VEC>
__global__ void k_ce_rows(const T* logits, const int* tgt, T* dlogits, float* loss, const float* denom,
                          float* rowloss, unsigned int* counter, int Nrows, int V, int* status) {
    __shared__ float sh[40];
    __shared__ float s_xt;
    __shared__ bool s_last;
    constexpr int N = Vec<T>::N;
    const float inv = 1.f / denom[0];
    for (int r = blockIdx.x; r < Nrows; r += gridDim.x) {
        const T* lr = logits + (long long)r * V;
        T* dr = dlogits + (long long)r * V;
        int t = tgt[r];
        if (t >= V) {
            if (threadIdx.x == 0 && status) atomicExch(status, STAT_INDEX | 3);
            t = -1;
        }
        if (t < 0) {
            if (VEC) {
                float z[N];
#pragma unroll
                for (int q = 0; q < N; q++) z[q] = 0.f;
                for (int j = threadIdx.x * N; j < V; j += blockDim.x * N) Vec<T>::st(dr + j, z);
            } else {
                for (int j = threadIdx.x; j < V; j += blockDim.x) stf(dr, j, 0.f);
            }
            if (threadIdx.x == 0) rowloss[r] = 0.f;
            continue;
        }
        if (threadIdx.x == 0) s_xt = ldf(lr, t);
        __syncthreads();
        float m = -3.0e38f, s = 0.f;
        if (VEC) {
            for (int j = threadIdx.x * N; j < V; j += blockDim.x * N) {
                float f[N];
                Vec<T>::ld(lr + j, f);
                float mx = f[0];
#pragma unroll
                for (int q = 1; q < N; q++) mx = fmaxf(mx, f[q]);
                if (mx > m) { s *= expf(m - mx); m = mx; }
#pragma unroll
                for (int q = 0; q < N; q++) s += expf(f[q] - m);
            }
        } else {
            for (int j = threadIdx.x; j < V; j += blockDim.x) {
                const float f = ldf(lr, j);
                if (f > m) { s *= expf(m - f); m = f; }
                s += expf(f - m);
            }
        }
        const float M = block_max(m, sh);
        s = (m > -3.0e38f) ? s * expf(m - M) : 0.f;
        const float S = block_sum(s, sh);
        const float invS = 1.f / S;
        if (VEC) {
            for (int j = threadIdx.x * N; j < V; j += blockDim.x * N) {
                float f[N];
                Vec<T>::ld(lr + j, f);
#pragma unroll
                for (int q = 0; q < N; q++) f[q] = (expf(f[q] - M) * invS - ((j + q) == t ? 1.f : 0.f)) * inv;
                Vec<T>::st(dr + j, f);
            }
        } else {
            for (int j = threadIdx.x; j < V; j += blockDim.x)
                stf(dr, j, (expf(ldf(lr, j) - M) * invS - (j == t ? 1.f : 0.f)) * inv);
        }
        if (threadIdx.x == 0) rowloss[r] = logf(S) - (s_xt - M);
        __syncthreads();
    }
    // last block standing reduces the row terms in index order
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    __syncthreads();
    if (s_last) {
        __threadfence();
        float acc = 0.f;
        for (int i = threadIdx.x; i < Nrows; i += blockDim.x) acc += __ldcg(rowloss + i);
        acc = block_sum(acc, sh);
        if (threadIdx.x == 0) loss[0] = acc * inv;
    }
}
// bf16 rows of up to 512 * 8 * 8 = 32768 logits: the row is read from DRAM once into registers
// (8 packed 16-byte vectors per thread), reduced, and written back — one read and one write per element.
#define CE_VPT 8
__global__ void __launch_bounds__(512, 2)
k_ce_rows_reg(const bf16* logits, const int* __restrict__ tgt, bf16* dlogits, float* loss, const float* denom,
              float* rowloss, unsigned int* counter, int Nrows, int V, int* status) {
    __shared__ float sh[40];
    __shared__ float s_xt;
    __shared__ bool s_last;
    const float inv = 1.f / denom[0];
    const int nvec = V >> 3;
    for (int r = blockIdx.x; r < Nrows; r += gridDim.x) {
        const bf16* lr = logits + (long long)r * V;
        bf16* dr = dlogits + (long long)r * V;
        int t = tgt[r];
        if (t >= V) {
            if (threadIdx.x == 0 && status) atomicExch(status, STAT_INDEX | 3);
            t = -1;
        }
        if (t < 0) {
            const uint4 z = make_uint4(0, 0, 0, 0);
            for (int j = threadIdx.x; j < nvec; j += 512) reinterpret_cast<uint4*>(dr)[j] = z;
            if (threadIdx.x == 0) rowloss[r] = 0.f;
            continue;
        }
        uint4 pk[CE_VPT];
#pragma unroll
        for (int i = 0; i < CE_VPT; i++) {
            const int j = threadIdx.x + i * 512;
            pk[i] = j < nvec ? reinterpret_cast<const uint4*>(lr)[j] : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);  // -inf
        }
        if (threadIdx.x == 0) s_xt = __bfloat162float(lr[t]);
        float m = -3.0e38f;
#pragma unroll
        for (int i = 0; i < CE_VPT; i++) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk[i]);
#pragma unroll
            for (int q = 0; q < 4; q++) { const float2 f = __bfloat1622float2(h[q]); m = fmaxf(m, fmaxf(f.x, f.y)); }
        }
        const float M = block_max(m, sh);
        // one exponential per element: e = exp(x - M) replaces x in the same registers as packed fp16 (e <= 1,
        // 11-bit mantissa: finer than the bf16 the gradient is stored in); the sum uses the fp32 values
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < CE_VPT; i++) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk[i]);
            __half2 eh[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 f = __bfloat1622float2(h[q]);
                const float e0 = __expf(f.x - M), e1 = __expf(f.y - M);
                s += e0 + e1;
                eh[q] = __floats2half2_rn(e0, e1);
            }
            pk[i] = *reinterpret_cast<const uint4*>(eh);
        }
        const float S = block_sum(s, sh);
        const float sc = inv / S;
#pragma unroll
        for (int i = 0; i < CE_VPT; i++) {
            const int j = threadIdx.x + i * 512;
            if (j < nvec) {
                const __half2* h = reinterpret_cast<const __half2*>(&pk[i]);
                float f[8];
#pragma unroll
                for (int q = 0; q < 4; q++) { const float2 v = __half22float2(h[q]); f[2 * q] = v.x; f[2 * q + 1] = v.y; }
#pragma unroll
                for (int q = 0; q < 8; q++) f[q] = f[q] * sc - ((j * 8 + q) == t ? inv : 0.f);
                Vec<bf16>::st(dr + j * 8, f);
            }
        }
        if (threadIdx.x == 0) rowloss[r] = logf(S) - (s_xt - M);
        __syncthreads();
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    __syncthreads();
    if (s_last) {
        __threadfence();
        float acc = 0.f;
        for (int i = threadIdx.x; i < Nrows; i += blockDim.x) acc += __ldcg(rowloss + i);
        acc = block_sum(acc, sh);
        if (threadIdx.x == 0) loss[0] = acc * inv;
    }
}

int ax_ce_fused(int dt, const void* logits, const int* tgt, void* dlogits, float* loss, float* denom,
                float* scratch, int N, int V, int* status, cudaStream_t st) {
    if (N <= 0 || V <= 0) return 0;
    unsigned int* counter = reinterpret_cast<unsigned int*>(scratch);
    float* rowloss = scratch + 8;
    k_ce_prepare<<<1, 1024, 0, st>>>(tgt, denom, loss, counter, N, V);
    const int per = dt == 1 ? 8 : 4;
    const bool vec = V % per == 0 && aligned16(logits) && aligned16(dlogits);
    const int thr = V >= 4096 ? 512 : 256;
    const int grid = N < AX_SMS * 16 ? N : AX_SMS * 16;
    ax_variant = 0x10;
    if (dt == 1 && vec && V >= 2048 && V <= 512 * 8 * CE_VPT) {
        const int g2 = N < AX_SMS * 8 ? N : AX_SMS * 8;
        ax_variant = 0x11;
        k_ce_rows_reg<<<g2, 512, 0, st>>>((const bf16*)logits, tgt, (bf16*)dlogits, loss, denom, rowloss, counter, N, V, status);
        return 0;
    }
    if (dt == 1) {
        if (vec) k_ce_rows<bf16, true><<<grid, thr, 0, st>>>((const bf16*)logits, tgt, (bf16*)dlogits, loss, denom, rowloss, counter, N, V, status);
        else k_ce_rows<bf16, false><<<grid, thr, 0, st>>>((const bf16*)logits, tgt, (bf16*)dlogits, loss, denom, rowloss, counter, N, V, status);
    } else {
        if (vec) k_ce_rows<float, true><<<grid, thr, 0, st>>>((const float*)logits, tgt, (float*)dlogits, loss, denom, rowloss, counter, N, V, status);
        else k_ce_rows<float, false><<<grid, thr, 0, st>>>((const float*)logits, tgt, (float*)dlogits, loss, denom, rowloss, counter, N, V, status);
    }
    return 0;
}
