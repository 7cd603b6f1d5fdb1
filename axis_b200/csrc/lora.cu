// Weight gradients of low-rank adapters: out[F, R] = alpha * X^T S for a wide activation X [N, F] and a skinny
// factor S [N, R] (R = 8, 16 or 32), both bf16, reduced over the N tokens.
//
// The reference computes these as GEMMs like any other (axis/compile.py:270-305: dA = x^T (g B^T), dB = (x A)^T g);
// with R = 16 such a product is a stream over X — 16 flops per byte — and runs at HBM speed only if X is read once,
// by many CTAs, with next to no work per byte.  A tcgen05 tile would be 1/16 full and a split-K launch per product
// costs more in fill, drain and reduction than the product itself.  So: one launch covers up to sixteen products (all
// adapters of a layer); a
// CTA takes 256 columns of one X and a slice of the tokens, stages 64-token pieces with cp.async, multiplies with
// mma.sync (the fragments are transposed on the way out of shared memory by ldmatrix.trans) and leaves an fp32
// partial [F, R] per token slice; a second small kernel sums the slices in a fixed order (bit-reproducible), scales
// and writes either [F, R] or its transpose [R, F] — the layout of the adapter's other factor.
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.h"

static __device__ __forceinline__ uint32_t lg_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

#define LG_COLS 256          // columns of X per CTA
#define LG_TOK 64            // tokens per stage
#define LG_XS (LG_COLS * 2 + 16)   // padded row pitch of the X stage in bytes (conflict-free ldmatrix)
#define LG_THREADS 256

struct LoraGradProb {
    const bf16* X;
    const bf16* S;
    float* out;
    int F;                   // columns of X == rows of out
    int chunks;              // ceil(F / LG_COLS)
    int layout;              // 0: out is [F, R], 1: [R, F]
    long long ws_off;        // offset of this product's partials in the workspace (floats)
};
#define LG_MAX_PROBS 16
struct LoraGradArgs {
    LoraGradProb p[LG_MAX_PROBS];
    int count, N, nsplit, tok_per;
    float alpha;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t* r) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_t(uint32_t addr, uint32_t* r) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, const uint32_t* b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// NT = R / 8.  grid = (column chunks of all products, token slices)
template <int NT>
__global__ void __launch_bounds__(LG_THREADS) k_lora_grad_partial(const LoraGradArgs a, float* __restrict__ ws) {
    constexpr int R = NT * 8;
    constexpr int SS = R * 2 + 16;                         // padded row pitch of the S stage
    constexpr int STAGE = LG_TOK * LG_XS + LG_TOK * SS;
    extern __shared__ __align__(128) uint8_t lg_smem[];
    const uint32_t sbase = lg_smem_u32(lg_smem);
    int g = 0, chunk = blockIdx.x;
    while (g + 1 < a.count && chunk >= a.p[g].chunks) { chunk -= a.p[g].chunks; g++; }
    const LoraGradProb P = a.p[g];
    const int f0 = chunk * LG_COLS;
    const int split = blockIdx.y;
    const int t_begin = split * a.tok_per, t_end = min(a.N, t_begin + a.tok_per);
    const int nstage = t_end > t_begin ? (t_end - t_begin + LG_TOK - 1) / LG_TOK : 0;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    auto load_stage = [&](int st, int buf) {
        const int t0 = t_begin + st * LG_TOK;
        const uint32_t xs = sbase + buf * STAGE, ss = xs + LG_TOK * LG_XS;
        // X: 64 rows x 32 chunks of 16 bytes; out-of-range rows / columns are zero-filled
#pragma unroll
        for (int q = 0; q < (LG_TOK * LG_COLS / 8) / LG_THREADS; q++) {
            const int idx = q * LG_THREADS + tid;
            const int r = idx >> 5, c8 = idx & 31;
            const int t = t0 + r, f = f0 + c8 * 8;
            const bool ok = t < t_end && f < P.F;
            cp_async16(xs + r * LG_XS + c8 * 16, ok ? (const void*)(P.X + (long long)t * P.F + f) : (const void*)P.X, ok ? 16 : 0);
        }
        // S: 64 rows x NT chunks
        if (tid < LG_TOK * NT) {
            const int r = tid / NT, c8 = tid % NT;
            const int t = t0 + r;
            const bool ok = t < t_end;
            cp_async16(ss + r * SS + c8 * 16, ok ? (const void*)(P.S + (long long)t * R + c8 * 8) : (const void*)P.S, ok ? 16 : 0);
        }
        cp_async_commit();
    };

    float acc[2][NT][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0.f;

    if (nstage > 0) load_stage(0, 0);
    for (int st = 0; st < nstage; st++) {
        if (st + 1 < nstage) { load_stage(st + 1, (st + 1) & 1); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        const uint32_t xs = sbase + (st & 1) * STAGE, ss = xs + LG_TOK * LG_XS;
        const int mi = lane >> 3, ri = lane & 7;           // ldmatrix: matrix index and row inside it
#pragma unroll
        for (int ks = 0; ks < LG_TOK / 16; ks++) {
            const int t0 = ks * 16;
            uint32_t bfr[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)                // S^T fragments: stored rows are tokens (k), columns ranks (n)
                ldsm_x2_t(ss + (t0 + (mi & 1) * 8 + ri) * SS + nt * 16, bfr[nt]);
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const int fc = warp * 32 + mt * 16;
                uint32_t afr[4];                            // X^T fragments: m0 (f 0-7, t 0-7) m1 (f 8-15, t 0-7) m2 (f 0-7, t 8-15) m3
                ldsm_x4_t(xs + (t0 + (mi >> 1) * 8 + ri) * LG_XS + (fc + (mi & 1) * 8) * 2, afr);
#pragma unroll
                for (int nt = 0; nt < NT; nt++) mma_bf16_16816(acc[mt][nt], afr, bfr[nt]);
            }
        }
        __syncthreads();
    }
    // partial [split][F][R]
    float* dst = ws + P.ws_off + (long long)split * P.F * R;
    const int gq = lane >> 2, q2 = (lane & 3) * 2;
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int f = f0 + warp * 32 + mt * 16 + h * 8 + gq;
            if (f < P.F) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
                    *reinterpret_cast<float2*>(dst + (long long)f * R + nt * 8 + q2) = make_float2(acc[mt][nt][h * 2], acc[mt][nt][h * 2 + 1]);
            }
        }
}

// out = alpha * sum over token slices, in slice order; layout 0: [F, R], 1: [R, F]
__global__ void k_lora_grad_reduce(const LoraGradArgs a, const float* __restrict__ ws, int R) {
    int g = blockIdx.y;
    const LoraGradProb P = a.p[g];
    const long long n = (long long)P.F * R;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int sp = 0; sp < a.nsplit; sp++) s += ws[P.ws_off + sp * n + i];
        const int f = (int)(i / R), r = (int)(i % R);
        P.out[P.layout ? (long long)r * P.F + f : i] = a.alpha * s;
    }
}

static bool g_lora_attr = false;

// X[g] [N, F[g]] bf16, S[g] [N, R] bf16 -> out[g] fp32 ([F, R], or [R, F] where layout[g] is 1).  ws: fp32 workspace of
// ws_bytes.  Returns -1 when the request is outside what the kernel serves (the caller then uses GEMMs).
int ax_lora_grad(int count, const void* const* X, const void* const* S, float* const* out, const int* F, const int* layout,
                 int N, int R, float alpha, float* ws, size_t ws_bytes, cudaStream_t st) {
    if (count < 1 || count > LG_MAX_PROBS || N < 1 || !(R == 8 || R == 16 || R == 32) || !ws) return -1;
    LoraGradArgs a = {};
    a.count = count; a.N = N; a.alpha = alpha;
    int chunks = 0, fmax = 0;
    long long fsum = 0;
    for (int g = 0; g < count; g++) {
        if (F[g] < 8 || F[g] % 8 || !aligned16(X[g]) || !aligned16(S[g]) || !out[g]) return -1;
        a.p[g].X = (const bf16*)X[g]; a.p[g].S = (const bf16*)S[g]; a.p[g].out = out[g]; a.p[g].F = F[g];
        a.p[g].layout = layout[g] ? 1 : 0;
        a.p[g].chunks = (F[g] + LG_COLS - 1) / LG_COLS;
        chunks += a.p[g].chunks; fsum += F[g]; fmax = F[g] > fmax ? F[g] : fmax;
    }
    // token slices: as many CTAs as are resident at once (three per SM) and no more — a second, partial wave would cost
    // as much as the first; at least one 64-token stage each, partials inside the workspace
    int nsplit = (3 * AX_SMS) / chunks;
    if (nsplit < 1) nsplit = 1;
    const int max_split = (N + LG_TOK - 1) / LG_TOK;
    if (nsplit > max_split) nsplit = max_split;
    if (nsplit > 64) nsplit = 64;
    while (nsplit > 1 && (size_t)nsplit * fsum * R * 4 > ws_bytes) nsplit--;
    if ((size_t)nsplit * fsum * R * 4 > ws_bytes) return -1;
    a.tok_per = ((N + nsplit - 1) / nsplit + LG_TOK - 1) / LG_TOK * LG_TOK;
    nsplit = (N + a.tok_per - 1) / a.tok_per;
    a.nsplit = nsplit;
    long long off = 0;
    for (int g = 0; g < count; g++) { a.p[g].ws_off = off; off += (long long)nsplit * F[g] * R; }
    const int NT = R / 8;
    const size_t smem = 2 * (size_t)(LG_TOK * LG_XS + LG_TOK * (R * 2 + 16));
    if (!g_lora_attr) {
        cudaFuncSetAttribute(k_lora_grad_partial<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * (LG_TOK * LG_XS + LG_TOK * 32));
        cudaFuncSetAttribute(k_lora_grad_partial<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * (LG_TOK * LG_XS + LG_TOK * 48));
        cudaFuncSetAttribute(k_lora_grad_partial<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * (LG_TOK * LG_XS + LG_TOK * 80));
        g_lora_attr = true;
    }
    const dim3 grid(chunks, nsplit);
    if (NT == 1) k_lora_grad_partial<1><<<grid, LG_THREADS, smem, st>>>(a, ws);
    else if (NT == 2) k_lora_grad_partial<2><<<grid, LG_THREADS, smem, st>>>(a, ws);
    else k_lora_grad_partial<4><<<grid, LG_THREADS, smem, st>>>(a, ws);
    const int rb = (int)(((long long)fmax * R + 255) / 256);
    k_lora_grad_reduce<<<dim3(rb > 592 ? 592 : rb, count), 256, 0, st>>>(a, ws, R);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// ── the skinny products of an adapter: out[N, R] = alpha * X W (W [F, R]) or alpha * X W^T (W [R, F]) ──────────────────
// u = x A in the forward and t = g B^T in the backward: again a stream over the wide operand with 16 flops per byte.
// A CTA takes 32 tokens and walks F in pieces of 256 columns (three cp.async stages); its eight warps are two row tiles
// times four quarters of a piece's depth, and the four partial accumulators of a row tile meet in shared memory.
#define LP_TOK 32
#define LP_COLS 256
#define LP_STAGES 3

struct LoraProjProb {
    const bf16* X;
    const bf16* W;
    bf16* out;
    int F;
};
struct LoraProjArgs {
    LoraProjProb p[3];
    int count, N;
    float alpha;
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t* r) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t* r) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

// TB = 0: W is [F, R] (row pitch of its stage R*2+16 bytes); TB = 1: W is [R, F] (row pitch LG_XS).  grid = (token blocks, products)
template <int NT, int TB>
__global__ void __launch_bounds__(256) k_lora_proj(const LoraProjArgs a) {
    constexpr int R = NT * 8;
    constexpr int WS = TB ? LG_XS : R * 2 + 16;
    constexpr int WROWS = TB ? R : LP_COLS;
    constexpr int XBYTES = LP_TOK * LG_XS;
    constexpr int STAGE = XBYTES + WROWS * WS;
    extern __shared__ __align__(128) uint8_t lg_smem[];
    const uint32_t sbase = lg_smem_u32(lg_smem);
    const LoraProjProb P = a.p[blockIdx.y];
    const int t0 = blockIdx.x * LP_TOK;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nstage = (P.F + LP_COLS - 1) / LP_COLS;

    auto load_stage = [&](int st) {
        const int f0 = st * LP_COLS;
        const uint32_t xs = sbase + (st % LP_STAGES) * STAGE, ws_ = xs + XBYTES;
#pragma unroll
        for (int q = 0; q < (LP_TOK * LP_COLS / 8) / 256; q++) {        // X: 32 rows x 32 chunks
            const int idx = q * 256 + tid;
            const int r = idx >> 5, c8 = idx & 31;
            const int t = t0 + r, f = f0 + c8 * 8;
            const bool ok = t < a.N && f < P.F;
            cp_async16(xs + r * LG_XS + c8 * 16, ok ? (const void*)(P.X + (long long)t * P.F + f) : (const void*)P.X, ok ? 16 : 0);
        }
        if (TB) {                                                       // W [R, F]: R rows x 32 chunks
#pragma unroll
            for (int q = 0; q < (R * 32 + 255) / 256; q++) {
                const int idx = q * 256 + tid;
                const int r = idx >> 5, c8 = idx & 31;
                const int f = f0 + c8 * 8;
                if (r < R) {
                    const bool ok = f < P.F;
                    cp_async16(ws_ + r * WS + c8 * 16, ok ? (const void*)(P.W + (long long)r * P.F + f) : (const void*)P.W, ok ? 16 : 0);
                }
            }
        } else {                                                        // W [F, R]: 256 rows x NT chunks
#pragma unroll
            for (int q = 0; q < NT; q++) {
                const int idx = q * 256 + tid;
                const int r = idx / NT, c8 = idx % NT;
                const int f = f0 + r;
                const bool ok = f < P.F;
                cp_async16(ws_ + r * WS + c8 * 16, ok ? (const void*)(P.W + (long long)f * R + c8 * 8) : (const void*)P.W, ok ? 16 : 0);
            }
        }
        cp_async_commit();
    };

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[j][e] = 0.f;
    const int mt = warp & 1, kq = warp >> 1;               // row tile, quarter of the piece's depth
    const int mi = lane >> 3, ri = lane & 7;

    for (int st = 0; st < LP_STAGES - 1 && st < nstage; st++) load_stage(st);
    for (int st = 0; st < nstage; st++) {
        if (st + LP_STAGES - 1 < nstage) { load_stage(st + LP_STAGES - 1); cp_async_wait<LP_STAGES - 1>(); }
        else if (st + 2 == nstage) cp_async_wait<1>();
        else if (st + 1 == nstage) cp_async_wait<0>();
        else cp_async_wait<LP_STAGES - 2>();
        __syncthreads();
        const uint32_t xs = sbase + (st % LP_STAGES) * STAGE, ws_ = xs + XBYTES;
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            const int k0 = kq * 64 + ks * 16;
            uint32_t afr[4];                                 // X fragments: (rows 0-7, k 0-7) (rows 8-15, k 0-7) (rows 0-7, k 8-15) (rows 8-15, k 8-15)
            ldsm_x4(xs + (mt * 16 + (mi & 1) * 8 + ri) * LG_XS + (k0 + (mi >> 1) * 8) * 2, afr);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                uint32_t bfr[2];
                if (TB) ldsm_x2(ws_ + (nt * 8 + ri) * WS + (k0 + (mi & 1) * 8) * 2, bfr);           // W^T stored [n][k]
                else ldsm_x2_t(ws_ + (k0 + (mi & 1) * 8 + ri) * WS + nt * 16, bfr);                  // W stored [k][n]
                mma_bf16_16816(acc[nt], afr, bfr);
            }
        }
        __syncthreads();
    }
    // the four depth quarters of a row tile meet in shared memory (the operand stages are free now)
    float* red = reinterpret_cast<float*>(lg_smem);         // [kq][32 rows][R]
    const int gq = lane >> 2, q2 = (lane & 3) * 2;
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
            *reinterpret_cast<float2*>(red + ((kq * LP_TOK) + mt * 16 + h * 8 + gq) * R + nt * 8 + q2) = make_float2(acc[nt][h * 2], acc[nt][h * 2 + 1]);
    __syncthreads();
    for (int i = tid; i < LP_TOK * R / 2; i += 256) {
        const int r = (i * 2) / R, c = (i * 2) % R;
        if (t0 + r < a.N) {
            float2 s = make_float2(0.f, 0.f);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 v = *reinterpret_cast<const float2*>(red + (q * LP_TOK + r) * R + c);
                s.x += v.x; s.y += v.y;
            }
            *reinterpret_cast<__nv_bfloat162*>(P.out + (long long)(t0 + r) * R + c) = __floats2bfloat162_rn(a.alpha * s.x, a.alpha * s.y);
        }
    }
}

template <int NT, int TB> static size_t lora_proj_smem() {
    constexpr int R = NT * 8;
    return (size_t)LP_STAGES * (LP_TOK * LG_XS + (TB ? R * LG_XS : LP_COLS * (R * 2 + 16)));
}
template <int NT, int TB> static int lora_proj_launch(const LoraProjArgs& a, cudaStream_t st) {
    static bool attr = false;
    const size_t smem = lora_proj_smem<NT, TB>();
    if (!attr) { cudaFuncSetAttribute(k_lora_proj<NT, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr = true; }
    k_lora_proj<NT, TB><<<dim3((a.N + LP_TOK - 1) / LP_TOK, a.count), 256, smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// out[g] [N, R] bf16 = alpha * X[g] [N, F[g]] W[g]; tb 0: W [F, R], tb 1: W [R, F].  -1 when not served.
int ax_lora_proj(int count, int tb, const void* const* X, const void* const* W, void* const* out, const int* F, int N, int R,
                 float alpha, cudaStream_t st) {
    if (count < 1 || count > 3 || N < 1 || !(R == 8 || R == 16 || R == 32) || tb < 0 || tb > 1) return -1;
    LoraProjArgs a = {};
    a.count = count; a.N = N; a.alpha = alpha;
    for (int g = 0; g < count; g++) {
        if (F[g] < 8 || F[g] % 8 || !aligned16(X[g]) || !aligned16(W[g]) || !out[g] || ((uintptr_t)out[g] & 3)) return -1;
        a.p[g].X = (const bf16*)X[g]; a.p[g].W = (const bf16*)W[g]; a.p[g].out = (bf16*)out[g]; a.p[g].F = F[g];
    }
#define LP(NT_) (tb ? lora_proj_launch<NT_, 1>(a, st) : lora_proj_launch<NT_, 0>(a, st))
    return R == 8 ? LP(1) : (R == 16 ? LP(2) : LP(4));
#undef LP
}
