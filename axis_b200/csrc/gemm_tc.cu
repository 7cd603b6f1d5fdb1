// bf16 GEMM on the 5th-generation tensor cores: TMA-fed shared-memory stages,
// tcgen05.mma with fp32 accumulators in TMEM, double-buffered accumulators so
// that the epilogue of one tile overlaps the main loop of the next.
//
//   C[m,n] = alpha * op(A) op(B) + beta * D          (fp32 accumulate)
//   tb = 0: A [m,k] (K-major),  B [k,n] (N-major)      forward  y = x W
//   tb = 1: A [m,k] (K-major),  B [n,k] (K-major)      dX = g W^T, logits = x E^T
//   tb = 2: A [k,m] (M-major),  B [k,n] (N-major)      dW = x^T g   (fp32 out)
//
// One persistent CTA per SM, 192 threads: warp 0 lane 0 issues TMA loads,
// warp 1 lane 0 issues the MMAs, warps 2..5 read TMEM and write C.  Tile
// 128 x BN x 64 with BN = 128 or 256.  All barrier waits are bounded.
#include <cuda_bf16.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

#define BM 128
#define BK 64
#define GEMM_THREADS 192
#define STAT_GEMM 0x100

// ── host helpers shared with the attention kernels ──────────────────────────
static PFN_tmapEncodeTiled g_encode = nullptr;
PFN_tmapEncodeTiled tc_encode_fn() {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return nullptr;
        g_encode = (PFN_tmapEncodeTiled)fn;
    }
    return g_encode;
}
int tc_make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box, bool swizzle128) {
    PFN_tmapEncodeTiled enc = tc_encode_fn();
    if (!enc) return 1;
    cuuint64_t gd[5]; cuuint64_t gs[4]; cuuint32_t bx[5]; cuuint32_t es[5];
    for (int i = 0; i < rank; i++) { gd[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
    for (int i = 0; i + 1 < rank; i++) gs[i] = strides_bytes[i];
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gd, gs, bx, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 2;
}

template <int BN> struct GemmCfg {
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;                 // two accumulators
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

#include "gemm_epi.cuh"

// A_MN / B_MN: 1 when that operand is MN-major in global memory (see header).
template <int BN, int A_MN, int B_MN, typename TO>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_gemm_tc(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
          TO* __restrict__ C, const TO* D, int m, int n, int k, float alpha, float beta, int* status,
          int ksplit, float* __restrict__ ws) {
    using Cfg = GemmCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    // bars: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then tmem base word, abort flag
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t smem_base = smem_u32(smem);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (m + BM - 1) / BM, tiles_n = (n + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int kblocks_all = (k + BK - 1) / BK;
    // split-K: unit u = (split, tile); split s covers k-blocks [s*kb_per, min(all, (s+1)*kb_per)) and
    // writes raw fp32 partial sums to ws[s][m][n]; a second kernel adds the splits in order
    const int kb_per = (kblocks_all + ksplit - 1) / ksplit;
    const int num_units = num_tiles * ksplit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 128); }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: let the next kernel in the stream start its own set-up as
    // SMs free up, and do not touch global memory until everything before this kernel is done.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0 && lane == 0) {
        // ── TMA producer ──
        uint32_t it = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
            const int tile = unit % num_tiles, split = unit / num_tiles;
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            const int kb0 = split * kb_per, kb1 = min(kblocks_all, kb0 + kb_per);
            for (int kb = kb0; kb < kb1; kb++, it++) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (it >= (uint32_t)STAGES && !mbar_wait(bar_empty + 8 * s, ph ^ 1)) { ok = false; break; }
                if (*abort_flag) { ok = false; break; }
                const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES, sb = sa + Cfg::A_BYTES;
                mbar_expect_tx(bar_full + 8 * s, Cfg::STAGE_BYTES);
                if (A_MN) {     // A [k, m]: boxes of 64 (m) x 64 (k)
#pragma unroll
                    for (int b = 0; b < BM / 64; b++) tma_load_2d(sa + b * 8192, &tmA, bar_full + 8 * s, tm * BM + b * 64, kb * BK);
                } else {        // A [m, k]: one box 64 (k) x 128 (m)
                    tma_load_2d(sa, &tmA, bar_full + 8 * s, kb * BK, tm * BM);
                }
                if (B_MN) {     // B [k, n]: boxes of 64 (n) x 64 (k)
#pragma unroll
                    for (int b = 0; b < BN / 64; b++) tma_load_2d(sb + b * 8192, &tmB, bar_full + 8 * s, tn * BN + b * 64, kb * BK);
                } else {        // B [n, k]: one box 64 (k) x BN (n)
                    tma_load_2d(sb, &tmB, bar_full + 8 * s, kb * BK, tn * BN);
                }
            }
        }
        if (!ok) { *abort_flag = 1; atomicExch(status, STAT_GEMM | 1); }
        // before leaving, wait (bounded) for every load this thread issued
        const uint32_t issued = it;
        for (uint32_t j = (issued > (uint32_t)STAGES ? issued - STAGES : 0); j < issued; j++)
            mbar_wait(bar_full + 8 * (j % STAGES), (j / STAGES) & 1);
    } else if (warp == 1 && lane == 0) {
        // ── MMA issuer ──
        constexpr uint32_t idesc = tc_idesc_bf16(BM, BN, A_MN, B_MN);
        uint32_t it = 0, tcount = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, tcount++) {
            const int split = unit / num_tiles;
            const int kb0 = split * kb_per, kb1 = min(kblocks_all, kb0 + kb_per);
            const int acc = tcount & 1;
            const uint32_t aph = (tcount >> 1) & 1;
            if (tcount >= 2 && !mbar_wait(bar_tempty + 8 * acc, aph ^ 1)) { ok = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN;
            for (int kb = kb0; kb < kb1; kb++, it++) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(bar_full + 8 * s, ph) || *abort_flag) { ok = false; break; }
                tc_fence_after();
                const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES, sb = sa + Cfg::A_BYTES;
#pragma unroll
                for (int kk = 0; kk < BK / 16; kk++) {
                    // K-major: 16 k-elements = 32 bytes inside the 128-byte row; MN-major: 16 k-rows = 2048 bytes
                    const uint64_t ad = A_MN ? tc_smem_desc(sa + kk * 2048, 8192, 1024) : tc_smem_desc(sa + kk * 32, 16, 1024);
                    const uint64_t bd = B_MN ? tc_smem_desc(sb + kk * 2048, 8192, 1024) : tc_smem_desc(sb + kk * 32, 16, 1024);
                    tc_mma_ss(d_tmem, ad, bd, idesc, (kb != kb0) || (kk != 0));
                }
                tc_commit(bar_empty + 8 * s);          // frees the stage when these MMAs finish
            }
            if (ok) tc_commit(bar_tfull + 8 * acc);    // accumulator complete
        }
        if (!ok) { *abort_flag = 1; atomicExch(status, STAT_GEMM | 2); }
    } else if (warp >= 2) {
        // ── epilogue: TMEM -> registers -> global ──
        const int quad = warp & 3;                     // TMEM lane quadrant this warp may read
        uint32_t tcount = 0;
        bool ok = true;
        const bool vec_ok = (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (n % (16 / (int)sizeof(TO))) == 0 &&
                            (!D || (reinterpret_cast<uintptr_t>(D) & 15) == 0);
        for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, tcount++) {
            const int tile = unit % num_tiles, split = unit / num_tiles;
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            const int acc = tcount & 1;
            const uint32_t aph = (tcount >> 1) & 1;
            if (!mbar_wait(bar_tfull + 8 * acc, aph) || *abort_flag) { ok = false; break; }
            tc_fence_after();
            const int row = tm * BM + quad * 32 + lane;
            const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16);
            TO* crow = C + (long long)row * n;
            const TO* drow = (D && beta != 0.f) ? D + (long long)row * n : nullptr;
            float* wrow = ws + ((long long)split * m + row) * n;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + c, r);
                tmem_ld_wait();
                const int col0 = tn * BN + c;
                if (row < m && col0 < n) {
                    if (ksplit > 1) epi_store<float>(wrow, nullptr, r, col0, n - col0, 1.f, 0.f, (n & 3) == 0);
                    else epi_store<TO>(crow, drow, r, col0, n - col0, alpha, beta, vec_ok);
                }
            }
            tc_fence_before();
            mbar_arrive(bar_tempty + 8 * acc);
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, STAT_GEMM | 3); }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, Cfg::TMEM_COLS); }
}

// C = alpha * (ws[0] + ws[1] + ... in split order) + beta * D
template <typename TO>
__global__ void k_splitk_reduce(const float* __restrict__ ws, int ksplit, TO* __restrict__ C, const TO* D,
                                long long mn, float alpha, float beta) {
    const long long n4 = mn / 4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 a = *reinterpret_cast<const float4*>(ws + i * 4);
        for (int s = 1; s < ksplit; s++) {
            const float4 b = *reinterpret_cast<const float4*>(ws + (long long)s * mn + i * 4);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        float f[4] = {alpha * a.x, alpha * a.y, alpha * a.z, alpha * a.w};
        if (D && beta != 0.f)
            for (int q = 0; q < 4; q++) f[q] += beta * ldf(D, i * 4 + q);
        for (int q = 0; q < 4; q++) stf(C, i * 4 + q, f[q]);
    }
}

static float* g_splitk_ws = nullptr;
static const size_t SPLITK_WS_BYTES = 160u << 20;
static int g_pair_mode = 0;        // 0 auto, 1 never use the paired-CTA kernel, 2 use it whenever the shape allows
static int g_pairs_avail = 0;      // co-resident CTA pairs of the paired kernel (0 = unavailable)
// programmatic dependent launch of the GEMM kernels (AXENG_NO_PDL=1 turns it off)
// GEMMs queued on a side stream (weight gradients that overlap the main chain): no programmatic dependent
// launch (their predecessor in the stream is an event wait, not a kernel of the chain) and no split-K (the
// split-K workspace is one buffer, owned by the main stream's launches)
static int g_side = 0;
void ax_gemm_side(int on) { g_side = on; }
int ax_gemm_pdl(void) {
    static const int on = getenv("AXENG_NO_PDL") ? 0 : 1;
    return on && !g_side;
}
// output tiles written by TMA stores from a shared-memory staging area (AXENG_NO_TMA_OUT=1: per-thread stores)
int ax_gemm_tma_out(void) {
    static const int on = getenv("AXENG_NO_TMA_OUT") ? 0 : 1;
    return on;
}
float* ax_splitk_ws(size_t* bytes) { if (bytes) *bytes = SPLITK_WS_BYTES; return g_splitk_ws; }
void ax_gemm_set_mode(int mode) { g_pair_mode = mode; }
template <typename TO>
void ax_splitk_reduce_launch(const float* ws, int ksplit, TO* C, const TO* D, long long mn, float alpha, float beta, cudaStream_t st) {
    k_splitk_reduce<TO><<<ew_grid(mn / 4, 256), 256, 0, st>>>(ws, ksplit, C, D, mn, alpha, beta);
}
template void ax_splitk_reduce_launch<bf16>(const float*, int, bf16*, const bf16*, long long, float, float, cudaStream_t);
template void ax_splitk_reduce_launch<float>(const float*, int, float*, const float*, long long, float, float, cudaStream_t);

template <int BN, int A_MN, int B_MN, typename TO>
static int gemm_set_attr() {
    return (int)cudaFuncSetAttribute(k_gemm_tc<BN, A_MN, B_MN, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::SMEM);
}
int ax_gemm_tc_init(void) {
    if (!tc_encode_fn()) return 1;
    int rc = 0;
    if (!g_splitk_ws && cudaMalloc(&g_splitk_ws, SPLITK_WS_BYTES) != cudaSuccess) { g_splitk_ws = nullptr; cudaGetLastError(); }
    g_pairs_avail = ax_gemm_tc2_init();
    if (g_pairs_avail < 1) g_pairs_avail = 0;
    rc |= gemm_set_attr<128, 0, 1, bf16>(); rc |= gemm_set_attr<256, 0, 1, bf16>();
    rc |= gemm_set_attr<128, 0, 0, bf16>(); rc |= gemm_set_attr<256, 0, 0, bf16>();
    rc |= gemm_set_attr<128, 1, 1, bf16>(); rc |= gemm_set_attr<256, 1, 1, bf16>();
    rc |= gemm_set_attr<128, 0, 1, float>(); rc |= gemm_set_attr<256, 0, 1, float>();
    rc |= gemm_set_attr<128, 0, 0, float>(); rc |= gemm_set_attr<256, 0, 0, float>();
    rc |= gemm_set_attr<128, 1, 1, float>(); rc |= gemm_set_attr<256, 1, 1, float>();
    return rc;
}

template <int BN, int A_MN, int B_MN, typename TO>
static int gemm_launch(const void* A, const void* B, void* C, const void* D, int m, int n, int k,
                       float alpha, float beta, int* status, int ksplit, cudaStream_t st) {
    CUtensorMap tmA, tmB;
    {
        // A: K-major [m,k] -> dims {k, m}, box {64, 128};  M-major [k,m] -> dims {m, k}, box {64, 64}
        uint64_t dims[2], strides[1]; uint32_t box[2];
        if (A_MN) { dims[0] = m; dims[1] = k; strides[0] = (uint64_t)m * 2; box[0] = 64; box[1] = BK; }
        else { dims[0] = k; dims[1] = m; strides[0] = (uint64_t)k * 2; box[0] = BK; box[1] = BM; }
        if (tc_make_tmap_bf16(&tmA, A, 2, dims, strides, box, true)) return 2;
        // B: N-major [k,n] -> dims {n, k}, box {64, 64};  K-major [n,k] -> dims {k, n}, box {64, BN}
        if (B_MN) { dims[0] = n; dims[1] = k; strides[0] = (uint64_t)n * 2; box[0] = 64; box[1] = BK; }
        else { dims[0] = k; dims[1] = n; strides[0] = (uint64_t)k * 2; box[0] = BK; box[1] = BN; }
        if (tc_make_tmap_bf16(&tmB, B, 2, dims, strides, box, true)) return 2;
    }
    const int units = ((m + BM - 1) / BM) * ((n + BN - 1) / BN) * ksplit;
    const int grid = units < AX_SMS ? units : AX_SMS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = GemmCfg<BN>::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = ax_gemm_pdl() ? 1 : 0;
    TO* Cp = (TO*)C; const TO* Dp = (const TO*)D;
    float* wsp = g_splitk_ws;
    if (cudaLaunchKernelEx(&cfg, k_gemm_tc<BN, A_MN, B_MN, TO>, tmA, tmB, Cp, Dp, m, n, k, alpha, beta, status, ksplit, wsp) != cudaSuccess) return 3;
    if (ksplit > 1) {
        const long long mn = (long long)m * n;
        k_splitk_reduce<TO><<<ew_grid(mn / 4, 256), 256, 0, st>>>(g_splitk_ws, ksplit, (TO*)C, (const TO*)D, mn, alpha, beta);
    }
    return 0;
}

int ax_gemm_tc(int out_bf16, int tb, const void* A, const void* B, void* C, const void* D,
               int m, int n, int k, float alpha, float beta, int* status, cudaStream_t st) {
    // shapes the TMA path serves: 16-byte aligned bases and row pitches.  Extents smaller
    // than a tile (rank-16 adapter GEMMs) are fine: TMA zero-fills the part of a box that
    // lies outside the tensor and the epilogue is bounds-checked.
    if (!aligned16(A) || !aligned16(B)) return -1;
    if (m < 8 || n < 8 || k < 8) return -1;
    if (tb == 0) { if (k % 8 || n % 8) return -1; }
    else if (tb == 1) { if (k % 8) return -1; }
    else { if (m % 8 || n % 8) return -1; }
    // Tile width and split-K factor from a small cost model (unit: one 128x256 k-block):
    // waves(units) * k-blocks per unit * cost(BN) + the split-K reduction traffic.
    const int kblocks = (k + BK - 1) / BK;
    const long long tm_ = (m + BM - 1) / BM;
    auto waves = [](long long t) { return (t + AX_SMS - 1) / AX_SMS; };
    int best_bn = 128, best_s = 1;
    double best = 1e30;
    for (int bn = 128; bn <= 256; bn += 128) {
        if (bn == 256 && n < 256) break;
        const long long tiles = tm_ * ((n + bn - 1) / bn);
        for (int sk = 1; sk <= 4; sk++) {
            if (sk > 1 && (g_side || kblocks < 16 * sk || (n & 3) || !g_splitk_ws ||
                           (size_t)sk * m * n * 4 > SPLITK_WS_BYTES)) break;
            const double per_kb = bn == 256 ? 1.0 : 0.72;
            double cost = (double)waves(tiles * sk) * ((kblocks + sk - 1) / sk) * per_kb;
            if (sk > 1) cost += (2.0 * sk + 1.0) * m * n * 4.0 / 4.0e12 / 0.45e-6 + 4.0;   // reduce pass, in k-block units
            if (cost < best - 1e-9) { best = cost; best_bn = bn; best_s = sk; }
        }
    }
    const bool use256 = best_bn == 256;
    int ks = best_s;
    // paired-CTA kernel (256 x 256 tile per two SMs): same cost model, cheaper k-blocks
    if (g_pair_mode != 1 && g_pairs_avail > 0 && m >= 256 && n >= 256) {
        const long long tiles2 = (long long)((m + 255) / 256) * ((n + 255) / 256);
        int best2_s = 1;
        double best2 = 1e30;
        for (int sk = 1; sk <= 4; sk++) {
            if (sk > 1 && (g_side || kblocks < 16 * sk || (n & 3) || !g_splitk_ws || (size_t)sk * m * n * 4 > SPLITK_WS_BYTES)) break;
            double cost = (double)((tiles2 * sk + g_pairs_avail - 1) / g_pairs_avail) * ((kblocks + sk - 1) / sk) * 0.70;
            if (sk > 1) cost += (2.0 * sk + 1.0) * m * n * 4.0 / 4.0e12 / 0.45e-6 + 4.0;
            if (cost < best2 - 1e-9) { best2 = cost; best2_s = sk; }
        }
        if (g_pair_mode == 2 || best2 < best) {
            const int rc = ax_gemm_tc2(out_bf16, tb, A, B, C, D, m, n, k, alpha, beta, status, best2_s, st);
            if (rc >= 0) { ax_variant = 0x22 + 0x100 * best2_s; return rc; }
        }
    }
#define GL(BN_, AM, BMj)                                                                                       \
    (out_bf16 ? gemm_launch<BN_, AM, BMj, bf16>(A, B, C, D, m, n, k, alpha, beta, status, ks, st)            \
              : gemm_launch<BN_, AM, BMj, float>(A, B, C, D, m, n, k, alpha, beta, status, ks, st))
    ax_variant = 0x21 + 0x100 * ks;
    if (tb == 0) return use256 ? GL(256, 0, 1) : GL(128, 0, 1);
    if (tb == 1) return use256 ? GL(256, 0, 0) : GL(128, 0, 0);
    return use256 ? GL(256, 1, 1) : GL(128, 1, 1);
#undef GL
}
