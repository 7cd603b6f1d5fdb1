// Causal grouped-query flash attention on the 5th-generation tensor cores
// (tcgen05 + TMEM), bf16, head_dim 64 (head_dim 128: attn_tc128.cu), on the [B,T,H,DH] layout that the
// projections produce.  Q/K/V/dO tiles arrive by TMA (128-byte swizzle, no
// multicast); scores and gradients live in TMEM; probabilities go back into
// TMEM as packed bf16 and feed the next MMA as its A operand.
//
// Forward:  one CTA per (128 queries, head, batch).  S = Q K^T -> online
//   softmax by 128 threads (one row each, lazy rescale) -> P (bf16, TMEM) ->
//   O += P V.  Saves LSE (natural log) for the backward.
// Backward: one CTA per (128 keys, kv head, batch).  K/V resident; loops over
//   the group's query heads and the causal query tiles:
//     S^T = K Q^T, dP^T = V dO^T            (TMEM, lanes = keys; 64 queries at a time, two buffers)
//     P^T = exp2(S^T c - lse), dS^T = P^T (dP^T - D)
//     dV += P^T dO, dK += dS^T Q            (A from TMEM; summed over the group)
//     dQ  = dS K                            (A = dS^T staged in shared memory)
//   dK/dV are written once (no atomics, GQA sum on chip); dQ tiles are added
//   into an fp32 buffer with TMA reduce-add and converted afterwards.
// Every mbarrier wait is bounded; on a timeout the kernel records a status
// code, unwinds and frees its TMEM.
#include <cuda_bf16.h>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"
#include "attn_common.cuh"

#define AT 128                 // queries / keys per tile
#define ADH 64                 // head dim served
#define ATT_THREADS 160        // 4 softmax warps + 1 control warp
#define STAT_FWD 0x200
#define STAT_BWD 0x300

// ════════════════════════════════ forward ═══════════════════════════════════
struct FwdSmem {
    static constexpr int Q = 0, K0 = 16384, V0 = K0 + 2 * 16384, BARS = V0 + 2 * 16384, TOTAL = BARS + 128 + 1024;
};

__global__ void __launch_bounds__(ATT_THREADS, 2)
k_attn_fwd_tc(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, bf16* __restrict__ o, float* __restrict__ lse,
              int T, int H, int KV, float scale, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sb = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FwdSmem::BARS);
    const uint32_t b_q = smem_u32(bars), b_kvf = b_q + 8, b_kve = b_kvf + 16, b_s = b_kve + 16, b_p = b_s + 8, b_o = b_p + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // 1-D grid ordered by decreasing work: all (head, batch) pairs of the last query tile first
    const int nqt_ = T / AT, nhb = gridDim.x / nqt_;
    const int qt = nqt_ - 1 - (int)(blockIdx.x / nhb);
    const int hb = blockIdx.x % nhb;
    const int h = hb % H, b = hb / H, g = h / (H / KV);
    const int nkt = qt + 1;

    if (threadIdx.x == 0) {
        mbar_init(b_q, 1);
        for (int s = 0; s < 2; s++) { mbar_init(b_kvf + 8 * s, 1); mbar_init(b_kve + 8 * s, 1); }
        mbar_init(b_s, 1); mbar_init(b_p, 128); mbar_init(b_o, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) { tmem_alloc(smem_u32(tmem_slot), 256); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_S = tmem, t_O = tmem + 128;

    if (warp == 4) {
        if (lane == 0) {
            bool ok = true;
            constexpr uint32_t id_s = tc_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t id_pv = tc_idesc_bf16(128, 64, 0, 1);
            const uint32_t loQ = desc_lo(sb + FwdSmem::Q, 16), loK = desc_lo(sb + FwdSmem::K0, 16), loV = desc_lo(sb + FwdSmem::V0, 16384);
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
            mbar_expect_tx(b_q, 16384);
            tma_load_4d(sb + FwdSmem::Q, &tmQ, b_q, 0, h, qt * AT, b);
            mbar_expect_tx(b_kvf, 32768);
            tma_load_4d(sb + FwdSmem::K0, &tmK, b_kvf, 0, g, 0, b);
            tma_load_4d(sb + FwdSmem::V0, &tmV, b_kvf, 0, g, 0, b);
            if (!mbar_wait(b_q, 0)) ok = false;
            for (int j = 0; j < nkt && ok; j++) {
                const int s = j & 1;
                if (!mbar_wait(b_kvf + 8 * s, (j >> 1) & 1)) { ok = false; break; }
                // S(j) overwrites the columns that P V(j-1) reads P from: MMAs on different accumulators are not
                // ordered against each other, so wait for that MMA's completion instead of relying on issue order
                if (j >= 1 && !mbar_wait(b_o, (j - 1) & 1)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < ADH / 16; kk++)
                    tc_mma_ss(t_S, desc_of(loQ + kk * 2), desc_of(loK + s * 1024 + kk * 2), id_s, kk != 0);
                tc_commit(b_s);
                if (j + 1 < nkt) {      // next K/V tile into the other stage, once PV(j-1) has released it
                    const int s2 = s ^ 1;
                    if (j >= 1 && !mbar_wait(b_kve + 8 * s2, ((j - 1) >> 1) & 1)) { ok = false; break; }
                    mbar_expect_tx(b_kvf + 8 * s2, 32768);
                    tma_load_4d(sb + FwdSmem::K0 + s2 * 16384, &tmK, b_kvf + 8 * s2, 0, g, (j + 1) * AT, b);
                    tma_load_4d(sb + FwdSmem::V0 + s2 * 16384, &tmV, b_kvf + 8 * s2, 0, g, (j + 1) * AT, b);
                }
                if (!mbar_wait(b_p, j & 1)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < AT / 16; kk++)
                    tc_mma_ts(t_O, t_S + kk * 8, desc_of(loV + s * 1024 + kk * 128), id_pv, (j | kk) != 0);
                tc_commit(b_kve + 8 * s);
                tc_commit(b_o);
            }
            if (!ok) { *abort_flag = 1; atomicExch(status, STAT_FWD | 1); }
        }
    } else {
        const int r = threadIdx.x;                         // query row within the tile == TMEM lane
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float c = scale * LOG2E;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nkt && ok; j++) {
            if (!mbar_wait(b_s, j & 1) || *abort_flag) { ok = false; break; }
            tc_fence_after();
            const bool diag = j == qt;
            // the whole S row (128 scores) stays in registers between the max pass and the exp pass
            uint32_t sv[128];
#pragma unroll
            for (int ch = 0; ch < 4; ch++) tmem_ld32(t_S + lane_base + ch * 32, sv + ch * 32);
            tmem_ld_wait();
            // raw maximum first (c > 0), one multiply at the end; the mask only on the diagonal tile
            if (diag) {
#pragma unroll
                for (int q = 0; q < 128; q++)
                    if (q > r) sv[q] = 0xff800000u;              // -inf: exp2 gives 0
            }
            float mx;
            {
                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                for (int q = 0; q < 128; q += 8) {
                    m0 = fmax3(m0, __uint_as_float(sv[q]), __uint_as_float(sv[q + 1]));
                    m1 = fmax3(m1, __uint_as_float(sv[q + 2]), __uint_as_float(sv[q + 3]));
                    m2 = fmax3(m2, __uint_as_float(sv[q + 4]), __uint_as_float(sv[q + 5]));
                    m3 = fmax3(m3, __uint_as_float(sv[q + 6]), __uint_as_float(sv[q + 7]));
                }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            }
            mx *= c;
            if (j == 0) {
                m_used = mx;
            } else {
                const bool need = mx > m_used + 8.f;
                if (__any_sync(0xffffffffu, need)) {
                    // rescale this warp's rows of O; PV(j-1) must have landed first
                    if (!mbar_wait(b_o, (j - 1) & 1)) { ok = false; break; }
                    tc_fence_after();
                    const float m_new = fmaxf(m_used, mx);
                    const float f = fast_exp2(m_used - m_new);
                    m_used = m_new;
                    l *= f;
#pragma unroll 1
                    for (int ch = 0; ch < 2; ch++) {
                        uint32_t v[32];
                        tmem_ld32(t_O + lane_base + ch * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 32; q++) v[q] = __float_as_uint(__uint_as_float(v[q]) * f);
                        tmem_st16(t_O + lane_base + ch * 32, v);
                        tmem_st16(t_O + lane_base + ch * 32 + 16, v + 16);
                    }
                    tmem_st_wait();
                }
            }
            {
                float l0 = 0.f, l1 = 0.f;
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    uint32_t w[16];
#pragma unroll
                    for (int q = 0; q < 32; q += 4) {
                        const float p0 = fast_exp2(__uint_as_float(sv[ch * 32 + q]) * c - m_used);
                        const float p1 = fast_exp2(__uint_as_float(sv[ch * 32 + q + 1]) * c - m_used);
                        const float p2 = fast_exp2(__uint_as_float(sv[ch * 32 + q + 2]) * c - m_used);
                        const float p3 = fast_exp2(__uint_as_float(sv[ch * 32 + q + 3]) * c - m_used);
                        l0 += p0 + p1;
                        l1 += p2 + p3;
                        w[q >> 1] = pack_bf16(p0, p1);
                        w[(q >> 1) + 1] = pack_bf16(p2, p3);
                    }
                    tmem_st16(t_S + lane_base + ch * 16, w);   // P replaces S (all of it is in registers by now)
                }
                l += l0 + l1;
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(b_p);
        }
        if (ok && mbar_wait(b_o, (nkt - 1) & 1)) {
            tc_fence_after();
            const int t = qt * AT + r;
            const float il = 1.f / l;
            bf16* orow = o + (((long long)b * T + t) * H + h) * ADH;
#pragma unroll 1
            for (int ch = 0; ch < 2; ch++) {
                uint32_t v[32];
                tmem_ld32(t_O + lane_base + ch * 32, v);
                tmem_ld_wait();
                if (t < T) {
#pragma unroll
                    for (int q = 0; q < 32; q += 8) {
                        uint4 pk;
                        pk.x = pack_bf16(__uint_as_float(v[q]) * il, __uint_as_float(v[q + 1]) * il);
                        pk.y = pack_bf16(__uint_as_float(v[q + 2]) * il, __uint_as_float(v[q + 3]) * il);
                        pk.z = pack_bf16(__uint_as_float(v[q + 4]) * il, __uint_as_float(v[q + 5]) * il);
                        pk.w = pack_bf16(__uint_as_float(v[q + 6]) * il, __uint_as_float(v[q + 7]) * il);
                        *reinterpret_cast<uint4*>(orow + ch * 32 + q) = pk;
                    }
                }
            }
            if (t < T) lse[((long long)b * H + h) * T + t] = (m_used + log2f(l)) * LN2;
        } else if (lane == 0) {
            *abort_flag = 1;
            atomicExch(status, STAT_FWD | 2);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, 256); }
}

// ════════════════════════════════ backward ══════════════════════════════════
// D[b,h,t] = sum_d dO*O on the [B,T,H,DH] layout, written as [B,H,T].  Eight lanes
// share a 64-element row (one 16-byte vector of each tensor per lane).
__global__ void k_attn_bwd_prep(const bf16* __restrict__ o, const bf16* __restrict__ dO, float* __restrict__ Dv,
                                int B, int T, int H) {
    const long long nvec = (long long)B * T * H * (ADH / 8);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec + 7; i += stride) {
        float a[8], g[8], acc = 0.f;
        if (i < nvec) {
            Vec<bf16>::ld(o + i * 8, a);
            Vec<bf16>::ld(dO + i * 8, g);
#pragma unroll
            for (int q = 0; q < 8; q++) acc += a[q] * g[q];
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        if ((i & 7) == 0 && i < nvec) {
            const long long row = i >> 3;
            const int hh = (int)(row % H);
            const long long bt = row / H;
            const int t = (int)(bt % T), bb = (int)(bt / T);
            Dv[((long long)bb * H + hh) * T + t] = acc;
        }
    }
}

// Backward CTA: two softmax groups of 4 warps (group e owns the sub-tiles of parity e and TMEM buffer e; a
// thread owns one key row and all 64 query columns of its sub-tile), 4 warps that move finished dQ tiles out
// (TMEM -> shared memory -> TMA reduce-add), 1 MMA-issue warp, 1 TMA-load warp.
#define BWD_SM_WARPS 8
#define BWD_SM_THREADS (BWD_SM_WARPS * 32)
#define BWD_DRAIN_THREADS 128
#define BWD_THREADS (BWD_SM_THREADS + BWD_DRAIN_THREADS + 64)
// The backward works on sub-tiles of 64 queries so that the tensor pipe and the softmax warps overlap:
// while one group turns S^T/dP^T of sub-tile u into P^T/dS^T, the other group does the same for sub-tile
// u+1, and the tensor cores compute dV/dK/dQ of earlier sub-tiles and S^T/dP^T of later ones.
struct BwdSmem {
    static constexpr int K = 0, V = 16384, Q0 = 32768, DO0 = Q0 + 4 * 8192, DS0 = DO0 + 4 * 8192, DQ = DS0 + 2 * 32768,
                         STAT = DQ + 32768, BARS = STAT + 8192, TOTAL = BARS + 256 + 1024;
};
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}

__global__ void __launch_bounds__(BWD_THREADS, 1)
k_attn_bwd_tc(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
              const __grid_constant__ CUtensorMap tmdQ, const float* __restrict__ lse, const float* __restrict__ Dv,
              bf16* __restrict__ dk, bf16* __restrict__ dv, int T, int H, int KV, float scale, int* status,
              long long* prof) {
    // prof (optional, normally null): per-CTA cycle counts of the phases of softmax thread 0 —
    // [0] wait S/dP, [1] softmax + stores, [2] wait for the dS buffer, [3] unused, [4] total, [5] query tiles
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sb = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BwdSmem::BARS);
    // kv_full, q_full[4], q_empty[4], sdp_full[2], pds_full[2], dq_full[2], dq_empty[2]
    const uint32_t b_kv = smem_u32(bars), b_qf = b_kv + 8, b_qe = b_qf + 32, b_sdp = b_qe + 32, b_pds = b_sdp + 16,
                   b_dq = b_pds + 16, b_dqe = b_dq + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_stat = reinterpret_cast<float*>(smem + BwdSmem::STAT);   // [softmax warp][2][lse*log2(e) 64 | D 64]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int CTRL_WARP = BWD_SM_WARPS + 4;
    // 1-D grid ordered by decreasing work: key tile 0 (attended by every query tile) of all
    // (kv head, batch) pairs first
    const int rep = H / KV, nqt = T / AT;
    const int ngb = gridDim.x / nqt;
    const int j = blockIdx.x / ngb, gb = blockIdx.x % ngb;
    const int g = gb % KV, b = gb / KV;
    const int per_head = nqt - j;                                     // causal: query tiles j .. nqt-1
    const int n_it = rep * per_head;                                  // 128-query tiles
    const int n_sub = 2 * n_it;                                       // 64-query sub-tiles

    if (threadIdx.x == 0) {
        mbar_init(b_kv, 1);
        for (int s = 0; s < 4; s++) { mbar_init(b_qf + 8 * s, 1); mbar_init(b_qe + 8 * s, 1); }
        for (int s = 0; s < 2; s++) {
            mbar_init(b_sdp + 8 * s, 1); mbar_init(b_pds + 8 * s, 128);
            mbar_init(b_dq + 8 * s, 1); mbar_init(b_dqe + 8 * s, BWD_DRAIN_THREADS);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == CTRL_WARP) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // columns: S^T/P^T [2] 0..127, dP^T/dS^T [2] 128..255, dV 256..319, dK 320..383, dQ[0] 384..447, dQ[1] 448..511
    const uint32_t t_S = tmem, t_dP = tmem + 128, t_dV = tmem + 256, t_dK = tmem + 320, t_dQ = tmem + 384;

    if (warp == CTRL_WARP) {
        if (lane == 0) {
            bool ok = true;
            constexpr uint32_t id_s = tc_idesc_bf16(128, 64, 0, 0);        // S^T = K Q^T, dP^T = V dO^T (64 queries)
            constexpr uint32_t id_acc = tc_idesc_bf16(128, 64, 0, 1);      // dV/dK: A in TMEM, B N-major
            constexpr uint32_t id_dq = tc_idesc_bf16(128, 64, 1, 1);       // dQ: A M-major (dS^T in smem), B N-major
            // descriptor base words (K-major operands step 32 B = 2 units per k-step, MN-major ones 2048 B = 128 units)
            const uint32_t loK_k = desc_lo(sb + BwdSmem::K, 16), loV_k = desc_lo(sb + BwdSmem::V, 16);
            const uint32_t loK_n = desc_lo(sb + BwdSmem::K, 16384), loDS = desc_lo(sb + BwdSmem::DS0, 16384);
            const uint32_t loQ_k = desc_lo(sb + BwdSmem::Q0, 16), loQ_n = desc_lo(sb + BwdSmem::Q0, 16384);
            const uint32_t loO_k = desc_lo(sb + BwdSmem::DO0, 16), loO_n = desc_lo(sb + BwdSmem::DO0, 16384);
            auto issue_sdp = [&](int u) {           // S^T and dP^T of sub-tile u into TMEM buffer u & 1
                const int e = u & 1;
                const uint32_t so = (uint32_t)(u & 3) * 512;           // ring slot offset (8192 B)
#pragma unroll
                for (int kk = 0; kk < ADH / 16; kk++)
                    tc_mma_ss(t_S + e * 64, desc_of(loK_k + kk * 2), desc_of(loQ_k + so + kk * 2), id_s, kk != 0);
#pragma unroll
                for (int kk = 0; kk < ADH / 16; kk++)
                    tc_mma_ss(t_dP + e * 64, desc_of(loV_k + kk * 2), desc_of(loO_k + so + kk * 2), id_s, kk != 0);
                tc_commit(b_sdp + 8 * e);
            };
            if (!mbar_wait(b_kv, 0)) ok = false;
            for (int u = 0; u < 2 && ok; u++) {
                if (!mbar_wait(b_qf + 8 * u, 0)) { ok = false; break; }
                tc_fence_after();
                issue_sdp(u);
            }
            for (int u = 0; u < n_sub && ok; u++) {
                const int e = u & 1, it = u >> 1, sl = u & 3;
                if (!mbar_wait(b_pds + 8 * e, (u >> 1) & 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t so = (uint32_t)sl * 512;
                // P^T / dS^T in TMEM: the 64 queries packed in columns 0..31 of the buffer
#pragma unroll
                for (int kk = 0; kk < 4; kk++)             // dV += P^T dO   (k = queries)
                    tc_mma_ts(t_dV, t_S + e * 64 + kk * 8, desc_of(loO_n + so + kk * 128), id_acc, (u | kk) != 0);
#pragma unroll
                for (int kk = 0; kk < 4; kk++)             // dK += dS^T Q
                    tc_mma_ts(t_dK, t_dP + e * 64 + kk * 8, desc_of(loQ_n + so + kk * 128), id_acc, (u | kk) != 0);
                tc_commit(b_qe + 8 * sl);                  // the ring slot is free once these have run
                if (u + 2 < n_sub) {
                    if (!mbar_wait(b_qf + 8 * ((u + 2) & 3), ((u + 2) >> 2) & 1)) { ok = false; break; }
                    // S^T/dP^T(u+2) overwrite the buffer whose P^T/dS^T the dV/dK MMAs above read as their A operands:
                    // MMAs on different accumulators are not ordered against each other, so wait for their completion
                    if (!mbar_wait(b_qe + 8 * sl, (u >> 2) & 1)) { ok = false; break; }
                    tc_fence_after();
                    issue_sdp(u + 2);
                }
                if (e == 1) {
                    // the dQ accumulator of tile it-2 must have been moved out
                    if (it >= 2 && !mbar_wait(b_dqe + 8 * (it & 1), ((it >> 1) & 1) ^ 1)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < AT / 16; kk++)   // dQ = dS K   (k = keys) for the whole 128-query tile
                        tc_mma_ss(t_dQ + (it & 1) * 64, desc_of(loDS + (it & 1) * 2048 + kk * 128), desc_of(loK_n + kk * 128), id_dq, kk != 0);
                    tc_commit(b_dq + 8 * (it & 1));
                }
            }
            if (!ok) { *abort_flag = 1; atomicExch(status, STAT_BWD | 1); }
        }
    } else if (warp == CTRL_WARP + 1) {
        // ── TMA loads: K/V once, then the Q/dO sub-tiles through a ring of four slots ──
        if (lane == 0) {
            bool ok = true;
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
            mbar_expect_tx(b_kv, 32768);
            tma_load_4d(sb + BwdSmem::K, &tmK, b_kv, 0, g, j * AT, b);
            tma_load_4d(sb + BwdSmem::V, &tmV, b_kv, 0, g, j * AT, b);
            for (int u = 0; u < n_sub && ok; u++) {
                const int sl = u & 3, it = u >> 1, hh = it / per_head, i = j + it % per_head, h = g * rep + hh;
                // slot sl was last used by sub-tile u-4: free once its dV/dK MMAs have run
                if (u >= 4 && (!mbar_wait(b_qe + 8 * sl, ((u - 4) >> 2) & 1) || *abort_flag)) { ok = false; break; }
                mbar_expect_tx(b_qf + 8 * sl, 16384);
                tma_load_4d(sb + BwdSmem::Q0 + sl * 8192, &tmQ, b_qf + 8 * sl, 0, h, i * AT + (u & 1) * 64, b);
                tma_load_4d(sb + BwdSmem::DO0 + sl * 8192, &tmdO, b_qf + 8 * sl, 0, h, i * AT + (u & 1) * 64, b);
            }
            if (!ok) { *abort_flag = 1; atomicExch(status, STAT_BWD | 4); }
        }
    } else if (warp >= BWD_SM_WARPS) {
        // ── dQ movers: tile t from TMEM -> swizzled fp32 staging -> TMA reduce-add into the fp32 dq buffer ──
        const int dt_ = threadIdx.x - BWD_SM_THREADS;        // 0..127 == TMEM lane == query row
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        bool ok = true;
        for (int t = 0; t < n_it && ok; t++) {
            if (!mbar_wait(b_dq + 8 * (t & 1), (t >> 1) & 1) || *abort_flag) { ok = false; break; }
            tc_fence_after();
            if (dt_ == 0) bulk_wait_read0();                 // the previous reduce has finished reading the staging
            named_bar_sync(2, BWD_DRAIN_THREADS);
#pragma unroll 1
            for (int hf = 0; hf < 2; hf++) {
                uint32_t v[32];
                tmem_ld32(t_dQ + (t & 1) * 64 + lane_base + hf * 32, v);
                tmem_ld_wait();
                uint8_t* dq_row = smem + BwdSmem::DQ + hf * 16384 + dt_ * 128;
#pragma unroll
                for (int k4 = 0; k4 < 8; k4++) {
                    float4 f = make_float4(__uint_as_float(v[k4 * 4]) * scale, __uint_as_float(v[k4 * 4 + 1]) * scale,
                                           __uint_as_float(v[k4 * 4 + 2]) * scale, __uint_as_float(v[k4 * 4 + 3]) * scale);
                    *reinterpret_cast<float4*>(dq_row + ((k4 ^ (dt_ & 7)) << 4)) = f;
                }
            }
            tc_fence_before();
            mbar_arrive(b_dqe + 8 * (t & 1));                // the accumulator may be overwritten
            fence_async_smem();
            named_bar_sync(2, BWD_DRAIN_THREADS);
            if (dt_ == 0) {
                const int hh = t / per_head, i = j + t % per_head, h = g * rep + hh;
                tma_reduce_add_4d(&tmdQ, sb + BwdSmem::DQ, 0, h, i * AT, b);
                tma_reduce_add_4d(&tmdQ, sb + BwdSmem::DQ + 16384, 32, h, i * AT, b);
                bulk_commit();
            }
        }
        if (dt_ == 0) bulk_wait0();
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, STAT_BWD | 3); }
    } else {
        const int r = threadIdx.x & 127;                    // key row of S^T == TMEM lane
        const int e = threadIdx.x >> 7;                     // softmax group == parity of its sub-tiles == TMEM buffer
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const float c = scale * LOG2E;
        float* my_stat = s_stat + warp * 256;               // every warp keeps its own copy: no group barrier needed
        bool ok = true;
        // row statistics of sub-tile u (64 queries): lane l holds lse of queries l, l+32 and D of queries l, l+32
        auto stat_of = [&](int u, float* st4) {
            const int it = u >> 1, hh = it / per_head, i = j + it % per_head, h = g * rep + hh;
            const long long idx = ((long long)b * H + h) * T + i * AT + (u & 1) * 64 + lane;
            st4[0] = lse[idx] * LOG2E; st4[1] = lse[idx + 32] * LOG2E; st4[2] = Dv[idx]; st4[3] = Dv[idx + 32];
        };
        auto stat_put = [&](int buf, const float* st4) {
            float* d = my_stat + buf * 128;
            d[lane] = st4[0]; d[lane + 32] = st4[1]; d[64 + lane] = st4[2]; d[96 + lane] = st4[3];
        };
        {
            float st4[4];
            stat_of(e, st4);
            stat_put(0, st4);
        }
        long long pc[2] = {0, 0};
        const bool timing = prof != nullptr && threadIdx.x == 0;
        const long long t_begin = timing ? clock64() : 0;
        __syncwarp();
        for (int u = e; u < n_sub && ok; u += 2) {
            const int it = u >> 1;
            const int i = j + it % per_head;
            float nxt[4] = {0.f, 0.f, 0.f, 0.f};
            if (u + 2 < n_sub) stat_of(u + 2, nxt);              // this group's next statistics into registers
            const long long c0t = timing ? clock64() : 0;
            if (!mbar_wait(b_sdp + 8 * e, it & 1) || *abort_flag) { ok = false; break; }
            // the dS buffer of this tile was last read by dQ of tile it-2
            if (it >= 2 && !mbar_wait(b_dq + 8 * (it & 1), ((it >> 1) & 1) ^ 1)) { ok = false; break; }
            tc_fence_after();
            const long long c1t = timing ? clock64() : 0;
            const bool diag = i == j;
            const float* L = my_stat + (it & 1) * 128;
            const float* Dr = L + 64;
            uint8_t* ds_row = smem + BwdSmem::DS0 + (it & 1) * 32768 + e * 16384 + r * 128;
#pragma unroll 1
            for (int ch = 0; ch < 2; ch++) {
                uint32_t sv[32], dp[32], wp[16], wd[16];
                tmem_ld32(t_S + e * 64 + lane_base + ch * 32, sv);
                tmem_ld32(t_dP + e * 64 + lane_base + ch * 32, dp);
                tmem_ld_wait();
                if (diag) {                                      // query < key: masked (score -> -inf, so P = dS = 0)
#pragma unroll
                    for (int q = 0; q < 32; q++)
                        if (e * 64 + ch * 32 + q < r) sv[q] = 0xff800000u;
                }
#pragma unroll
                for (int q = 0; q < 32; q += 4) {
                    const int cs = ch * 32 + q;                  // query column within the sub-tile
                    const float4 l4 = *reinterpret_cast<const float4*>(L + cs);       // broadcast 16-byte loads
                    const float4 d4 = *reinterpret_cast<const float4*>(Dr + cs);
                    const float p0 = fast_exp2(__uint_as_float(sv[q]) * c - l4.x);
                    const float p1 = fast_exp2(__uint_as_float(sv[q + 1]) * c - l4.y);
                    const float p2 = fast_exp2(__uint_as_float(sv[q + 2]) * c - l4.z);
                    const float p3 = fast_exp2(__uint_as_float(sv[q + 3]) * c - l4.w);
                    wp[q >> 1] = pack_bf16(p0, p1);
                    wp[(q >> 1) + 1] = pack_bf16(p2, p3);
                    wd[q >> 1] = pack_bf16(p0 * (__uint_as_float(dp[q]) - d4.x), p1 * (__uint_as_float(dp[q + 1]) - d4.y));
                    wd[(q >> 1) + 1] = pack_bf16(p2 * (__uint_as_float(dp[q + 2]) - d4.z), p3 * (__uint_as_float(dp[q + 3]) - d4.w));
                }
                // packed columns ch*16 .. ch*16+15 of the buffer: inside the columns this thread has already read
                tmem_st16(t_S + e * 64 + lane_base + ch * 16, wp);
                tmem_st16(t_dP + e * 64 + lane_base + ch * 16, wd);
                // dS^T also to shared memory (A operand of dQ): block = sub-tile, 16-byte chunk index XOR (row & 7)
#pragma unroll
                for (int k4 = 0; k4 < 4; k4++) {
                    const int chunk = ch * 4 + k4;
                    uint4 pk = make_uint4(wd[k4 * 4], wd[k4 * 4 + 1], wd[k4 * 4 + 2], wd[k4 * 4 + 3]);
                    *reinterpret_cast<uint4*>(ds_row + ((chunk ^ (r & 7)) << 4)) = pk;
                }
            }
            tmem_st_wait();
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(b_pds + 8 * e);
            if (timing) { const long long c2t = clock64(); pc[0] += c1t - c0t; pc[1] += c2t - c1t; }
            if (u + 2 < n_sub) stat_put((it + 1) & 1, nxt);
            __syncwarp();                                    // publishes the statistics just written within the warp
        }
        if (timing) {
            long long* pp = prof + 8 * (long long)blockIdx.x;
            pp[0] = pc[0]; pp[1] = pc[1]; pp[2] = 0; pp[3] = 0; pp[4] = clock64() - t_begin; pp[5] = n_it;
        }
        // dV (group 0) and dK (group 1): complete once the last dQ commit has fired
        if (ok && !mbar_wait(b_dq + 8 * ((n_it - 1) & 1), ((n_it - 1) >> 1) & 1)) ok = false;
        if (ok) {
            tc_fence_after();
            const int t = j * AT + r;
            const uint32_t ta = e ? t_dK : t_dV;
            const float f = e ? scale : 1.f;
            bf16* dst = (e ? dk : dv) + (((long long)b * T + t) * KV + g) * ADH;
#pragma unroll 1
            for (int ch = 0; ch < 2; ch++) {
                uint32_t v[32];
                tmem_ld32(ta + lane_base + ch * 32, v);
                tmem_ld_wait();
                if (t < T) {
#pragma unroll
                    for (int q = 0; q < 32; q += 8) {
                        uint4 pk;
                        pk.x = pack_bf16(__uint_as_float(v[q]) * f, __uint_as_float(v[q + 1]) * f);
                        pk.y = pack_bf16(__uint_as_float(v[q + 2]) * f, __uint_as_float(v[q + 3]) * f);
                        pk.z = pack_bf16(__uint_as_float(v[q + 4]) * f, __uint_as_float(v[q + 5]) * f);
                        pk.w = pack_bf16(__uint_as_float(v[q + 6]) * f, __uint_as_float(v[q + 7]) * f);
                        *reinterpret_cast<uint4*>(dst + ch * 32 + q) = pk;
                    }
                }
            }
        } else if (lane == 0) {
            *abort_flag = 1;
            atomicExch(status, STAT_BWD | 2);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == CTRL_WARP) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// fp32 dq accumulator -> bf16 dq (same [B,T,H,DH] layout)
__global__ void k_dq_convert(const float* __restrict__ src, bf16* __restrict__ dst, long long n8) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        float f[8];
        Vec<float>::ld(src + i * 8, f);
        Vec<float>::ld(src + i * 8 + 4, f + 4);
        Vec<bf16>::st(dst + i * 8, f);
    }
}

// ── host ────────────────────────────────────────────────────────────────────
int ax_attn_tc_init(void) {
    int rc = ax_attn_tc128_init();
    rc |= (int)cudaFuncSetAttribute(k_attn_fwd_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem::TOTAL);
    rc |= (int)cudaFuncSetAttribute(k_attn_bwd_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::TOTAL);
    return rc;
}

static bool served(const AttnShape& s) {
    // [B,T,H,DH] layout, head_dim 64, whole tiles
    return s.DH == ADH && s.T % AT == 0 && s.T >= AT && s.qh == ADH && s.kh == ADH &&
           s.qt == (long long)s.H * ADH && s.kt == (long long)s.KV * ADH && s.H % s.KV == 0;
}
static int map_bthd(CUtensorMap* m, const void* base, int B, int T, int heads, int rows = AT) {
    uint64_t dims[4] = {ADH, (uint64_t)heads, (uint64_t)T, (uint64_t)B};
    uint64_t strides[3] = {(uint64_t)ADH * 2, (uint64_t)heads * ADH * 2, (uint64_t)T * heads * ADH * 2};
    uint32_t box[4] = {ADH, 1, (uint32_t)rows, 1};
    return tc_make_tmap_bf16(m, base, 4, dims, strides, box, true);
}
static int map_dq_f32(CUtensorMap* m, const void* base, int B, int T, int heads) {
    PFN_tmapEncodeTiled enc = tc_encode_fn();
    if (!enc) return 1;
    cuuint64_t gd[4] = {ADH, (cuuint64_t)heads, (cuuint64_t)T, (cuuint64_t)B};
    cuuint64_t gs[3] = {(cuuint64_t)ADH * 4, (cuuint64_t)heads * ADH * 4, (cuuint64_t)T * heads * ADH * 4};
    cuuint32_t bx[4] = {32, 1, AT, 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 2;
}

int ax_attn_fwd_tc(const void* q, const void* k, const void* v, void* o, float* lse,
                   const AttnShape& s, int* status, cudaStream_t st) {
    if (s.DH == 128) return ax_attn_fwd_tc128(q, k, v, o, lse, s, status, st);
    if (!served(s) || !lse || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return -1;
    CUtensorMap tq, tk, tv;
    if (map_bthd(&tq, q, s.B, s.T, s.H) || map_bthd(&tk, k, s.B, s.T, s.KV) || map_bthd(&tv, v, s.B, s.T, s.KV)) return 2;
    dim3 grid((s.T / AT) * s.H * s.B);
    k_attn_fwd_tc<<<grid, ATT_THREADS, FwdSmem::TOTAL, st>>>(tq, tk, tv, (bf16*)o, lse, s.T, s.H, s.KV, s.scale, status);
    return 0;
}

int ax_attn_bwd_tc(const void* q, const void* k, const void* v, const void* o, const void* dO,
                   const float* lse, float* Dscratch, float* g_dq_acc, void* dq, void* dk, void* dv,
                   const AttnShape& s, int* status, cudaStream_t st) {
    if (s.DH == 128) return ax_attn_bwd_tc128(q, k, v, o, dO, lse, Dscratch, g_dq_acc, dq, dk, dv, s, status, st);
    if (!served(s) || !g_dq_acc || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(dO) ||
        !aligned16(dq) || !aligned16(dk) || !aligned16(dv) || !aligned16(g_dq_acc)) return -1;
    const size_t need = (size_t)s.B * s.T * s.H * ADH * 4;
    CUtensorMap tq, tk, tv, tdo, tdq;
    if (map_bthd(&tq, q, s.B, s.T, s.H, 64) || map_bthd(&tk, k, s.B, s.T, s.KV) || map_bthd(&tv, v, s.B, s.T, s.KV) ||
        map_bthd(&tdo, dO, s.B, s.T, s.H, 64) || map_dq_f32(&tdq, g_dq_acc, s.B, s.T, s.H)) return 2;
    cudaMemsetAsync(g_dq_acc, 0, need, st);
    const long long rows = (long long)s.B * s.T * s.H;
    k_attn_bwd_prep<<<ew_grid(rows * 8, 256), 256, 0, st>>>((const bf16*)o, (const bf16*)dO, Dscratch, s.B, s.T, s.H);
    dim3 grid((s.T / AT) * s.KV * s.B);
    static const bool want_prof = getenv("AXENG_ATTN_PROF") != nullptr;
    long long* prof = nullptr;
    const int nblk = (s.T / AT) * s.KV * s.B;
    if (want_prof && cudaMalloc(&prof, (size_t)nblk * 64) != cudaSuccess) prof = nullptr;
    k_attn_bwd_tc<<<grid, BWD_THREADS, BwdSmem::TOTAL, st>>>(tq, tk, tv, tdo, tdq, lse, Dscratch, (bf16*)dk, (bf16*)dv,
                                                              s.T, s.H, s.KV, s.scale, status, prof);
    if (prof) {     // debugging aid: phase cycle counts summed over CTAs, printed to stderr
        std::vector<long long> h((size_t)nblk * 8);
        cudaStreamSynchronize(st);
        cudaMemcpy(h.data(), prof, (size_t)nblk * 64, cudaMemcpyDeviceToHost);
        cudaFree(prof);
        long long sum[6] = {0, 0, 0, 0, 0, 0}, mx = 0;
        for (int i = 0; i < nblk; i++) { for (int q = 0; q < 6; q++) sum[q] += h[i * 8 + q]; if (h[i * 8 + 4] > mx) mx = h[i * 8 + 4]; }
        fprintf(stderr, "attn_bwd phases (cycles per 128-query tile): wait_sdp %.0f softmax %.0f total %.0f | tiles %lld, longest CTA %lld cycles\n",
                (double)sum[0] / sum[5], (double)sum[1] / sum[5], (double)sum[4] / sum[5], sum[5], mx);
    }
    const long long n8 = rows * ADH / 8;
    k_dq_convert<<<ew_grid(n8, 256), 256, 0, st>>>(g_dq_acc, (bf16*)dq, n8);
    return 0;
}
