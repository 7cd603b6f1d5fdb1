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

#ifdef AXENG_PROF
#include <cstdio>
#include <cstdlib>
#include <vector>
#endif

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

// Issue forms for a converged warp: every lane executes the surrounding code (so addresses and descriptors stay
// warp-uniform and cheap to form) and the elected lane issues.  Measured on B200: a 128 x 64 x 16 MMA with A in
// TMEM issues every 32.6 cycles this way (its 32 cycles of math) against 45-50 from a lone thread in a divergent branch.
__device__ __forceinline__ void mma_ts_e(uint32_t d, uint32_t a, uint64_t bd, uint32_t id, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p, q;\n\telect.sync _|q, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d), "r"(a), "l"(bd), "r"(id), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma_ss_e(uint32_t d, uint64_t ad, uint64_t bd, uint32_t id, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p, q;\n\telect.sync _|q, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d), "l"(ad), "l"(bd), "r"(id), "r"(acc) : "memory");
}
__device__ __forceinline__ void commit_e(uint32_t bar) {
    asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
                 "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar) : "memory");
}

// Forward CTA: 128 queries of one head; four softmax warps (a thread owns a query row) and one control warp that
// loads by TMA and issues the MMAs.  TMEM (256 columns, two CTAs per SM): S 0..127, P 128..191 (packed bf16),
// O 192..255.  P has columns of its own, so S(j+1) = Q K(j+1)^T is issued as soon as the softmax threads have read
// S(j) into registers and runs under the exponentials of tile j; K and V tiles travel on separate barriers (a K slot
// is free once its S MMA has run, a V slot once its P V MMA has).
__global__ void __launch_bounds__(ATT_THREADS, 2)
k_attn_fwd_tc(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, bf16* __restrict__ o, float* __restrict__ lse,
              int T, int H, int KV, float scale, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sb = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FwdSmem::BARS);
    // q_full, k_full[2], v_full[2], s_full, s_free, p_full, o_done
    const uint32_t b_q = smem_u32(bars), b_kf = b_q + 8, b_vf = b_kf + 16, b_s = b_vf + 16, b_sfree = b_s + 8, b_p = b_sfree + 8,
                   b_o = b_p + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
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
        for (int s = 0; s < 2; s++) { mbar_init(b_kf + 8 * s, 1); mbar_init(b_vf + 8 * s, 1); }
        mbar_init(b_s, 1); mbar_init(b_sfree, 128); mbar_init(b_p, 128); mbar_init(b_o, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) { tmem_alloc(smem_u32(tmem_slot), 256); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_S = tmem, t_P = tmem + 128, t_O = tmem + 192;

    if (warp == 4) {
        // ── control warp (converged; one elected lane issues MMAs, lane 0 issues the TMA loads) ──
        bool ok = true;
        constexpr uint32_t id_s = tc_idesc_bf16(128, 128, 0, 0);
        constexpr uint32_t id_pv = tc_idesc_bf16(128, 64, 0, 1);
        const uint32_t loQ = desc_lo(sb + FwdSmem::Q, 16), loK = desc_lo(sb + FwdSmem::K0, 16), loV = desc_lo(sb + FwdSmem::V0, 16384);
        auto load_k = [&](int j) {
            if (lane == 0) {
                mbar_expect_tx(b_kf + 8 * (j & 1), 16384);
                tma_load_4d(sb + FwdSmem::K0 + (j & 1) * 16384, &tmK, b_kf + 8 * (j & 1), 0, g, j * AT, b);
            }
        };
        auto load_v = [&](int j) {
            if (lane == 0) {
                mbar_expect_tx(b_vf + 8 * (j & 1), 16384);
                tma_load_4d(sb + FwdSmem::V0 + (j & 1) * 16384, &tmV, b_vf + 8 * (j & 1), 0, g, j * AT, b);
            }
        };
        auto issue_s = [&](int j) {
#pragma unroll
            for (int kk = 0; kk < ADH / 16; kk++)
                mma_ss_e(t_S, desc_of(loQ + kk * 2), desc_of(loK + (j & 1) * 1024 + kk * 2), id_s, kk != 0);
            commit_e(b_s);
        };
        if (lane == 0) {
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
            mbar_expect_tx(b_q, 16384);
            tma_load_4d(sb + FwdSmem::Q, &tmQ, b_q, 0, h, qt * AT, b);
        }
        load_k(0); load_v(0);
        if (nkt > 1) { load_k(1); load_v(1); }
        __syncwarp();
        if (!mbar_wait_park(b_q, 0) || !mbar_wait_park(b_kf, 0)) ok = false;
        if (ok) { tc_fence_after(); issue_s(0); }
        for (int j = 0; j < nkt && ok; j++) {
            const int s = j & 1;
            if (j + 1 < nkt) {
                // S(j+1): its K tile has landed and every softmax thread holds S(j) in registers
                if (!mbar_wait_park(b_kf + 8 * (s ^ 1), ((j + 1) >> 1) & 1) || !mbar_wait_park(b_sfree, j & 1) || *abort_flag) { ok = false; break; }
                tc_fence_after();
                issue_s(j + 1);
                // K slot s was read by S(j), complete long since (its result has been read): K(j+2) may overwrite it
                if (j + 2 < nkt) { load_k(j + 2); __syncwarp(); }
            }
            // O += P(j) V(j)
            if (!mbar_wait_park(b_vf + 8 * s, (j >> 1) & 1) || !mbar_wait_park(b_p, j & 1) || *abort_flag) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < AT / 16; kk++)
                mma_ts_e(t_O, t_P + kk * 8, desc_of(loV + s * 1024 + kk * 128), id_pv, (j | kk) != 0);
            commit_e(b_o);
            if (j + 2 < nkt) {                          // V slot s is free once P V(j) has run
                if (!mbar_wait_park(b_o, j & 1)) { ok = false; break; }
                load_v(j + 2);
                __syncwarp();
            }
        }
        __syncwarp();
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, STAT_FWD | 1); }
    } else {
        const int r = threadIdx.x;                         // query row within the tile == TMEM lane
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float c = scale * LOG2E;
        const float2 c2 = make_float2(c, c);
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nkt && ok; j++) {
            if (!mbar_wait_park(b_s, j & 1) || *abort_flag) { ok = false; break; }
            tc_fence_after();
            const bool diag = j == qt;
            // the whole S row (128 scores) goes into registers; the buffer is then free for S(j+1)
            uint32_t sv[128];
#pragma unroll
            for (int ch = 0; ch < 4; ch++) tmem_ld32(t_S + lane_base + ch * 32, sv + ch * 32);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(b_sfree);
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
                    if (!mbar_wait_park(b_o, (j - 1) & 1)) { ok = false; break; }
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
            // P(j-1) is read by P V(j-1): it must have run before the columns are rewritten
            if (j >= 1 && !mbar_wait_park(b_o, (j - 1) & 1)) { ok = false; break; }
            {
                const float2 nm2 = make_float2(-m_used, -m_used);
                float2 l2 = make_float2(0.f, 0.f);
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    uint32_t w[16];
#pragma unroll
                    for (int q = 0; q < 32; q += 4) {
                        // packed fp32x2 arithmetic: one instruction per pair of scores
                        const float2 x01 = __ffma2_rn(make_float2(__uint_as_float(sv[ch * 32 + q]), __uint_as_float(sv[ch * 32 + q + 1])), c2, nm2);
                        const float2 x23 = __ffma2_rn(make_float2(__uint_as_float(sv[ch * 32 + q + 2]), __uint_as_float(sv[ch * 32 + q + 3])), c2, nm2);
                        const float2 p01 = make_float2(fast_exp2(x01.x), fast_exp2(x01.y));
                        const float2 p23 = make_float2(fast_exp2(x23.x), fast_exp2(x23.y));
                        l2 = __fadd2_rn(l2, __fadd2_rn(p01, p23));
                        w[q >> 1] = pack_bf16(p01.x, p01.y);
                        w[(q >> 1) + 1] = pack_bf16(p23.x, p23.y);
                    }
                    tmem_st16(t_P + lane_base + ch * 16, w);
                }
                l += l2.x + l2.y;
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(b_p);
        }
        if (ok && mbar_wait_park(b_o, (nkt - 1) & 1)) {
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

// Backward CTA (800 threads): sixteen softmax warps — two groups (group e owns the sub-tiles of parity e and the
// TMEM buffers e), each of two column halves times four lane quarters, so that a thread owns one key row and 32
// of the 64 query columns of its sub-tile — 4 warps that move finished dQ tiles out (TMEM -> shared memory -> TMA
// reduce-add), 5 MMA-issue warps (one per product; the S^T issuer also feeds the Q / dO ring by TMA).  Four softmax warps per scheduler hide the 250-cycle
// round trip of a TMEM load behind each other's arithmetic.
//
// The backward works on sub-tiles of 64 queries.  An MMA whose two operands both come from shared memory is
// bound by the operand fetch, not the math (a 128 x 64 x 16 step reads 6 KB for 32 cycles of math and takes
// about three times that), so every product that can takes its 128-row operand from TMEM instead:
//   K, V              copied once into TMEM as packed bf16 (32 columns each): the A operands of S^T = K Q^T and
//                     dP^T = V dO^T; only the 64-query Q / dO tiles are read from shared memory.
//   S^T[e], dP^T[e]   fp32 scores of sub-tile u (e = u & 1); P^T and dS^T replace them in place as packed bf16
//                     (columns 0..31) and are the A operands of dV += P^T dO and dK += dS^T Q.
//   dS^T              also goes to shared memory (swizzled rows of 64 queries): the M-major A operand of
//                     dQ = dS K per 128-query tile, the one product with both operands in shared memory.
//   dV, dK, dQ        accumulators; dQ is single: the movers drain tile t while the sub-tiles of t+1 run.
// Every product has its own issuing warp, each in program order behind its own barriers: a warp issues one small
// MMA about every 50 cycles in this code, and the batches of a sub-tile (S^T and dP^T; dV and dK) sit on the
// critical path between two softmax passes, so they are issued side by side instead of one after the other.
// A softmax thread takes its 32 columns in two rounds of 16 (S^T and dP^T loaded together, P^T and dS^T written
// back in place), with packed fp32x2 arithmetic.
#define BWD_SM_WARPS 16
#define BWD_SM_THREADS (BWD_SM_WARPS * 32)
#define BWD_DRAIN_THREADS 128
#define BWD_THREADS (BWD_SM_THREADS + BWD_DRAIN_THREADS + 160)
#define BWD_SLOTS 5            // Q/dO ring: 64-query sub-tiles in flight
struct BwdSmem {
    static constexpr int K = 0, V = 16384, Q0 = 32768, DO0 = Q0 + BWD_SLOTS * 8192, DS0 = DO0 + BWD_SLOTS * 8192,
                         DQ = DS0 + 2 * 32768, STAT = DQ + 32768, BARS = STAT + 8192, TOTAL = BARS + 512 + 1024;
};
static_assert(BwdSmem::TOTAL <= 227 * 1024, "backward shared memory exceeds the per-CTA limit");
static_assert(BwdSmem::DO0 % 1024 == 0 && BwdSmem::DS0 % 1024 == 0 && BwdSmem::DQ % 1024 == 0, "swizzled tiles need 1024-byte alignment");

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}

#ifdef AXENG_PROF
// instrumented builds only: per-CTA cycle counters (16 long long per CTA), see the host launcher
__device__ long long* g_bwd_prof = nullptr;
#define PROF_T() clock64()
#define PROF_ADD(slot, v) do { pa[slot] += (v); } while (0)
#define PROF_FLUSH(lo, hi) do { if (pf) for (int q_ = (lo); q_ < (hi); q_++) pf[q_] = pa[q_]; } while (0)
#else
#define PROF_T() 0ll
#define PROF_ADD(slot, v) do { } while (0)
#define PROF_FLUSH(lo, hi) do { } while (0)
#endif

__global__ void __launch_bounds__(BWD_THREADS, 1)
k_attn_bwd_tc(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
              const __grid_constant__ CUtensorMap tmdQ, const float* __restrict__ lse, const float* __restrict__ Dv,
              bf16* __restrict__ dk, bf16* __restrict__ dv, int T, int H, int KV, float scale,
              const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sb = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BwdSmem::BARS);
    // kv_full, q_full[5], q_empty[5], sdp_full[2], (unused)[2], pds_full[2], dq_full[2], dq_empty, kv_in_tmem
    const uint32_t b_kv = smem_u32(bars), b_qf = b_kv + 8, b_qe = b_qf + 8 * BWD_SLOTS, b_s = b_qe + 8 * BWD_SLOTS,
                   b_dp = b_s + 16, b_pds = b_dp + 16, b_dq = b_pds + 16, b_dqe = b_dq + 16, b_kvt = b_dqe + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_stat = reinterpret_cast<float*>(smem + BwdSmem::STAT);   // [softmax warp][2][lse*log2(e) 64 | D 64]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int CTRL_WARP = BWD_SM_WARPS + 4;
#ifdef AXENG_PROF
    // slots: softmax group 0 thread 0: [0] wait S [1] phase A [2] wait dP/dS buffer [3] phase B [4] wait P^T free
    // [5] stores; issuing thread: [8] loop cycles [9] idle polls [10] batches issued [11] cycles inside issue;
    // mover thread 0: [12] wait [13] work; [15] sub-tiles
    long long* pf = (g_bwd_prof && (threadIdx.x == 0 || threadIdx.x == CTRL_WARP * 32 || threadIdx.x == (CTRL_WARP + 2) * 32 || threadIdx.x == BWD_SM_THREADS))
                        ? g_bwd_prof + 32 * (long long)blockIdx.x : nullptr;
    long long pa[24] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};      // kept in registers, written once at the end
#endif
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
        for (int s = 0; s < BWD_SLOTS; s++) { mbar_init(b_qf + 8 * s, 1); mbar_init(b_qe + 8 * s, 2); }
        for (int s = 0; s < 2; s++) {
            mbar_init(b_s + 8 * s, 2); mbar_init(b_dp + 8 * s, 1);
            mbar_init(b_pds + 8 * s, 256); mbar_init(b_dq + 8 * s, 1);
        }
        mbar_init(b_dqe, BWD_DRAIN_THREADS);
        mbar_init(b_kvt, BWD_SM_THREADS);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == CTRL_WARP) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // columns: S^T/P^T[2] 0..127, dP^T/dS^T[2] 128..255, dV 256..319, dK 320..383, dQ 384..447, K 448..479, V 480..511
    const uint32_t t_S = tmem, t_dP = tmem + 128, t_dV = tmem + 256, t_dK = tmem + 320, t_dQ = tmem + 384,
                   t_K = tmem + 448, t_V = tmem + 480;

    if (warp == CTRL_WARP || warp == CTRL_WARP + 1) {
        // ── issuers of S^T = K Q^T (warp CTRL_WARP, which also feeds the Q / dO ring) and dP^T = V dO^T
        //    (CTRL_WARP + 1): the whole warp runs converged, one elected lane issues ──
        const bool is_s = warp == CTRL_WARP;
        bool ok = true;
        constexpr uint32_t id_s = tc_idesc_bf16(128, 64, 0, 0);        // A in TMEM, B K-major
        const uint32_t loB = is_s ? desc_lo(sb + BwdSmem::Q0, 16) : desc_lo(sb + BwdSmem::DO0, 16);
        const uint32_t tA = is_s ? t_K : t_V, tD = is_s ? t_S : t_dP;
        // ring producer state (S issuer only): next sub-tile to load, its head / causal tile, and the slot it goes to
        int lu = 0, lhh = 0, lii = 0;
        auto load_sub = [&](int slot) {
            if (lane == 0) {
                const int i = j + lii, h = g * rep + lhh;
                mbar_expect_tx(b_qf + 8 * slot, 16384 + 512);
                tma_load_4d(sb + BwdSmem::Q0 + slot * 8192, &tmQ, b_qf + 8 * slot, 0, h, i * AT + (lu & 1) * 64, b);
                tma_load_4d(sb + BwdSmem::DO0 + slot * 8192, &tmdO, b_qf + 8 * slot, 0, h, i * AT + (lu & 1) * 64, b);
                // the sub-tile's row statistics (64 lse, 64 D) ride on the same barrier
                const long long sidx = ((long long)b * H + h) * T + i * AT + (lu & 1) * 64;
                bulk_load_1d(sb + BwdSmem::STAT + 4096 + slot * 512, lse + sidx, 256, b_qf + 8 * slot);
                bulk_load_1d(sb + BwdSmem::STAT + 4096 + slot * 512 + 256, Dv + sidx, 256, b_qf + 8 * slot);
            }
            if ((lu & 1) && ++lii == per_head) { lii = 0; lhh++; }
            lu++;
        };
        if (is_s) {
            if (lane == 0) {
                tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
                mbar_expect_tx(b_kv, 32768);
                tma_load_4d(sb + BwdSmem::K, &tmK, b_kv, 0, g, j * AT, b);
                tma_load_4d(sb + BwdSmem::V, &tmV, b_kv, 0, g, j * AT, b);
            }
            for (int q = 0; q < BWD_SLOTS && q < n_sub; q++) load_sub(q);
            __syncwarp();
        }
        if (!mbar_wait_park(b_kvt, 0)) ok = false;           // K and V are in TMEM
        tc_fence_after();
        int sl = 0, ph = 0;                             // ring slot of sub-tile u and its fill parity
        int sl_p = 0, ph_p = 0;                         // slot / release parity of sub-tile u - 2
        const long long t_loop = PROF_T();
        for (int u = 0; u < n_sub && ok; u++) {
            const long long tw = PROF_T();
            if (!mbar_wait_park(b_qf + 8 * sl, ph) || *abort_flag) { ok = false; break; }
            // dV/dK(u-2) have finished reading P^T / dS^T out of the two buffers that S^T / dP^T(u) overwrite
            // (MMAs on different accumulators are not ordered against each other: wait for the commits)
            int freed = -1;
            if (u >= 2) {
                if (!mbar_wait_park(b_qe + 8 * sl_p, ph_p)) { ok = false; break; }
                freed = sl_p;                           // that sub-tile's ring slot is free as well
                if (++sl_p == BWD_SLOTS) { sl_p = 0; ph_p ^= 1; }
            }
            tc_fence_after();
            const long long tq = PROF_T();
            PROF_ADD(9, tq - tw);
            const uint32_t so = (uint32_t)sl * 512;          // ring slot offset (8192 B)
            const uint32_t d_ = tD + (u & 1) * 64;
#pragma unroll
            for (int kk = 0; kk < ADH / 16; kk++)
                mma_ts_e(d_, tA + kk * 8, desc_of(loB + so + kk * 2), id_s, kk != 0);
            commit_e(b_s + 8 * (u & 1));               // two arrivals (S^T and dP^T) complete the phase
            PROF_ADD(16, PROF_T() - tq);
            if (is_s && freed >= 0 && lu < n_sub) { load_sub(freed); __syncwarp(); }
            if (++sl == BWD_SLOTS) { sl = 0; ph ^= 1; }
        }
        PROF_ADD(8, PROF_T() - t_loop); PROF_ADD(15, n_sub);
        __syncwarp();
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, STAT_BWD | 1); }
        if (is_s) { PROF_FLUSH(8, 12); PROF_FLUSH(15, 20); }
    } else if (warp == CTRL_WARP + 2 || warp == CTRL_WARP + 3) {
        // ── issuers of dV += P^T dO (CTRL_WARP + 2) and dK += dS^T Q (CTRL_WARP + 3) ──
        const bool is_v = warp == CTRL_WARP + 2;
        bool ok = true;
        constexpr uint32_t id_acc = tc_idesc_bf16(128, 64, 0, 1);      // A in TMEM, B N-major
        const uint32_t loB = is_v ? desc_lo(sb + BwdSmem::DO0, 16384) : desc_lo(sb + BwdSmem::Q0, 16384);
        const uint32_t tA = is_v ? t_S : t_dP, tD = is_v ? t_dV : t_dK;
        int sl = 0;
        for (int u = 0; u < n_sub && ok; u++) {
            const int e = u & 1, it = u >> 1;
            const long long tw = PROF_T();
            if (!mbar_wait_park(b_pds + 8 * e, it & 1) || *abort_flag) { ok = false; break; }
            tc_fence_after();
            const long long tq = PROF_T();
            PROF_ADD(20, tq - tw);
            const uint32_t so = (uint32_t)sl * 512;
            const uint32_t acc = u != 0;
            // A operand: packed bf16 in the sub-tile's buffer; 16 queries per k-step = 8 packed columns, the packed
            // columns of column half h start at column 32 h
#pragma unroll
            for (int kk = 0; kk < 4; kk++)
                mma_ts_e(tD, tA + e * 64 + (kk >> 1) * 32 + (kk & 1) * 8, desc_of(loB + so + kk * 128), id_acc, kk ? 1u : acc);
            commit_e(b_qe + 8 * sl);                   // two arrivals (dV and dK): the ring slot and both buffers are free
            PROF_ADD(19, PROF_T() - tq);
            if (++sl == BWD_SLOTS) sl = 0;
        }
        __syncwarp();
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, STAT_BWD | 5); }
        if (is_v) PROF_FLUSH(18, 22);
    } else if (warp == CTRL_WARP + 4) {
        // ── issuer of dQ(it) = dS K for every 128-query tile: both sub-tiles' dS^T are in shared memory and the
        //    movers have drained the accumulator of tile it-1 ──
        bool ok = true;
        constexpr uint32_t id_dq = tc_idesc_bf16(128, 64, 1, 1);       // A M-major (dS^T in smem), B N-major
        const uint32_t loK_n = desc_lo(sb + BwdSmem::K, 16384), loDS_m = desc_lo(sb + BwdSmem::DS0, 16384);
        for (int it = 0; it < n_it && ok; it++) {
            if (!mbar_wait_park(b_pds, it & 1) || !mbar_wait_park(b_pds + 8, it & 1) || *abort_flag) { ok = false; break; }
            if (it >= 1 && !mbar_wait_park(b_dqe, (it - 1) & 1)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < AT / 16; kk++)   // k = keys
                mma_ss_e(t_dQ, desc_of(loDS_m + (it & 1) * 2048 + kk * 128), desc_of(loK_n + kk * 128), id_dq, kk != 0);
            commit_e(b_dq + 8 * (it & 1));
        }
        __syncwarp();
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, STAT_BWD | 6); }
    } else if (warp >= BWD_SM_WARPS) {
        // ── dQ movers: tile t from TMEM -> swizzled fp32 staging -> TMA reduce-add into the fp32 dq buffer ──
        const int dt_ = threadIdx.x - BWD_SM_THREADS;        // 0..127 == TMEM lane == query row
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        bool ok = true;
        int hh = 0, ii = 0;
        for (int t = 0; t < n_it && ok; t++) {
            const long long tm0 = PROF_T();
            if (!mbar_wait_park(b_dq + 8 * (t & 1), (t >> 1) & 1) || *abort_flag) { ok = false; break; }
            tc_fence_after();
            const long long tm1 = PROF_T();
            PROF_ADD(12, tm1 - tm0);
            if (dt_ == 0) bulk_wait_read0();                 // the previous reduce has finished reading the staging
            named_bar_sync(2, BWD_DRAIN_THREADS);
#pragma unroll 1
            for (int hf = 0; hf < 2; hf++) {
                uint32_t v[32];
                tmem_ld32(t_dQ + lane_base + hf * 32, v);
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
            mbar_arrive(b_dqe);                              // the accumulator may be overwritten
            fence_async_smem();
            named_bar_sync(2, BWD_DRAIN_THREADS);
            if (dt_ == 0) {
                const int i = j + ii, h = g * rep + hh;
                tma_reduce_add_4d(&tmdQ, sb + BwdSmem::DQ, 0, h, i * AT, b);
                tma_reduce_add_4d(&tmdQ, sb + BwdSmem::DQ + 16384, 32, h, i * AT, b);
                bulk_commit();
            }
            if (++ii == per_head) { ii = 0; hh++; }
            PROF_ADD(13, PROF_T() - tm1);
        }
        if (dt_ == 0) bulk_wait0();
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, STAT_BWD | 3); }
        if (dt_ == 0) PROF_FLUSH(12, 14);
    } else {
        // warp = 8 e + 4 hc + quarter: group e, column half hc, TMEM lane quarter (a warp reaches the 32 lanes
        // of quarter warp % 4 only)
        const int r = threadIdx.x & 127;                    // key row of S^T == TMEM lane
        const int e = warp >> 3;                            // softmax group == parity of its sub-tiles == TMEM buffer
        const int hc = (warp >> 2) & 1;                     // which 32 of the sub-tile's 64 query columns
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const float c = scale * LOG2E;
        // The TMA warp brings the 64 lse and 64 D values of a sub-tile into the ring slot beside its Q / dO tiles.
        // Each warp turns its 32 of them into -lse*log2(e) and -D in a private area (no barrier beyond the warp),
        // from where the arithmetic loop takes them with broadcast 16-byte loads.  (A softmax warp never loads
        // from global memory itself: the first scoreboard wait behind such a load would expose its latency.)
        float* my_stat = s_stat + warp * 64;                // [-lse*log2(e) 32 | -D 32]
        const float* ring_stat = s_stat + 1024;             // [slot][lse 64 | D 64]
        bool ok = true;
        int sl_u = e, ph_u = 0, ii_c = 0;                    // ring slot (with fill parity) and causal tile index of the current sub-tile
        // K (group 0) / V (group 1) from the swizzled shared-memory tile into TMEM: a thread copies half of its row
        // (a row is 128 bytes = 32 packed columns; 16-byte chunk c sits at position c ^ (row & 7))
        if (!mbar_wait_park(b_kv, 0)) ok = false;
        if (ok) {
            const uint8_t* row = smem + (e ? BwdSmem::V : BwdSmem::K) + r * 128;
            uint32_t w[16];
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
                const uint4 x = *reinterpret_cast<const uint4*>(row + (((hc * 4 + c4) ^ (r & 7)) << 4));
                w[c4 * 4] = x.x; w[c4 * 4 + 1] = x.y; w[c4 * 4 + 2] = x.z; w[c4 * 4 + 3] = x.w;
            }
            tmem_st16((e ? t_V : t_K) + lane_base + hc * 16, w);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(b_kvt);
        }
        const float2 c2 = make_float2(c, c);
        long long t_prev = PROF_T();
        for (int u = e; u < n_sub && ok; u += 2) {
            const int it = u >> 1;
            const bool diag = ii_c == 0;
            if (++ii_c == per_head) ii_c = 0;
            const float* L = my_stat;
            const float* Dr = L + 32;
            const long long ta0 = PROF_T();
            PROF_ADD(6, ta0 - t_prev);
            if (!mbar_wait_park(b_s + 8 * e, it & 1) || *abort_flag) { ok = false; break; }
            // the dS^T shared-memory buffer of this tile parity was last read by dQ of tile it-2
            if (it >= 2 && !mbar_wait_park(b_dq + 8 * (it & 1), ((it >> 1) & 1) ^ 1)) { ok = false; break; }
            tc_fence_after();
            const long long ta1 = PROF_T();
            PROF_ADD(0, ta1 - ta0);
            {
                // the slot's barrier completed long ago (S^T was issued behind it); observing it here makes the
                // bulk-copied statistics visible to this thread
                if (!mbar_wait_park(b_qf + 8 * sl_u, ph_u)) { ok = false; break; }
                const float* rs = ring_stat + sl_u * 128 + hc * 32 + lane;
                my_stat[lane] = -rs[0] * LOG2E;
                my_stat[32 + lane] = -rs[64];
                sl_u += 2;
                if (sl_u >= BWD_SLOTS) { sl_u -= BWD_SLOTS; ph_u ^= 1; }
                __syncwarp();
            }
            uint8_t* ds_row = smem + BwdSmem::DS0 + (it & 1) * 32768 + e * 16384 + r * 128;
            const uint32_t tS = t_S + e * 64 + hc * 32 + lane_base, tdP = t_dP + e * 64 + hc * 32 + lane_base;
#pragma unroll
            for (int rd = 0; rd < 2; rd++) {                     // two rounds of 16 query columns
                uint32_t sv[16], dp[16], wp[8], wd[8];
                tmem_ld16(tS + rd * 16, sv);
                tmem_ld16(tdP + rd * 16, dp);
                tmem_ld_wait();
                if (diag) {                                      // query < key: masked (score -> -inf, so P = dS = 0)
#pragma unroll
                    for (int q = 0; q < 16; q++)
                        if (e * 64 + hc * 32 + rd * 16 + q < r) sv[q] = 0xff800000u;
                }
#pragma unroll
                for (int q = 0; q < 16; q += 4) {
                    const float4 l4 = *reinterpret_cast<const float4*>(L + rd * 16 + q);       // broadcast 16-byte loads
                    const float4 d4 = *reinterpret_cast<const float4*>(Dr + rd * 16 + q);
                    // packed fp32x2 arithmetic: one instruction per pair of columns
                    const float2 x01 = __ffma2_rn(make_float2(__uint_as_float(sv[q]), __uint_as_float(sv[q + 1])), c2, make_float2(l4.x, l4.y));
                    const float2 x23 = __ffma2_rn(make_float2(__uint_as_float(sv[q + 2]), __uint_as_float(sv[q + 3])), c2, make_float2(l4.z, l4.w));
                    const float2 p01 = make_float2(fast_exp2(x01.x), fast_exp2(x01.y));
                    const float2 p23 = make_float2(fast_exp2(x23.x), fast_exp2(x23.y));
                    const float2 g01 = __fadd2_rn(make_float2(__uint_as_float(dp[q]), __uint_as_float(dp[q + 1])), make_float2(d4.x, d4.y));
                    const float2 g23 = __fadd2_rn(make_float2(__uint_as_float(dp[q + 2]), __uint_as_float(dp[q + 3])), make_float2(d4.z, d4.w));
                    const float2 s01 = __fmul2_rn(p01, g01), s23 = __fmul2_rn(p23, g23);
                    wp[q >> 1] = pack_bf16(p01.x, p01.y);
                    wp[(q >> 1) + 1] = pack_bf16(p23.x, p23.y);
                    wd[q >> 1] = pack_bf16(s01.x, s01.y);
                    wd[(q >> 1) + 1] = pack_bf16(s23.x, s23.y);
                }
                // in place: the packed columns of round rd lie inside the columns this thread has already read
                // (its own 32-column half, columns 8 rd .. 8 rd + 7 of it)
                tmem_st8(tS + rd * 8, wp);
                tmem_st8(tdP + rd * 8, wd);
                // dS^T also into the shared-memory tile of the sub-tile: row = key, 16-byte chunk index XOR (row & 7)
#pragma unroll
                for (int k4 = 0; k4 < 2; k4++) {
                    const int chunk = hc * 4 + rd * 2 + k4;
                    *reinterpret_cast<uint4*>(ds_row + ((chunk ^ (r & 7)) << 4)) =
                        make_uint4(wd[k4 * 4], wd[k4 * 4 + 1], wd[k4 * 4 + 2], wd[k4 * 4 + 3]);
                }
            }
            const long long tc1 = PROF_T();
            PROF_ADD(1, tc1 - ta1);
            tmem_st_wait();
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(b_pds + 8 * e);
            PROF_ADD(5, PROF_T() - tc1);
            __syncwarp();                                    // the private statistics are rewritten at the top of the next iteration
            t_prev = PROF_T();
        }
        if (threadIdx.x == 0) PROF_FLUSH(0, 8);
        // dV (group 0) and dK (group 1): complete once the last sub-tile's dV and dK commits have fired.  Column half hc writes head
        // dimensions 16 hc .. 16 hc + 15 and their rotary partners 32 further on.
        if (ok && !mbar_wait_park(b_qe + 8 * ((n_sub - 1) % BWD_SLOTS), ((n_sub - 1) / BWD_SLOTS) & 1)) ok = false;
        if (ok) {
            tc_fence_after();
            const int t = j * AT + r;
            const uint32_t ta = (e ? t_dK : t_dV) + lane_base + hc * 16;
            const float f = e ? scale : 1.f;
            bf16* dst = (e ? dk : dv) + (((long long)b * T + t) * KV + g) * ADH + hc * 16;
            uint32_t v1[16], v2[16];
            tmem_ld16(ta, v1);
            tmem_ld16(ta + 32, v2);
            tmem_ld_wait();
            if (e && rope_cos) {
                // inverse rotary on dK (pairs are 32 columns apart): out1 = g1 c + g2 s, out2 = -g1 s + g2 c
                const float* cr = rope_cos + (long long)t * (ADH / 2) + hc * 16;
                const float* sr = rope_sin + (long long)t * (ADH / 2) + hc * 16;
#pragma unroll
                for (int q = 0; q < 16; q += 4) {
                    const float4 c4 = *reinterpret_cast<const float4*>(cr + q), s4 = *reinterpret_cast<const float4*>(sr + q);
                    const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                    for (int z = 0; z < 4; z++) {
                        const float g1 = __uint_as_float(v1[q + z]) * f, g2 = __uint_as_float(v2[q + z]) * f;
                        v1[q + z] = __float_as_uint(g1 * cc[z] + g2 * ss[z]);
                        v2[q + z] = __float_as_uint(g2 * cc[z] - g1 * ss[z]);
                    }
                }
            } else {
#pragma unroll
                for (int q = 0; q < 16; q++) {
                    v1[q] = __float_as_uint(__uint_as_float(v1[q]) * f);
                    v2[q] = __float_as_uint(__uint_as_float(v2[q]) * f);
                }
            }
#pragma unroll
            for (int q = 0; q < 16; q += 8) {
                uint4 pk;
                pk.x = pack_bf16(__uint_as_float(v1[q]), __uint_as_float(v1[q + 1]));
                pk.y = pack_bf16(__uint_as_float(v1[q + 2]), __uint_as_float(v1[q + 3]));
                pk.z = pack_bf16(__uint_as_float(v1[q + 4]), __uint_as_float(v1[q + 5]));
                pk.w = pack_bf16(__uint_as_float(v1[q + 6]), __uint_as_float(v1[q + 7]));
                *reinterpret_cast<uint4*>(dst + q) = pk;
                pk.x = pack_bf16(__uint_as_float(v2[q]), __uint_as_float(v2[q + 1]));
                pk.y = pack_bf16(__uint_as_float(v2[q + 2]), __uint_as_float(v2[q + 3]));
                pk.z = pack_bf16(__uint_as_float(v2[q + 4]), __uint_as_float(v2[q + 5]));
                pk.w = pack_bf16(__uint_as_float(v2[q + 6]), __uint_as_float(v2[q + 7]));
                *reinterpret_cast<uint4*>(dst + 32 + q) = pk;
            }
        } else if (!ok && lane == 0) {
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
// The same with the inverse rotary applied on the way (head_dim 64: pairs are 32 columns apart): a thread takes
// 8 columns of the first half of a row and their partners; rows = B*T*H, t = (row / H) % T.
__global__ void k_dq_convert_rope(const float* __restrict__ src, bf16* __restrict__ dst, const float* __restrict__ cs,
                                  const float* __restrict__ sn, long long rows, int T, int H) {
    const long long total = rows * 4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long row = i >> 2;
        const int jc = (int)(i & 3) * 8;
        const int t = (int)((row / H) % T);
        float g1[8], g2[8], c[8], s[8], o1[8], o2[8];
        Vec<float>::ld(src + row * ADH + jc, g1); Vec<float>::ld(src + row * ADH + jc + 4, g1 + 4);
        Vec<float>::ld(src + row * ADH + 32 + jc, g2); Vec<float>::ld(src + row * ADH + 32 + jc + 4, g2 + 4);
        Vec<float>::ld(cs + (long long)t * 32 + jc, c); Vec<float>::ld(cs + (long long)t * 32 + jc + 4, c + 4);
        Vec<float>::ld(sn + (long long)t * 32 + jc, s); Vec<float>::ld(sn + (long long)t * 32 + jc + 4, s + 4);
#pragma unroll
        for (int q = 0; q < 8; q++) { o1[q] = g1[q] * c[q] + g2[q] * s[q]; o2[q] = g2[q] * c[q] - g1[q] * s[q]; }
        Vec<bf16>::st(dst + row * ADH + jc, o1);
        Vec<bf16>::st(dst + row * ADH + 32 + jc, o2);
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
                   const AttnShape& s, const float* rope_cos, const float* rope_sin, int* status, cudaStream_t st) {
    if (s.DH == 128) {
        if (rope_cos) return -1;                 // the inverse rotary is fused for head_dim 64 only
        return ax_attn_bwd_tc128(q, k, v, o, dO, lse, Dscratch, g_dq_acc, dq, dk, dv, s, status, st);
    }
    if (!served(s) || !g_dq_acc || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(dO) ||
        !aligned16(dq) || !aligned16(dk) || !aligned16(dv) || !aligned16(g_dq_acc)) return -1;
    if (rope_cos && (!rope_sin || !aligned16(rope_cos) || !aligned16(rope_sin))) return -1;
    const size_t need = (size_t)s.B * s.T * s.H * ADH * 4;
    CUtensorMap tq, tk, tv, tdo, tdq;
    if (map_bthd(&tq, q, s.B, s.T, s.H, 64) || map_bthd(&tk, k, s.B, s.T, s.KV) || map_bthd(&tv, v, s.B, s.T, s.KV) ||
        map_bthd(&tdo, dO, s.B, s.T, s.H, 64) || map_dq_f32(&tdq, g_dq_acc, s.B, s.T, s.H)) return 2;
    cudaMemsetAsync(g_dq_acc, 0, need, st);
    const long long rows = (long long)s.B * s.T * s.H;
    k_attn_bwd_prep<<<ew_grid(rows * 8, 256), 256, 0, st>>>((const bf16*)o, (const bf16*)dO, Dscratch, s.B, s.T, s.H);
    dim3 grid((s.T / AT) * s.KV * s.B);
#ifdef AXENG_PROF       // instrumented builds: allocates, synchronises and prints per launch (AXENG_ATTN_PROF=1)
    static const bool want_prof = getenv("AXENG_ATTN_PROF") != nullptr;
    long long* prof = nullptr;
    const int nblk = (int)grid.x;
    if (want_prof && cudaMalloc(&prof, (size_t)nblk * 256) == cudaSuccess) cudaMemset(prof, 0, (size_t)nblk * 256); else prof = nullptr;
    cudaMemcpyToSymbol(g_bwd_prof, &prof, sizeof(prof));
#endif
    k_attn_bwd_tc<<<grid, BWD_THREADS, BwdSmem::TOTAL, st>>>(tq, tk, tv, tdo, tdq, lse, Dscratch, (bf16*)dk, (bf16*)dv,
                                                              s.T, s.H, s.KV, s.scale, rope_cos, rope_sin, status);
#ifdef AXENG_PROF
    if (prof) {
        std::vector<long long> h((size_t)nblk * 32);
        cudaStreamSynchronize(st);
        cudaMemcpy(h.data(), prof, (size_t)nblk * 256, cudaMemcpyDeviceToHost);
        cudaFree(prof);
        double sum[32] = {0};
        for (int i = 0; i < nblk; i++) for (int q = 0; q < 32; q++) sum[q] += (double)h[(size_t)i * 32 + q];
        const double nt = sum[15] / 2.0;       // 128-query tiles
        fprintf(stderr, "attn_bwd per 128-query tile (cycles): softmax w0 top %.0f wait %.0f compute %.0f (%.0f %.0f %.0f) store %.0f | "
                        "issuer A loop %.0f wait %.0f S+dP issue %.0f | issuer B wait %.0f dV/dK issue %.0f wait drain %.0f dQ issue %.0f | mover wait %.0f work %.0f | tiles %.0f\n",
                sum[6] / nt, sum[0] / nt, sum[1] / nt, sum[2] / nt, sum[3] / nt, sum[4] / nt, sum[5] / nt, sum[8] / nt, sum[9] / nt, sum[16] / nt,
                sum[20] / nt, sum[19] / nt, sum[21] / nt, sum[18] / nt, sum[12] / nt, sum[13] / nt, nt);
    }
#endif
    if (rope_cos) {
        k_dq_convert_rope<<<ew_grid(rows * 4, 256), 256, 0, st>>>(g_dq_acc, (bf16*)dq, rope_cos, rope_sin, rows, s.T, s.H);
    } else {
        const long long n8 = rows * ADH / 8;
        k_dq_convert<<<ew_grid(n8, 256), 256, 0, st>>>(g_dq_acc, (bf16*)dq, n8);
    }
    return 0;
}
