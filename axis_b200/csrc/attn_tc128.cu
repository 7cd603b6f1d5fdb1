// Causal grouped-query flash attention on tcgen05 + TMEM for head_dim 128 (bf16, [B,T,H,DH] layout,
// T a multiple of 128).  Same algorithm and conventions as the head_dim-64 kernels; what changes is
// the budget: a 128-wide head doubles every operand tile (two 128-byte swizzle blocks along the head
// dimension) and every dV/dK/O accumulator (128 TMEM columns).
//
// Forward: one CTA per (128 queries, head), two CTAs per SM (96 KB each: Q, one K tile, one V tile).
//   K and V have their own barriers: K(j+1) is fetched as soon as S(j) = Q K^T has run, V(j+1) as soon
//   as P V(j) has run, so each load overlaps the other half of the iteration.
// Backward: one CTA per (128 keys, kv head); K/V resident; query sub-tiles of 64 so that everything fits
//   the 512 TMEM columns: S^T 64, dP^T 64, dV 128, dK 128, and dQ^T twice 64.  dQ is accumulated
//   transposed, dQ^T (head dim x queries) = K^T dS^T, which keeps M = 128 for that MMA; the drain writes
//   it back through a transposing, swizzled fp32 staging tile and adds it to the fp32 dq buffer with TMA
//   reduce-add.  Softmax and MMAs alternate per sub-tile (one S^T/dP^T buffer), eight softmax warps.
// Every mbarrier wait is bounded; on a timeout the kernel records a status code, unwinds and frees TMEM.
#include <cuda_bf16.h>

#include "attn_common.cuh"
#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

#define AT 128                 // keys per tile; queries per forward tile
#define DH2 128                // head dim served here
#define ATT_THREADS 160        // 4 softmax warps + 1 control warp
#define STAT_FWD128 0x500
#define STAT_BWD128 0x600

// ════════════════════════════════ forward ═══════════════════════════════════
struct Fwd128Smem {
    static constexpr int Q = 0, K = 32768, V = 65536, BARS = 98304, TOTAL = BARS + 128 + 1024;
};

// Issue forms for a converged warp (every lane runs the surrounding code, the elected lane issues): a lone thread in a
// divergent branch needs 45-50 cycles per MMA issue, this form 33 (measured on B200).
__device__ __forceinline__ void mma128_ts_e(uint32_t d, uint32_t a, uint64_t bd, uint32_t id, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p, q;\n\telect.sync _|q, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d), "r"(a), "l"(bd), "r"(id), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma128_ss_e(uint32_t d, uint64_t ad, uint64_t bd, uint32_t id, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p, q;\n\telect.sync _|q, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d), "l"(ad), "l"(bd), "r"(id), "r"(acc) : "memory");
}
__device__ __forceinline__ void commit128_e(uint32_t bar) {
    asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
                 "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(ATT_THREADS, 2)
k_attn_fwd_tc128(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, bf16* __restrict__ o, float* __restrict__ lse,
                 int T, int H, int KV, float scale, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sb = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Fwd128Smem::BARS);
    // q_full, k_full, v_full, s_full, p_full, o_full, v_empty
    const uint32_t b_q = smem_u32(bars), b_kf = b_q + 8, b_vf = b_kf + 8, b_s = b_vf + 8, b_p = b_s + 8, b_o = b_p + 8, b_ve = b_o + 8;
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
        mbar_init(b_q, 1); mbar_init(b_kf, 1); mbar_init(b_vf, 1); mbar_init(b_s, 1);
        mbar_init(b_p, 128); mbar_init(b_o, 1); mbar_init(b_ve, 1);
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
        {   // the whole warp runs the loop converged; lane 0 issues the TMA loads, one elected lane the MMAs
            bool ok = true;
            constexpr uint32_t id_s = tc_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t id_pv = tc_idesc_bf16(128, 128, 0, 1);
            // K-major tiles: two 64-wide blocks 16 KB apart, 2 units (32 B) per k-step inside a block;
            // V as the MN-major B operand: head-dim blocks 16 KB apart (LBO), 128 units (2 KB) per 16 keys
            const uint32_t loQ = desc_lo(sb + Fwd128Smem::Q, 16), loK = desc_lo(sb + Fwd128Smem::K, 16), loV = desc_lo(sb + Fwd128Smem::V, 16384);
            if (lane == 0) { tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); }
            auto load_tile = [&](uint32_t dst, const CUtensorMap* m, uint32_t bar, int heads_idx, int row0) {
                if (lane == 0) {
                    mbar_expect_tx(bar, 32768);
                    tma_load_4d(dst, m, bar, 0, heads_idx, row0, b);
                    tma_load_4d(dst + 16384, m, bar, 64, heads_idx, row0, b);
                }
                __syncwarp();
            };
            load_tile(sb + Fwd128Smem::Q, &tmQ, b_q, h, qt * AT);
            load_tile(sb + Fwd128Smem::K, &tmK, b_kf, g, 0);
            load_tile(sb + Fwd128Smem::V, &tmV, b_vf, g, 0);
            if (!mbar_wait(b_q, 0)) ok = false;
            for (int j = 0; j < nkt && ok; j++) {
                const uint32_t ph = j & 1;
                if (!mbar_wait(b_kf, ph)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < DH2 / 16; kk++)
                    mma128_ss_e(t_S, desc_of(loQ + (kk >> 2) * 1024 + (kk & 3) * 2), desc_of(loK + (kk >> 2) * 1024 + (kk & 3) * 2), id_s, kk != 0);
                commit128_e(b_s);
                if (j + 1 < nkt) {          // K is free once S(j) has run
                    if (!mbar_wait(b_s, ph)) { ok = false; break; }
                    load_tile(sb + Fwd128Smem::K, &tmK, b_kf, g, (j + 1) * AT);
                }
                if (!mbar_wait(b_p, ph) || !mbar_wait(b_vf, ph)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < AT / 16; kk++)
                    mma128_ts_e(t_O, t_S + kk * 8, desc_of(loV + kk * 128), id_pv, (j | kk) != 0);
                commit128_e(b_ve);
                commit128_e(b_o);
                if (j + 1 < nkt) {          // V is free once P V(j) has run
                    if (!mbar_wait(b_ve, ph)) { ok = false; break; }
                    load_tile(sb + Fwd128Smem::V, &tmV, b_vf, g, (j + 1) * AT);
                }
            }
            __syncwarp();
            if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, STAT_FWD128 | 1); }
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
                    for (int ch = 0; ch < DH2 / 32; ch++) {
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
            bf16* orow = o + (((long long)b * T + t) * H + h) * DH2;
#pragma unroll 1
            for (int ch = 0; ch < DH2 / 32; ch++) {
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
            atomicExch(status, STAT_FWD128 | 2);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, 256); }
}

// ════════════════════════════════ backward ══════════════════════════════════
// D[b,h,t] = sum_d dO*O on the [B,T,H,128] layout, written as [B,H,T]: sixteen lanes share a row.
__global__ void k_attn_bwd_prep128(const bf16* __restrict__ o, const bf16* __restrict__ dO, float* __restrict__ Dv,
                                   int B, int T, int H) {
    const long long nvec = (long long)B * T * H * (DH2 / 8);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec + 15; i += stride) {
        float a[8], g[8], acc = 0.f;
        if (i < nvec) {
            Vec<bf16>::ld(o + i * 8, a);
            Vec<bf16>::ld(dO + i * 8, g);
#pragma unroll
            for (int q = 0; q < 8; q++) acc += a[q] * g[q];
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 8);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        if ((i & 15) == 0 && i < nvec) {
            const long long row = i >> 4;
            const int hh = (int)(row % H);
            const long long bt = row / H;
            const int t = (int)(bt % T), bb = (int)(bt / T);
            Dv[((long long)bb * H + hh) * T + t] = acc;
        }
    }
}

#define BWD128_THREADS 288     // 8 softmax warps (two per TMEM lane quadrant) + 1 control warp
#define QS 64                  // queries per sub-tile
#define QST 3                  // Q/dO ring stages
struct Bwd128Smem {
    // K, V: 128 keys x 128 (two blocks of 16 KB); Q/dO sub-tiles: 64 x 128 (two blocks of 8 KB), three stages;
    // dS^T: 128 keys x 64 queries bf16, two buffers; dQ staging: 64 queries x 128 fp32 (four blocks of 8 KB);
    // row statistics of a sub-tile (64 lse, 64 D) beside its Q/dO stage
    static constexpr int K = 0, V = 32768, Q0 = 65536, DO0 = Q0 + QST * 16384, DS = DO0 + QST * 16384, DQ = DS + 2 * 16384,
                         STAT = DQ + 32768, BARS = STAT + QST * 512, TOTAL = BARS + 256 + 1024;
};
static_assert(Bwd128Smem::TOTAL <= 227 * 1024, "head_dim-128 backward shared memory exceeds the per-CTA limit");

// One CTA per (128 keys, head) walks the query sub-tiles (64 queries) of the causal range.  Per sub-tile:
//   S^T = K Q^T, dP^T = V dO^T   16 MMAs into TMEM (lanes = keys)
//   softmax warps                 read their 32 + 32 values in one TMEM round trip and release the two accumulators at
//                                 once, so S^T / dP^T of the next sub-tile are computed under this one's arithmetic;
//                                 P^T and dS^T go to TMEM columns of their own (packed bf16) and dS^T to shared memory
//   dV += P^T dO, dK += dS^T Q    A operands from TMEM;  dQ^T = K^T dS^T with dS^T from shared memory (two buffers)
// The control warp issues S^T / dP^T of sub-tile i first and then dV, dK, dQ^T of sub-tile i-1, so the tensor pipe
// always has the independent half of the work queued.  TMEM (512 columns): S^T 64, dP^T 64, dV 128, dK 128, dQ^T 64,
// P^T 32, dS^T 32.  dQ^T is single: the softmax warps move it out (transposing staging + TMA reduce-add) right after
// they have handed over P^T / dS^T of the following sub-tile.
__global__ void __launch_bounds__(BWD128_THREADS, 1)
k_attn_bwd_tc128(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                 const __grid_constant__ CUtensorMap tmdQ, const float* __restrict__ lse, const float* __restrict__ Dv,
                 bf16* __restrict__ dk, bf16* __restrict__ dv, int T, int H, int KV, float scale, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sb = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Bwd128Smem::BARS);
    // kv_full, q_full[3], q_empty[3], sdp_full, sdp_free, pds_full, dq_full, dq_empty
    const uint32_t b_kv = smem_u32(bars), b_qf = b_kv + 8, b_qe = b_qf + 8 * QST, b_sdp = b_qe + 8 * QST, b_sfree = b_sdp + 8,
                   b_pds = b_sfree + 8, b_dq = b_pds + 8, b_dqe = b_dq + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_stat = reinterpret_cast<float*>(smem + Bwd128Smem::STAT);   // [stage][lse 64 | D 64]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // 1-D grid ordered by decreasing work: key tile 0 of all (kv head, batch) pairs first
    const int rep = H / KV, nkt = T / AT;
    const int ngb = gridDim.x / nkt;
    const int j = blockIdx.x / ngb, gb = blockIdx.x % ngb;
    const int g = gb % KV, b = gb / KV;
    const int per_head = 2 * (nkt - j);                               // causal: query sub-tiles 2j .. 2 nkt - 1
    const int n_it = rep * per_head;

    if (threadIdx.x == 0) {
        mbar_init(b_kv, 1);
        for (int s = 0; s < QST; s++) { mbar_init(b_qf + 8 * s, 1); mbar_init(b_qe + 8 * s, 1); }
        mbar_init(b_sdp, 1); mbar_init(b_sfree, 256); mbar_init(b_pds, 256); mbar_init(b_dq, 1); mbar_init(b_dqe, 256);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 8) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // columns: S^T 0..63, dP^T 64..127, dV 128..255, dK 256..383, dQ^T 384..447, P^T 448..479, dS^T 480..511 (packed bf16)
    const uint32_t t_S = tmem, t_dP = tmem + 64, t_dV = tmem + 128, t_dK = tmem + 256, t_dQ = tmem + 384, t_P = tmem + 448,
                   t_dS = tmem + 480;

    if (warp == 8) {
        {   // the whole warp runs the loop converged; lane 0 issues the TMA loads, one elected lane the MMAs
            bool ok = true;
            constexpr uint32_t id_s = tc_idesc_bf16(128, QS, 0, 0);        // S^T = K Q^T, dP^T = V dO^T (64 queries)
            constexpr uint32_t id_acc = tc_idesc_bf16(128, DH2, 0, 1);     // dV/dK: A in TMEM, B N-major (128 wide)
            constexpr uint32_t id_dq = tc_idesc_bf16(128, QS, 1, 1);       // dQ^T = K^T dS^T: A = K M-major, B = dS^T N-major
            const uint32_t loK_k = desc_lo(sb + Bwd128Smem::K, 16), loV_k = desc_lo(sb + Bwd128Smem::V, 16);
            const uint32_t loK_m = desc_lo(sb + Bwd128Smem::K, 16384), loDS = desc_lo(sb + Bwd128Smem::DS, 16);
            const uint32_t loQ_k = desc_lo(sb + Bwd128Smem::Q0, 16), loQ_n = desc_lo(sb + Bwd128Smem::Q0, 8192);
            const uint32_t loO_k = desc_lo(sb + Bwd128Smem::DO0, 16), loO_n = desc_lo(sb + Bwd128Smem::DO0, 8192);
            if (lane == 0) {
                tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
                mbar_expect_tx(b_kv, 65536);
                tma_load_4d(sb + Bwd128Smem::K, &tmK, b_kv, 0, g, j * AT, b);
                tma_load_4d(sb + Bwd128Smem::K + 16384, &tmK, b_kv, 64, g, j * AT, b);
                tma_load_4d(sb + Bwd128Smem::V, &tmV, b_kv, 0, g, j * AT, b);
                tma_load_4d(sb + Bwd128Smem::V + 16384, &tmV, b_kv, 64, g, j * AT, b);
            }
            auto load_q = [&](int it) {
                if (lane != 0) return;
                const int s = it % QST, hh = it / per_head, u = 2 * j + it % per_head, h = g * rep + hh;
                mbar_expect_tx(b_qf + 8 * s, 32768 + 512);
                // the sub-tile's row statistics ride on the same barrier (a softmax warp that loaded them from global
                // memory itself would expose that latency at its next scoreboard wait)
                const long long sidx = ((long long)b * H + h) * T + u * QS;
                bulk_load_1d(sb + Bwd128Smem::STAT + s * 512, lse + sidx, 256, b_qf + 8 * s);
                bulk_load_1d(sb + Bwd128Smem::STAT + s * 512 + 256, Dv + sidx, 256, b_qf + 8 * s);
                tma_load_4d(sb + Bwd128Smem::Q0 + s * 16384, &tmQ, b_qf + 8 * s, 0, h, u * QS, b);
                tma_load_4d(sb + Bwd128Smem::Q0 + s * 16384 + 8192, &tmQ, b_qf + 8 * s, 64, h, u * QS, b);
                tma_load_4d(sb + Bwd128Smem::DO0 + s * 16384, &tmdO, b_qf + 8 * s, 0, h, u * QS, b);
                tma_load_4d(sb + Bwd128Smem::DO0 + s * 16384 + 8192, &tmdO, b_qf + 8 * s, 64, h, u * QS, b);
            };
            load_q(0);
            __syncwarp();
            if (!mbar_wait(b_kv, 0)) ok = false;
            // iteration it: S^T / dP^T of sub-tile it, then dV, dK and dQ^T of sub-tile it - 1 (one more round at the end)
            for (int it = 0; it <= n_it && ok; it++) {
                if (it + 1 < n_it) {        // prefetch sub-tile it+1: its stage was last read by dV / dK of sub-tile it-2
                    if (it >= 2 && !mbar_wait(b_qe + 8 * ((it - 2) % QST), ((it - 2) / QST) & 1)) { ok = false; break; }
                    load_q(it + 1);
                    __syncwarp();
                }
                if (it < n_it) {
                    const uint32_t so = (uint32_t)(it % QST) * 1024;     // stage offset (16 KB) in 16-byte units
                    if (!mbar_wait(b_qf + 8 * (it % QST), (it / QST) & 1) || *abort_flag) { ok = false; break; }
                    // every softmax thread holds S^T / dP^T of sub-tile it-1 in registers
                    if (it >= 1 && !mbar_wait(b_sfree, (it - 1) & 1)) { ok = false; break; }
                    tc_fence_after();
                    // S^T (128 keys x 64 queries) = K Q^T and dP^T = V dO^T over the 128-wide head: 8 k-steps each
#pragma unroll
                    for (int kk = 0; kk < DH2 / 16; kk++)
                        mma128_ss_e(t_S, desc_of(loK_k + (kk >> 2) * 1024 + (kk & 3) * 2), desc_of(loQ_k + so + (kk >> 2) * 512 + (kk & 3) * 2), id_s, kk != 0);
#pragma unroll
                    for (int kk = 0; kk < DH2 / 16; kk++)
                        mma128_ss_e(t_dP, desc_of(loV_k + (kk >> 2) * 1024 + (kk & 3) * 2), desc_of(loO_k + so + (kk >> 2) * 512 + (kk & 3) * 2), id_s, kk != 0);
                    commit128_e(b_sdp);
                }
                if (it >= 1) {
                    const int p = it - 1;                                  // the sub-tile whose P^T / dS^T are due
                    const uint32_t so = (uint32_t)(p % QST) * 1024;
                    if (!mbar_wait(b_pds, p & 1) || *abort_flag) { ok = false; break; }
                    tc_fence_after();
                    // P^T / dS^T: 64 queries packed in 32 columns, 16 queries (8 columns) per k-step
#pragma unroll
                    for (int kk = 0; kk < QS / 16; kk++)       // dV += P^T dO   (k = queries; B = dO sub-tile, head-dim blocks 8 KB apart)
                        mma128_ts_e(t_dV, t_P + kk * 8, desc_of(loO_n + so + kk * 128), id_acc, (p | kk) != 0);
#pragma unroll
                    for (int kk = 0; kk < QS / 16; kk++)       // dK += dS^T Q
                        mma128_ts_e(t_dK, t_dS + kk * 8, desc_of(loQ_n + so + kk * 128), id_acc, (p | kk) != 0);
                    commit128_e(b_qe + 8 * (p % QST));          // the Q/dO stage and the P^T / dS^T columns are free once these have run
                    // the single dQ^T accumulator: sub-tile p-1 has been moved out
                    if (p >= 1 && !mbar_wait(b_dqe, (p - 1) & 1)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < AT / 16; kk++)       // dQ^T = K^T dS^T   (k = keys), dS^T from its shared-memory buffer
                        mma128_ss_e(t_dQ, desc_of(loK_m + kk * 128), desc_of(loDS + (p & 1) * 1024 + kk * 128), id_dq, kk != 0);
                    commit128_e(b_dq);
                }
            }
            __syncwarp();
            if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, STAT_BWD128 | 1); }
        }
    } else {
        const int r = threadIdx.x & 127;                    // key row of S^T / head-dim row of dQ^T == TMEM lane
        const int hf = threadIdx.x >> 7;                    // which 32 query columns this thread handles
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const float c = scale * LOG2E;
        bool ok = true;
        // drain of dQ^T(t): TMEM (lanes = head dim, columns = queries) -> transposed, swizzled fp32 staging
        // (rows = queries, four 32-float blocks) -> TMA reduce-add into the fp32 dq buffer
        auto drain = [&](int t) -> bool {
            if (!mbar_wait(b_dq, t & 1) || *abort_flag) return false;
            tc_fence_after();
            if (threadIdx.x == 0) bulk_wait_read0();         // the previous reduce has finished reading the staging
            named_bar_sync(1, 256);
            uint32_t v[32];
            tmem_ld32(t_dQ + lane_base + hf * 32, v);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(b_dqe);                              // the accumulator may be overwritten by the next dQ^T
            // element (query q, head-dim r): block r/32, row q (128 B), 16-byte chunk ((r%32)/4) ^ (q & 7)
            uint8_t* col = smem + Bwd128Smem::DQ + (r >> 5) * 8192 + (r & 3) * 4;
            const int ch = (r & 31) >> 2;
#pragma unroll
            for (int q = 0; q < 32; q++) {
                const int qq = hf * 32 + q;
                *reinterpret_cast<float*>(col + qq * 128 + ((ch ^ (qq & 7)) << 4)) = __uint_as_float(v[q]) * scale;
            }
            fence_async_smem();
            named_bar_sync(1, 256);
            if (threadIdx.x == 0) {
                const int hh = t / per_head, u = 2 * j + t % per_head, h = g * rep + hh;
#pragma unroll
                for (int blk = 0; blk < 4; blk++)
                    tma_reduce_add_4d(&tmdQ, sb + Bwd128Smem::DQ + blk * 8192, blk * 32, h, u * QS, b);
                bulk_commit();
            }
            return true;
        };
        const float c_l = -LOG2E;
        for (int it = 0; it < n_it && ok; it++) {
            const int u = 2 * j + it % per_head;              // query sub-tile
            if (!mbar_wait(b_sdp, it & 1) || *abort_flag) { ok = false; break; }
            // the stage's barrier completed before S^T was issued; observing it makes the bulk-copied statistics visible
            if (!mbar_wait(b_qf + 8 * (it % QST), (it / QST) & 1)) { ok = false; break; }
            tc_fence_after();
            const bool diag = u < 2 * j + 2;                  // sub-tiles that straddle this key tile's diagonal
            const int qoff = u * QS - j * AT;                 // query index of column 0 relative to key row 0
            const float* L = s_stat + (it % QST) * 128;
            const float* Dr = L + 64;
            uint8_t* ds_row = smem + Bwd128Smem::DS + (it & 1) * 16384 + r * 128;
            {
                uint32_t sv[32], dp[32], wp[16], wd[16];
                tmem_ld32(t_S + lane_base + hf * 32, sv);
                tmem_ld32(t_dP + lane_base + hf * 32, dp);
                tmem_ld_wait();
                tc_fence_before();
                mbar_arrive(b_sfree);                            // the two accumulators are free for the next sub-tile
                if (diag) {                                      // query < key: masked (score -> -inf, so P = dS = 0)
#pragma unroll
                    for (int q = 0; q < 32; q++)
                        if (qoff + hf * 32 + q < r) sv[q] = 0xff800000u;
                }
#pragma unroll
                for (int q = 0; q < 32; q += 4) {
                    const int cs = hf * 32 + q;                  // query column within the sub-tile
                    const float4 l4 = *reinterpret_cast<const float4*>(L + cs);       // broadcast 16-byte loads
                    const float4 d4 = *reinterpret_cast<const float4*>(Dr + cs);
                    float p0 = fast_exp2(fmaf(__uint_as_float(sv[q]), c, l4.x * c_l));
                    float p1 = fast_exp2(fmaf(__uint_as_float(sv[q + 1]), c, l4.y * c_l));
                    float p2 = fast_exp2(fmaf(__uint_as_float(sv[q + 2]), c, l4.z * c_l));
                    float p3 = fast_exp2(fmaf(__uint_as_float(sv[q + 3]), c, l4.w * c_l));
                    wp[q >> 1] = pack_bf16(p0, p1);
                    wp[(q >> 1) + 1] = pack_bf16(p2, p3);
                    wd[q >> 1] = pack_bf16(p0 * (__uint_as_float(dp[q]) - d4.x), p1 * (__uint_as_float(dp[q + 1]) - d4.y));
                    wd[(q >> 1) + 1] = pack_bf16(p2 * (__uint_as_float(dp[q + 2]) - d4.z), p3 * (__uint_as_float(dp[q + 3]) - d4.w));
                }
                // P^T / dS^T columns were last read by dV / dK of the previous sub-tile (issued a whole pass of arithmetic
                // ago); the shared-memory dS^T buffer of this parity by dQ^T of sub-tile it-2, whose completion these
                // threads observed when they moved it out
                if (it >= 1 && !mbar_wait(b_qe + 8 * ((it - 1) % QST), ((it - 1) / QST) & 1)) { ok = false; break; }
                tc_fence_after();
                tmem_st16(t_P + lane_base + hf * 16, wp);
                tmem_st16(t_dS + lane_base + hf * 16, wd);
                // dS^T also to shared memory (B operand of dQ^T): row = key, 16-byte chunk index XOR (row & 7)
#pragma unroll
                for (int k4 = 0; k4 < 4; k4++) {
                    const int chunk = hf * 4 + k4;
                    uint4 pk = make_uint4(wd[k4 * 4], wd[k4 * 4 + 1], wd[k4 * 4 + 2], wd[k4 * 4 + 3]);
                    *reinterpret_cast<uint4*>(ds_row + ((chunk ^ (r & 7)) << 4)) = pk;
                }
            }
            tmem_st_wait();
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(b_pds);
            // dQ^T of the previous sub-tile: its MMA was issued right after that sub-tile's P^T / dS^T were handed over
            if (it >= 1 && !drain(it - 1)) { ok = false; break; }
        }
        if (ok && !drain(n_it - 1)) ok = false;
        if (threadIdx.x == 0) bulk_wait0();
        if (ok) {
            // dV (half 0 threads) and dK (half 1 threads): complete once the last commit has fired — waited in drain
            const int t = j * AT + r;
            const uint32_t ta = hf ? t_dK : t_dV;
            const float f = hf ? scale : 1.f;
            bf16* dst = (hf ? dk : dv) + (((long long)b * T + t) * KV + g) * DH2;
#pragma unroll 1
            for (int ch = 0; ch < DH2 / 32; ch++) {
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
            atomicExch(status, STAT_BWD128 | 2);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// fp32 dq accumulator -> bf16 dq (same [B,T,H,DH] layout)
__global__ void k_dq_convert128(const float* __restrict__ src, bf16* __restrict__ dst, long long n8) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        float f[8];
        Vec<float>::ld(src + i * 8, f);
        Vec<float>::ld(src + i * 8 + 4, f + 4);
        Vec<bf16>::st(dst + i * 8, f);
    }
}

// ── host ────────────────────────────────────────────────────────────────────
int ax_attn_tc128_init(void) {
    int rc = 0;
    rc |= (int)cudaFuncSetAttribute(k_attn_fwd_tc128, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd128Smem::TOTAL);
    rc |= (int)cudaFuncSetAttribute(k_attn_bwd_tc128, cudaFuncAttributeMaxDynamicSharedMemorySize, Bwd128Smem::TOTAL);
    return rc;
}

static bool served128(const AttnShape& s) {
    // [B,T,H,DH] layout, head_dim 128, whole tiles
    return s.DH == DH2 && s.T % AT == 0 && s.T >= AT && s.qh == DH2 && s.kh == DH2 &&
           s.qt == (long long)s.H * DH2 && s.kt == (long long)s.KV * DH2 && s.H % s.KV == 0;
}
// [B,T,heads,128] bf16; a box is 64 head-dim elements (one 128-byte swizzle block) x `rows` tokens
static int map_bthd128(CUtensorMap* m, const void* base, int B, int T, int heads, int rows) {
    uint64_t dims[4] = {DH2, (uint64_t)heads, (uint64_t)T, (uint64_t)B};
    uint64_t strides[3] = {(uint64_t)DH2 * 2, (uint64_t)heads * DH2 * 2, (uint64_t)T * heads * DH2 * 2};
    uint32_t box[4] = {64, 1, (uint32_t)rows, 1};
    return tc_make_tmap_bf16(m, base, 4, dims, strides, box, true);
}
static int map_dq_f32_128(CUtensorMap* m, const void* base, int B, int T, int heads) {
    PFN_tmapEncodeTiled enc = tc_encode_fn();
    if (!enc) return 1;
    cuuint64_t gd[4] = {DH2, (cuuint64_t)heads, (cuuint64_t)T, (cuuint64_t)B};
    cuuint64_t gs[3] = {(cuuint64_t)DH2 * 4, (cuuint64_t)heads * DH2 * 4, (cuuint64_t)T * heads * DH2 * 4};
    cuuint32_t bx[4] = {32, 1, QS, 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 2;
}

int ax_attn_fwd_tc128(const void* q, const void* k, const void* v, void* o, float* lse,
                      const AttnShape& s, int* status, cudaStream_t st) {
    if (!served128(s) || !lse || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return -1;
    CUtensorMap tq, tk, tv;
    if (map_bthd128(&tq, q, s.B, s.T, s.H, AT) || map_bthd128(&tk, k, s.B, s.T, s.KV, AT) || map_bthd128(&tv, v, s.B, s.T, s.KV, AT)) return 2;
    dim3 grid((s.T / AT) * s.H * s.B);
    k_attn_fwd_tc128<<<grid, ATT_THREADS, Fwd128Smem::TOTAL, st>>>(tq, tk, tv, (bf16*)o, lse, s.T, s.H, s.KV, s.scale, status);
    return 0;
}

int ax_attn_bwd_tc128(const void* q, const void* k, const void* v, const void* o, const void* dO,
                      const float* lse, float* Dscratch, float* g_dq_acc, void* dq, void* dk, void* dv,
                      const AttnShape& s, int* status, cudaStream_t st) {
    if (!served128(s) || !g_dq_acc || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(dO) ||
        !aligned16(dq) || !aligned16(dk) || !aligned16(dv) || !aligned16(g_dq_acc)) return -1;
    const size_t need = (size_t)s.B * s.T * s.H * DH2 * 4;
    CUtensorMap tq, tk, tv, tdo, tdq;
    if (map_bthd128(&tq, q, s.B, s.T, s.H, QS) || map_bthd128(&tk, k, s.B, s.T, s.KV, AT) || map_bthd128(&tv, v, s.B, s.T, s.KV, AT) ||
        map_bthd128(&tdo, dO, s.B, s.T, s.H, QS) || map_dq_f32_128(&tdq, g_dq_acc, s.B, s.T, s.H)) return 2;
    cudaMemsetAsync(g_dq_acc, 0, need, st);
    const long long rows = (long long)s.B * s.T * s.H;
    k_attn_bwd_prep128<<<ew_grid(rows * 16, 256), 256, 0, st>>>((const bf16*)o, (const bf16*)dO, Dscratch, s.B, s.T, s.H);
    dim3 grid((s.T / AT) * s.KV * s.B);
    k_attn_bwd_tc128<<<grid, BWD128_THREADS, Bwd128Smem::TOTAL, st>>>(tq, tk, tv, tdo, tdq, lse, Dscratch, (bf16*)dk, (bf16*)dv,
                                                                       s.T, s.H, s.KV, s.scale, status);
    const long long n8 = rows * DH2 / 8;
    k_dq_convert128<<<ew_grid(n8, 256), 256, 0, st>>>(g_dq_acc, (bf16*)dq, n8);
    return 0;
}
