// bf16 GEMM with paired CTAs (tcgen05 cta_group::2): a cluster of two CTAs on
// neighbouring SMs computes one 256 x 256 output tile.  Each CTA loads its own
// 128 rows of A and its own 128 columns of B (plain TMA tile loads — nothing is
// multicast; the pair shares B through the MMA unit, which reads both CTAs'
// shared memory), so a k-block costs 32 KB of L2->smem traffic per SM instead of
// the 48 KB of the single-CTA 128 x 256 tile, and half the smem operand reads
// per flop.  CTA 0 of the pair issues the MMAs (M = 256); accumulators live in
// both CTAs' TMEM (128 lanes x 256 columns each, double-buffered); completion is
// signalled to both CTAs with multicast commits; every CTA writes its own 128
// rows of C.
//
// Same operand layouts, epilogue and split-K scheme as the single-CTA kernel.
// All mbarrier waits are bounded.
#include <cuda_bf16.h>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "gemm_epi.cuh"
#include "kernels.h"
#include "tc_common.cuh"

#define BM2 128            // rows per CTA (256 per pair)
#define BN2 256            // columns per pair (128 loaded by each CTA)
#define BK2 64
#define STAGES2 6
#define THREADS2 192
#define STAT_GEMM2 0x400
#define A_BYTES2 (BM2 * BK2 * 2)
#define B_BYTES2 (128 * BK2 * 2)
#define STAGE_BYTES2 (A_BYTES2 + B_BYTES2)
#define STG_BYTES2 (4 * 2 * 4096)      // output staging: per epilogue warp two buffers of 32 rows x 128 B
#define SMEM2 (STAGES2 * STAGE_BYTES2 + STG_BYTES2 + 1024 + 512)

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tile store from this CTA's shared memory (3-D map: column, row, split); bulk-group completion
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void bulk_commit2() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_le2() { asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory"); }
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void bulk_wait_read_le1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
// tile load whose completion is counted on an mbarrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_mma_ss2(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same two for a converged warp: every lane executes the surrounding code (addresses and descriptor words stay
// warp-uniform and cheap to form), the elected lane issues.  A lone thread in a divergent branch needs about
// 45-50 cycles per MMA issue where this form needs 33 (measured on B200).
__device__ __forceinline__ void tc_mma_ss2_e(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\telect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit2_e(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
                 "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}"
                 ::"r"(bar), "h"(mask) : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair once all prior MMAs finish
__device__ __forceinline__ void tc_commit2(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}

// Grouped launch: several GEMMs of one layer run as one persistent kernel.
//   mode 1: `count` problems share A; problem g has its own B (n[g] columns) and its own C — their column
//           tiles form one tile space (q/k/v or gate/up projections of the same input; their weight gradients).
//           With xkb > 0 every problem has an extra K-segment of its own behind the shared one: C_g = A B_g + A'_g B'_g
//           (xkb k-blocks; a low-rank adapter's contribution inside its projection's launch).
//   mode 2: one output accumulates over `count` (up to 6) K-segments, each with its own A and B (kb[s] k-blocks):
//           dX = dY0 W0^T + dY1 W1^T + ... without round trips of the partial sums through memory; an addend
//           (residual) may be fetched by TMA as in the plain GEMM.
//   mode 3: `count` independent problems of the same depth k, each with its own A, B, C, m[g] and n[g] (weight
//           gradients of different projections of a layer): their tiles form one tile space, so the second
//           problem fills the wave the first one leaves half empty.
//   mode 4: SwiGLU pair — gate and up projections of one input with the activation fused: a 256-wide pair tile holds
//           128 gate columns (B from problem 0, loaded by CTA 0) and the same 128 up columns (problem 1, CTA 1), so an
//           epilogue thread has g and u of its row side by side and writes g, u and h = silu(g) * u (three outputs).
// Grouped launches write through TMA stores and do not split K; only mode 2 takes an addend.
struct GemmGroup {
    int mode, count;
    int n[3];
    int kb[6];
    int m[3];
    int xkb;
    // rotary embedding in the epilogue of a mode-1 launch with bf16 output: the outputs g whose bit is set in
    // rope_mask are [rows, heads * 64] projections (row = batch * rope_T + token); every 64-column piece of the
    // epilogue is one head, its columns i and i + 32 form a rotary pair (tables: fp32 [rope_T, 32])
    const float* rope_cos;
    const float* rope_sin;
    int rope_T, rope_mask;
};
static GemmGroup g_rope_req = {};        // rotary request for the next grouped launch (host side, one stream of launches)
void ax_gemm_group_rope(const float* cs, const float* sn, int T, int mask) {
    g_rope_req.rope_cos = cs; g_rope_req.rope_sin = sn; g_rope_req.rope_T = T; g_rope_req.rope_mask = mask;
}

template <int A_MN, int B_MN, typename TO>
__global__ void __launch_bounds__(THREADS2, 1)
k_gemm_tc2(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
           const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmD,
           const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmA2,
           const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmB2,
           const __grid_constant__ CUtensorMap tmC1, const __grid_constant__ CUtensorMap tmC2,
           const __grid_constant__ CUtensorMap tmEA0, const __grid_constant__ CUtensorMap tmEA1,
           const __grid_constant__ CUtensorMap tmEA2, const __grid_constant__ CUtensorMap tmEB0,
           const __grid_constant__ CUtensorMap tmEB1, const __grid_constant__ CUtensorMap tmEB2,
           const GemmGroup grp, int tma_out,
           TO* __restrict__ C, const TO* D, int m, int n, int k, float alpha, float beta, int* status,
           int ksplit, float* __restrict__ ws, long long* prof) {
    // tma_out != 0: the epilogue stages 32 x 128-byte pieces in shared memory (128-byte swizzle) and writes
    // them with TMA tile stores through tmC — {n, m, 1} over C, or {n, m, ksplit} over the fp32 split-K
    // workspace; the hardware clips pieces that overhang the matrix.  Otherwise threads store their rows.
    // tma_out == 2: the addend D is fetched the same way (TMA tile loads through tmD, two pieces ahead, into
    // the staging buffer where the result then replaces it); the operand ring then runs with five stages and
    // the sixth stage's memory doubles the staging area (four buffers per epilogue warp).
    // prof (only in builds with -DAXENG_PROF, otherwise null and every stamp compiles out): clock64 stamps of
    // pair 0's leader CTA — [0] entry, [1] set-up done, [2] predecessor grid finished, [3] first operands landed,
    // [4] last MMA issued, [5] last accumulator complete, [6] last tile stored, [7] exit
#ifdef AXENG_PROF
    const bool timing = prof != nullptr && blockIdx.x == 0;
#else
    constexpr bool timing = false;
#endif
    if (timing && threadIdx.x == 0) prof[0] = clock64();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES2 * STAGE_BYTES2 + STG_BYTES2);
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * STAGES2;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES2, bar_tempty = bar_tfull + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES2 + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t smem_base = smem_u32(smem);
    const bool swiglu = grp.mode == 4;
    const bool wide_stg = tma_out == 2 || swiglu;                  // four staging buffers per epilogue warp, five stages
    const int nst = wide_stg ? STAGES2 - 1 : STAGES2;              // operand stages in use
    const uint32_t bar_d = smem_u32(bars + 20);                    // [4 warps][4 buffers] addend-arrival barriers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                 // 0 = leader (issues the MMAs)
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int tiles_m = (m + 2 * BM2 - 1) / (2 * BM2);
    int tiles_n = (n + BN2 - 1) / BN2, kblocks_all = (k + BK2 - 1) / BK2;
    const int kb_main = kblocks_all;                       // mode 1: k-blocks of the shared segment
    if (grp.mode == 1) {
        tiles_n = 0;
        for (int q = 0; q < grp.count; q++) tiles_n += (grp.n[q] + BN2 - 1) / BN2;
        kblocks_all += grp.xkb;
    }
    if (grp.mode == 2) { kblocks_all = 0; for (int q = 0; q < grp.count; q++) kblocks_all += grp.kb[q]; }
    if (swiglu) tiles_n = (n + 127) / 128;
    int num_tiles = tiles_m * tiles_n;
    if (grp.mode == 3) {
        num_tiles = 0;
        for (int q = 0; q < grp.count; q++) num_tiles += ((grp.m[q] + 2 * BM2 - 1) / (2 * BM2)) * ((grp.n[q] + BN2 - 1) / BN2);
    }
    // tile index -> problem g, row tile tm and column tile tl inside it (row tiles fastest)
    auto locate = [&](int tile, int& tm, int& tl) -> int {
        int q = 0;
        if (grp.mode == 3) {
            int tmq = (grp.m[0] + 2 * BM2 - 1) / (2 * BM2);
            for (; q + 1 < grp.count; q++) {
                const int tq = tmq * ((grp.n[q] + BN2 - 1) / BN2);
                if (tile < tq) break;
                tile -= tq;
                tmq = (grp.m[q + 1] + 2 * BM2 - 1) / (2 * BM2);
            }
            tm = tile % tmq; tl = tile / tmq;
            return q;
        }
        tm = tile % tiles_m;
        int tn = tile / tiles_m;
        if (grp.mode == 1)
            for (; q + 1 < grp.count; q++) { const int tq = (grp.n[q] + BN2 - 1) / BN2; if (tn < tq) break; tn -= tq; }
        tl = tn;
        return q;
    };
    const int kb_per = (kblocks_all + ksplit - 1) / ksplit;
    const int num_units = num_tiles * ksplit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES2; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 256); }
        for (int a = 0; a < 16; a++) mbar_init(bar_d + 8 * a, 1);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (grp.count > 1) { tma_prefetch_desc(grp.mode == 2 ? &tmA1 : &tmC1); tma_prefetch_desc(&tmB1); }
        if (grp.count > 2) { tma_prefetch_desc(grp.mode == 2 ? &tmA2 : &tmC2); tma_prefetch_desc(&tmB2); }
        if (tma_out) tma_prefetch_desc(&tmC);
        if (tma_out == 2) tma_prefetch_desc(&tmD);
    }
    if (warp == 1) { tmem_alloc2(smem_u32(tmem_slot), 512); tmem_relinquish2(); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                   // peer barriers are initialised before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t full_leader = map_to_cta(bar_full, 0);  // cluster address of the leader's full[0]
    const uint32_t tempty_leader = map_to_cta(bar_tempty, 0);
    // programmatic dependent launch: see the single-CTA kernel
    if (timing && threadIdx.x == 0) prof[1] = clock64();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (timing && threadIdx.x == 0) prof[2] = clock64();

    if (warp == 0 && lane == 0) {
        // ── TMA producer (both CTAs): own 128 rows of A, own 128 columns of B ──
        uint32_t it = 0, ph = 0;
        int s = 0;
        bool ok = true;
        for (int unit = pair; unit < num_units && ok; unit += npairs) {
            const int tile = unit % num_tiles, split = unit / num_tiles;
            const int kb0 = split * kb_per, kb1 = min(kblocks_all, kb0 + kb_per);
            int tm, tl;
            const int g = locate(tile, tm, tl);
            const int row0 = tm * 2 * BM2 + rank * BM2, col0 = swiglu ? tl * 128 : tl * BN2 + rank * 128;
            // operand maps: modes 1 and 3 pick B by problem (mode 3 also A), mode 2 walks A and B through the K-segments,
            // mode 4 gives CTA 0 the gate weights and CTA 1 the up weights (same 128 columns)
            const CUtensorMap* pA = grp.mode == 3 ? (g == 0 ? &tmA : (g == 1 ? &tmA1 : &tmA2)) : &tmA;
            const CUtensorMap* pB = (grp.mode == 1 || grp.mode == 3) ? (g == 0 ? &tmB : (g == 1 ? &tmB1 : &tmB2))
                                    : (swiglu && rank == 1 ? &tmB1 : &tmB);
            int seg = 0, kl = kb0;                       // segment and k-block inside it
            if (grp.mode == 2) while (seg + 1 < grp.count && kl >= grp.kb[seg]) { kl -= grp.kb[seg]; seg++; }
            for (int kb = kb0; kb < kb1; kb++, kl++, it++, s = (s + 1 == nst ? 0 : s + 1), ph ^= (s == 0)) {
                if (grp.mode == 2) {
                    while (seg + 1 < grp.count && kl >= grp.kb[seg]) { kl = 0; seg++; }
                    pA = seg == 0 ? &tmA : seg == 1 ? &tmA1 : seg == 2 ? &tmA2 : seg == 3 ? &tmEA0 : seg == 4 ? &tmEA1 : &tmEA2;
                    pB = seg == 0 ? &tmB : seg == 1 ? &tmB1 : seg == 2 ? &tmB2 : seg == 3 ? &tmEB0 : seg == 4 ? &tmEB1 : &tmEB2;
                } else if (grp.mode == 1 && kb == kb_main) {         // the problem's own extra segment
                    kl = 0;
                    pA = g == 0 ? &tmEA0 : (g == 1 ? &tmEA1 : &tmEA2);
                    pB = g == 0 ? &tmEB0 : (g == 1 ? &tmEB1 : &tmEB2);
                }
                if (it >= (uint32_t)nst && !mbar_wait(bar_empty + 8 * s, ph ^ 1)) { ok = false; break; }
                if (*abort_flag) { ok = false; break; }
                const uint32_t sa = smem_base + s * STAGE_BYTES2, sb = sa + A_BYTES2;
                const uint32_t fb = full_leader + 8 * s;
                if (rank == 0) mbar_expect_tx(bar_full + 8 * s, 2 * STAGE_BYTES2);   // both CTAs' bytes land on this barrier
                if (A_MN) {
#pragma unroll
                    for (int b = 0; b < 2; b++) tma_load_2d_pair(sa + b * 8192, pA, fb, row0 + b * 64, kl * BK2);
                } else {
                    tma_load_2d_pair(sa, pA, fb, kl * BK2, row0);
                }
                if (B_MN) {
#pragma unroll
                    for (int b = 0; b < 2; b++) tma_load_2d_pair(sb + b * 8192, pB, fb, col0 + b * 64, kl * BK2);
                } else {
                    tma_load_2d_pair(sb, pB, fb, kl * BK2, col0);
                }
            }
        }
        if (!ok) { *abort_flag = 1; atomicExch(status, STAT_GEMM2 | 1); }
    } else if (warp == 1 && rank == 0) {
        // ── MMA issuer (leader CTA only): the whole warp runs the loop converged, one elected lane issues ──
        constexpr uint32_t idesc = tc_idesc_bf16(256, BN2, A_MN, B_MN);
        // descriptor words: the upper one is a constant (SBO 1024, 128-byte swizzle), the lower one is
        // (address >> 4) | (LBO >> 4) << 16; a k-step of 16 advances it by 2048 B (MN-major) or 32 B (K-major)
        constexpr uint32_t dhi = (1024u >> 4) | (1u << 14) | (2u << 29);
        constexpr uint32_t a_step = A_MN ? 128 : 2, b_step = B_MN ? 128 : 2;
        constexpr uint32_t a_lbo = (A_MN ? 8192u : 16u) >> 4, b_lbo = (B_MN ? 8192u : 16u) >> 4;
        uint32_t it = 0, tcount = 0, ph = 0;
        int s = 0;
        bool ok = true;
        for (int unit = pair; unit < num_units && ok; unit += npairs, tcount++) {
            const int split = unit / num_tiles;
            const int kb0 = split * kb_per, kb1 = min(kblocks_all, kb0 + kb_per);
            const int acc = tcount & 1;
            const uint32_t aph = (tcount >> 1) & 1;
            if (tcount >= 2 && !mbar_wait(bar_tempty + 8 * acc, aph ^ 1)) { ok = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN2;
            for (int kb = kb0; kb < kb1; kb++, it++, s = (s + 1 == nst ? 0 : s + 1), ph ^= (s == 0)) {
                if (!mbar_wait(bar_full + 8 * s, ph) || *abort_flag) { ok = false; break; }
                tc_fence_after();
                if (timing && it == 0 && lane == 0) prof[3] = clock64();
                const uint32_t sa = smem_base + s * STAGE_BYTES2, sb = sa + A_BYTES2;
                const uint32_t a_lo = ((sa & 0x3FFFF) >> 4) | (a_lbo << 16), b_lo = ((sb & 0x3FFFF) >> 4) | (b_lbo << 16);
#pragma unroll
                for (int kk = 0; kk < BK2 / 16; kk++)
                    tc_mma_ss2_e(d_tmem, ((uint64_t)dhi << 32) | (a_lo + kk * a_step), ((uint64_t)dhi << 32) | (b_lo + kk * b_step),
                                 idesc, (kb != kb0) || (kk != 0));
                tc_commit2_e(bar_empty + 8 * s);       // frees the stage in both CTAs
            }
            if (ok) tc_commit2_e(bar_tfull + 8 * acc); // accumulator ready in both CTAs
            if (timing && lane == 0) prof[4] = clock64();
        }
        __syncwarp();
        if (lane != 0) ok = true;                      // one report is enough
        if (!ok) { *abort_flag = 1; atomicExch(status, STAT_GEMM2 | 2); }
    } else if (warp >= 2) {
        // ── epilogue (both CTAs): own 128 rows x 256 columns ──
        const int quad = warp & 3;
        uint32_t tcount = 0, pieces = 0;
        bool ok = true;
        const bool vec_ok = (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (n % (16 / (int)sizeof(TO))) == 0 &&
                            (!D || (reinterpret_cast<uintptr_t>(D) & 15) == 0);
        const bool f32_out = ksplit > 1 || sizeof(TO) == 4;
        const float a_eff = ksplit > 1 ? 1.f : alpha;
        // staging: two 4 KB buffers per warp behind the operand ring; four when the addend is fetched by TMA
        // (the ring's last stage is then unused and adjoins the staging area)
        const int nbuf = wide_stg ? 4 : 2;
        const uint32_t stg_off = wide_stg ? (STAGES2 - 1) * STAGE_BYTES2 + quad * 16384 : STAGES2 * STAGE_BYTES2 + quad * 8192;
        uint8_t* stg = smem + stg_off;
        const uint32_t stg_u32 = smem_base + stg_off;
        const uint32_t my_bar_d = bar_d + 32 * quad;
        uint32_t dpar = 0;                                      // phase parity of each addend barrier
        for (int unit = pair; unit < num_units && ok; unit += npairs, tcount++) {
            const int tile = unit % num_tiles, split = unit / num_tiles;
            int tm, tl;
            const int g = locate(tile, tm, tl);                  // grouped launch: which output, which tile of it
            const int tn = tl;
            const int acc = tcount & 1;
            const uint32_t aph = (tcount >> 1) & 1;
            const int row0 = tm * 2 * BM2 + rank * BM2 + quad * 32;
            const int row = row0 + lane;
            const int cw = f32_out ? 32 : 64;                   // columns per 128-byte piece
            const CUtensorMap* pC = g == 0 ? &tmC : (g == 1 ? &tmC1 : &tmC2);
            const int ncols = min(BN2, ((grp.mode == 1 || grp.mode == 3) ? grp.n[g] : n) - tl * BN2);
            const int m_g = grp.mode == 3 ? grp.m[g] : m;
            const int npc = (tma_out && !swiglu && row0 < m_g) ? (ncols + cw - 1) / cw : 0;   // pieces this warp writes
            const uint32_t pbase = pieces;
            const bool do_rope = sizeof(TO) == 2 && grp.mode == 1 && ((grp.rope_mask >> g) & 1);
            const int rope_t = do_rope ? (row < m_g ? row : 0) % grp.rope_T : 0;
            auto fetch_d = [&](int j) {                          // lane 0: addend piece j of this tile -> its buffer
                const uint32_t bi = (pbase + j) & 3;
                mbar_expect_tx(my_bar_d + 8 * bi, 4096);
                tma_load_3d(stg_u32 + bi * 4096, &tmD, my_bar_d + 8 * bi, tn * BN2 + j * cw, row0, 0);
            };
            if (tma_out == 2 && lane == 0 && npc > 0) {          // the first two addend pieces travel during the main loop
                bulk_wait_read_le2();
                fetch_d(0);
                if (npc > 1) fetch_d(1);
            }
            if (!mbar_wait(bar_tfull + 8 * acc, aph) || *abort_flag) { ok = false; break; }
            tc_fence_after();
            if (timing && threadIdx.x == 64) prof[5] = clock64();
            const uint32_t taddr = tmem_base + acc * BN2 + ((uint32_t)(quad * 32) << 16);
            if (swiglu) {
                // accumulator columns 0..127: gate, 128..255: up (same output columns tl*128 ..); per 64-column piece
                // three staged outputs g, u, h, each stored by its own bulk group so that the buffers rotate freely
                const int vcols = min(128, n - tl * 128);
                const int np2 = row0 < m ? (vcols + 63) / 64 : 0;
#pragma unroll 1
                for (int j = 0; j < np2; j++) {
                    if (lane == 0) bulk_wait_read_le1();        // only the latest store may still be reading its buffer
                    __syncwarp();
                    uint8_t* bg = stg + ((pieces) & 3) * 4096 + lane * 128;
                    uint8_t* bu = stg + ((pieces + 1) & 3) * 4096 + lane * 128;
                    uint8_t* bh = stg + ((pieces + 2) & 3) * 4096 + lane * 128;
#pragma unroll 1
                    for (int half = 0; half < 2; half++) {
                        uint32_t rg[32], ru[32];
                        tmem_ld32(taddr + j * 64 + half * 32, rg);
                        tmem_ld32(taddr + 128 + j * 64 + half * 32, ru);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            float g8[8], u8[8], h8[8];
#pragma unroll
                            for (int e2 = 0; e2 < 8; e2++) {
                                g8[e2] = alpha * __uint_as_float(rg[q * 8 + e2]);
                                u8[e2] = alpha * __uint_as_float(ru[q * 8 + e2]);
                                h8[e2] = g8[e2] / (1.f + __expf(-g8[e2])) * u8[e2];
                            }
                            const int sw = ((half * 4 + q) ^ (lane & 7)) << 4;
                            uint4 pk;
                            pk.x = pack2_bf16(g8[0], g8[1]); pk.y = pack2_bf16(g8[2], g8[3]); pk.z = pack2_bf16(g8[4], g8[5]); pk.w = pack2_bf16(g8[6], g8[7]);
                            *reinterpret_cast<uint4*>(bg + sw) = pk;
                            pk.x = pack2_bf16(u8[0], u8[1]); pk.y = pack2_bf16(u8[2], u8[3]); pk.z = pack2_bf16(u8[4], u8[5]); pk.w = pack2_bf16(u8[6], u8[7]);
                            *reinterpret_cast<uint4*>(bu + sw) = pk;
                            pk.x = pack2_bf16(h8[0], h8[1]); pk.y = pack2_bf16(h8[2], h8[3]); pk.z = pack2_bf16(h8[4], h8[5]); pk.w = pack2_bf16(h8[6], h8[7]);
                            *reinterpret_cast<uint4*>(bh + sw) = pk;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        const int cx = tl * 128 + j * 64;
                        tma_store_3d(&tmC, stg_u32 + ((pieces) & 3) * 4096, cx, row0, 0); bulk_commit2();
                        tma_store_3d(&tmC1, stg_u32 + ((pieces + 1) & 3) * 4096, cx, row0, 0); bulk_commit2();
                        tma_store_3d(&tmC2, stg_u32 + ((pieces + 2) & 3) * 4096, cx, row0, 0); bulk_commit2();
                    }
                    pieces += 3;
                }
            } else if (tma_out) {
#pragma unroll 1
                for (int j = 0; j < npc && ok; j++) {
                    const int c = j * cw;
                    const uint32_t bi = pieces & (nbuf - 1);
                    uint8_t* buf = stg + bi * 4096 + lane * 128;
                    if (lane == 0) bulk_wait_read_le1();        // all but the latest store have read their buffers
                    if (tma_out == 2) {
                        if (lane == 0 && j + 2 < npc) fetch_d(j + 2);
                        if (!mbar_wait(my_bar_d + 8 * bi, (dpar >> bi) & 1)) { ok = false; break; }
                        dpar ^= 1u << bi;
                    }
                    __syncwarp();
                    uint32_t r[32];
                    tmem_ld32(taddr + c, r);
                    tmem_ld_wait();
                    if (f32_out) {
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            float4* slot = reinterpret_cast<float4*>(buf + ((q ^ (lane & 7)) << 4));
                            float4 f = make_float4(a_eff * __uint_as_float(r[q * 4]), a_eff * __uint_as_float(r[q * 4 + 1]),
                                                   a_eff * __uint_as_float(r[q * 4 + 2]), a_eff * __uint_as_float(r[q * 4 + 3]));
                            if (tma_out == 2) {
                                const float4 d = *slot;
                                f.x += beta * d.x; f.y += beta * d.y; f.z += beta * d.z; f.w += beta * d.w;
                            }
                            *slot = f;
                        }
                    } else if (do_rope) {
                        // the piece is one head: rotate the pairs (i, i + 32) in fp32, round once
                        uint32_t r2[32];
                        tmem_ld32(taddr + c + 32, r2);
                        tmem_ld_wait();
                        const float* cr = grp.rope_cos + (long long)rope_t * 32;
                        const float* sr = grp.rope_sin + (long long)rope_t * 32;
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const float4 c0 = __ldg(reinterpret_cast<const float4*>(cr + q * 8)), c1 = __ldg(reinterpret_cast<const float4*>(cr + q * 8 + 4));
                            const float4 s0 = __ldg(reinterpret_cast<const float4*>(sr + q * 8)), s1 = __ldg(reinterpret_cast<const float4*>(sr + q * 8 + 4));
                            const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                            const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                            float o1[8], o2[8];
#pragma unroll
                            for (int e = 0; e < 8; e++) {
                                const float x1 = a_eff * __uint_as_float(r[q * 8 + e]), x2 = a_eff * __uint_as_float(r2[q * 8 + e]);
                                o1[e] = x1 * cc[e] - x2 * ss[e];
                                o2[e] = x1 * ss[e] + x2 * cc[e];
                            }
                            uint4 pk;
                            pk.x = pack2_bf16(o1[0], o1[1]); pk.y = pack2_bf16(o1[2], o1[3]); pk.z = pack2_bf16(o1[4], o1[5]); pk.w = pack2_bf16(o1[6], o1[7]);
                            *reinterpret_cast<uint4*>(buf + ((q ^ (lane & 7)) << 4)) = pk;
                            pk.x = pack2_bf16(o2[0], o2[1]); pk.y = pack2_bf16(o2[2], o2[3]); pk.z = pack2_bf16(o2[4], o2[5]); pk.w = pack2_bf16(o2[6], o2[7]);
                            *reinterpret_cast<uint4*>(buf + (((4 + q) ^ (lane & 7)) << 4)) = pk;
                        }
                    } else {
#pragma unroll
                        for (int half = 0; half < 2; half++) {
                            if (half) { tmem_ld32(taddr + c + 32, r); tmem_ld_wait(); }
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                uint4* slot = reinterpret_cast<uint4*>(buf + (((half * 4 + q) ^ (lane & 7)) << 4));
                                float f[8];
#pragma unroll
                                for (int e = 0; e < 8; e++) f[e] = a_eff * __uint_as_float(r[q * 8 + e]);
                                if (tma_out == 2) {
                                    const uint4 d = *slot;
                                    const uint32_t dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
                                    for (int e = 0; e < 4; e++) {
                                        f[2 * e] += beta * __uint_as_float(dw[e] << 16);
                                        f[2 * e + 1] += beta * __uint_as_float(dw[e] & 0xffff0000u);
                                    }
                                }
                                uint4 pk;
                                pk.x = pack2_bf16(f[0], f[1]); pk.y = pack2_bf16(f[2], f[3]);
                                pk.z = pack2_bf16(f[4], f[5]); pk.w = pack2_bf16(f[6], f[7]);
                                *slot = pk;
                            }
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(pC, stg_u32 + bi * 4096, tl * BN2 + c, row0, ksplit > 1 ? split : 0);
                        bulk_commit2();
                    }
                    pieces++;
                }
                if (!ok) break;
            } else {
                TO* crow = C + (long long)row * n;
                const TO* drow = (D && beta != 0.f) ? D + (long long)row * n : nullptr;
                float* wrow = ws + ((long long)split * m + row) * n;
#pragma unroll 1
                for (int c = 0; c < BN2; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c, r);
                    tmem_ld_wait();
                    const int col0 = tn * BN2 + c;
                    if (row < m && col0 < n) {
                        if (ksplit > 1) epi_store<float>(wrow, nullptr, r, col0, n - col0, 1.f, 0.f, (n & 3) == 0);
                        else epi_store<TO>(crow, drow, r, col0, n - col0, alpha, beta, vec_ok);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive_cluster(tempty_leader + 8 * acc);   // 256 arrivals (both CTAs) free the accumulator
            if (timing && threadIdx.x == 64) prof[6] = clock64();
        }
        if (tma_out && lane == 0) bulk_wait_read_all();       // staging stays valid until the last store has read it
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(status, STAT_GEMM2 | 3); }
    }
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();                                    // nobody frees TMEM while the peer may still use the pair
    if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc2(tmem_base, 512); }
    if (timing && threadIdx.x == 0) prof[7] = clock64();
}

// ── host ────────────────────────────────────────────────────────────────────
extern float* ax_splitk_ws(size_t* bytes);
extern int ax_gemm_pdl(void);
extern int ax_gemm_tma_out(void);
template <typename TO>
void ax_splitk_reduce_launch(const float* ws, int ksplit, TO* C, const TO* D, long long mn, float alpha, float beta, cudaStream_t st);

static int g_pairs[3][2];          // max co-resident pairs per kernel variant (0 = unknown)

template <int A_MN, int B_MN, typename TO>
static int pairs_for(int slot, int tslot) {
    if (g_pairs[slot][tslot] == 0) {
        cudaFuncSetAttribute(k_gemm_tc2<A_MN, B_MN, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * AX_SMS, 1, 1);
        cfg.blockDim = dim3(THREADS2, 1, 1);
        cfg.dynamicSmemBytes = SMEM2;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        int nc = 0;
        if (cudaOccupancyMaxActiveClusters(&nc, k_gemm_tc2<A_MN, B_MN, TO>, &cfg) != cudaSuccess || nc < 1) { cudaGetLastError(); nc = -1; }
        g_pairs[slot][tslot] = nc;
    }
    return g_pairs[slot][tslot];
}

// operand / output tensor maps of one problem
template <int A_MN> static int map_a(CUtensorMap* t, const void* A, int m, int k) {
    uint64_t dims[2], strides[1]; uint32_t box[2];
    if (A_MN) { dims[0] = m; dims[1] = k; strides[0] = (uint64_t)m * 2; box[0] = 64; box[1] = BK2; }
    else { dims[0] = k; dims[1] = m; strides[0] = (uint64_t)k * 2; box[0] = BK2; box[1] = BM2; }
    return tc_make_tmap_bf16(t, A, 2, dims, strides, box, true);
}
template <int B_MN> static int map_b(CUtensorMap* t, const void* B, int n, int k) {
    uint64_t dims[2], strides[1]; uint32_t box[2];
    if (B_MN) { dims[0] = n; dims[1] = k; strides[0] = (uint64_t)n * 2; box[0] = 64; box[1] = BK2; }
    else { dims[0] = k; dims[1] = n; strides[0] = (uint64_t)k * 2; box[0] = BK2; box[1] = 128; }
    return tc_make_tmap_bf16(t, B, 2, dims, strides, box, true);
}
// {n, m, nz} tensor of osz-byte elements, pieces of 128 bytes x 32 rows
static int map_c(CUtensorMap* t, void* base, int m, int n, int nz, int osz) {
    PFN_tmapEncodeTiled enc = tc_encode_fn();
    if (!enc) return 2;
    cuuint64_t gd[3] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)nz};
    cuuint64_t gs[2] = {(cuuint64_t)n * osz, (cuuint64_t)m * n * osz};
    cuuint32_t bx[3] = {(cuuint32_t)(128 / osz), 32, 1};
    cuuint32_t es[3] = {1, 1, 1};
    if (gs[1] % 16 != 0) gs[1] = (gs[1] + 15) / 16 * 16;     // only reached with nz == 1 (never indexed)
    const CUtensorMapDataType dtp = osz == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    return enc(t, dtp, 3, base, gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : 2;
}

// One launch.  grp.mode 0: the plain GEMM (A, B, C, D are element 0 of the arrays).  Grouped modes: see GemmGroup;
// n[] / k[] then hold the per-problem widths (mode 1) or per-segment depths (mode 2).
// Extra K-segments of a grouped launch: mode 1 — problem g adds XA[g] XB[g] (depth xk) to its output; mode 2 — they are
// appended to the launch's own segments (A, B, kv then hold count + xcount entries, at most 6).
template <int A_MN, int B_MN, typename TO>
static int gemm2_launch(int slot, int mode, int count, const void* const* A, const void* const* B, void* const* C, const void* D,
                        const int* mv, const int* nv, const int* kv, float alpha, float beta, int* status, int ksplit, cudaStream_t st,
                        const void* const* XA = nullptr, const void* const* XB = nullptr, int xk = 0) {
    const int maxp = pairs_for<A_MN, B_MN, TO>(slot, sizeof(TO) == 2 ? 0 : 1);
    if (maxp < 1) return -1;
    const int m = mv[0], n = nv[0], k = kv[0];
    GemmGroup grp = {};
    grp.mode = mode; grp.count = count;
    if (g_rope_req.rope_mask) {              // a rotary request is honoured by a mode-1 bf16 launch or refused
        grp.rope_cos = g_rope_req.rope_cos; grp.rope_sin = g_rope_req.rope_sin;
        grp.rope_T = g_rope_req.rope_T; grp.rope_mask = g_rope_req.rope_mask;
        g_rope_req.rope_mask = 0;
        if (mode != 1 || sizeof(TO) != 2 || grp.rope_T < 1 || !grp.rope_cos || !grp.rope_sin) return -1;
        for (int g = 0; g < count; g++) if (((grp.rope_mask >> g) & 1) && nv[g] % 64) return -1;
    }
    CUtensorMap tmA[3], tmB[3], tmC[3], tmD, tmEA[3], tmEB[3];
    bool have_x = false;
    int tiles_n = 0;
    if (mode == 0) {
        if (map_a<A_MN>(&tmA[0], A[0], m, k) || map_b<B_MN>(&tmB[0], B[0], n, k)) return 2;
        tiles_n = (n + 255) / 256;
    } else if (mode == 1) {
        if (map_a<A_MN>(&tmA[0], A[0], m, k)) return 2;
        for (int g = 0; g < count; g++) {
            if (map_b<B_MN>(&tmB[g], B[g], nv[g], k)) return 2;
            grp.n[g] = nv[g];
            tiles_n += (nv[g] + 255) / 256;
            if (XA && xk > 0) {
                if (map_a<A_MN>(&tmEA[g], XA[g], m, xk) || map_b<B_MN>(&tmEB[g], XB[g], nv[g], xk)) return 2;
                have_x = true;
            }
        }
        if (have_x) grp.xkb = (xk + BK2 - 1) / BK2;
    } else if (mode == 2) {
        if (count > 6) return -1;
        for (int g = 0; g < count; g++) {
            CUtensorMap* ta = g < 3 ? &tmA[g] : &tmEA[g - 3];
            CUtensorMap* tb_ = g < 3 ? &tmB[g] : &tmEB[g - 3];
            if (map_a<A_MN>(ta, A[g], m, kv[g]) || map_b<B_MN>(tb_, B[g], n, kv[g])) return 2;
            grp.kb[g] = (kv[g] + BK2 - 1) / BK2;
        }
        have_x = count > 3;
        tiles_n = (n + 255) / 256;
    } else if (mode == 3) {
        for (int g = 0; g < count; g++) {
            if (map_a<A_MN>(&tmA[g], A[g], mv[g], k) || map_b<B_MN>(&tmB[g], B[g], nv[g], k)) return 2;
            grp.m[g] = mv[g]; grp.n[g] = nv[g];
        }
    } else {        // mode 4: gate and up weights of the same width n; outputs g, u, h
        if (sizeof(TO) != 2 || count != 2) return -1;
        if (map_a<A_MN>(&tmA[0], A[0], m, k) || map_b<B_MN>(&tmB[0], B[0], n, k) || map_b<B_MN>(&tmB[1], B[1], n, k)) return 2;
    }
    const bool per_problem_c = mode == 1 || mode == 3;
    // output through TMA tile stores when the destination allows it: 1 = no addend to read, 2 = addend by TMA too
    const int osz = ksplit > 1 ? 4 : (int)sizeof(TO);
    const bool has_d = D != nullptr && beta != 0.f && ksplit == 1;
    int tma_out = 0;
    bool c_ok = ax_gemm_tma_out() != 0;
    for (int g = 0; g < (per_problem_c ? count : (mode == 4 ? 3 : 1)); g++)
        c_ok = c_ok && ((uintptr_t)C[g] & 15) == 0 && ((long long)nv[per_problem_c ? g : 0] * osz) % 16 == 0;
    if (c_ok && (!has_d || ((uintptr_t)D & 15) == 0)) tma_out = has_d ? 2 : 1;
    // grouped launches need the TMA-store epilogue; only the K-segment form takes an addend
    if (mode != 0 && (ksplit != 1 || !(tma_out == 1 || (tma_out == 2 && mode == 2)))) return -1;
    if (grp.rope_mask && tma_out != 1) return -1;
    if (tma_out) {
        size_t wsb0 = 0;
        if (per_problem_c) {
            for (int g = 0; g < count; g++) if (map_c(&tmC[g], C[g], mode == 3 ? mv[g] : m, nv[g], 1, osz)) return 2;
        } else if (mode == 4) {
            for (int g = 0; g < 3; g++) if (map_c(&tmC[g], C[g], m, n, 1, osz)) return 2;
        } else {
            void* base = ksplit > 1 ? (void*)ax_splitk_ws(&wsb0) : C[0];
            if (map_c(&tmC[0], base, m, n, ksplit > 1 ? ksplit : 1, osz)) return 2;
        }
        tmD = tmC[0];
        if (tma_out == 2 && map_c(&tmD, const_cast<void*>(D), m, n, 1, osz)) return 2;
    } else {
        tmC[0] = tmA[0]; tmD = tmA[0];
    }
    for (int g = 0; g < 3; g++) {           // unused slots carry valid (ignored) maps
        const bool used = mode == 1 ? (have_x && g < count) : (mode == 2 && g + 3 < count);
        if (!used) { tmEA[g] = tmA[0]; tmEB[g] = tmB[0]; }
    }
    for (int g = 1; g < 3; g++) {
        if ((mode != 2 && mode != 3) || g >= count) tmA[g] = tmA[0];
        if (mode == 0 || g >= count) tmB[g] = tmB[0];
        if (mode != 4 && (!per_problem_c || g >= count || !tma_out)) tmC[g] = tmC[0];
    }
    int units = ((m + 255) / 256) * tiles_n * ksplit;
    if (mode == 3) { units = 0; for (int g = 0; g < count; g++) units += ((mv[g] + 255) / 256) * ((nv[g] + 255) / 256); }
    if (mode == 4) units = ((m + 255) / 256) * ((n + 127) / 128);
    const int pairs = units < maxp ? units : maxp;
    size_t wsb = 0;
    float* ws = ax_splitk_ws(&wsb);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(THREADS2, 1, 1);
    cfg.dynamicSmemBytes = SMEM2;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = ax_gemm_pdl() ? 2 : 1;
    TO* Cp = (TO*)C[0]; const TO* Dp = (const TO*)D;
    long long* prof = nullptr;
#ifdef AXENG_PROF       // debugging aid of instrumented builds: allocates, synchronises and prints per launch
    static const bool want_prof = getenv("AXENG_GEMM_PROF") != nullptr;
    if (want_prof && (cudaMalloc(&prof, 64) != cudaSuccess || cudaMemset(prof, 0, 64) != cudaSuccess)) prof = nullptr;
#endif
    if (cudaLaunchKernelEx(&cfg, k_gemm_tc2<A_MN, B_MN, TO>, tmA[0], tmB[0], tmC[0], tmD, tmA[1], tmA[2], tmB[1], tmB[2], tmC[1], tmC[2],
                           tmEA[0], tmEA[1], tmEA[2], tmEB[0], tmEB[1], tmEB[2], grp, tma_out, Cp, Dp, m, n, k, alpha, beta, status, ksplit, ws, prof) != cudaSuccess) return 3;
#ifdef AXENG_PROF
    if (prof) {
        long long h[8];
        cudaStreamSynchronize(st);
        cudaMemcpy(h, prof, 64, cudaMemcpyDeviceToHost);
        cudaFree(prof);
        fprintf(stderr, "gemm2 %dx%dx%d mode %d split %d pairs %d (cycles from entry): setup %lld dep %lld first_full %lld last_mma %lld last_acc %lld stored %lld exit %lld\n",
                m, n, k, mode, ksplit, pairs, h[1] - h[0], h[2] - h[0], h[3] - h[0], h[4] - h[0], h[5] - h[0], h[6] - h[0], h[7] - h[0]);
    }
#endif
    if (ksplit > 1) ax_splitk_reduce_launch<TO>(ws, ksplit, Cp, Dp, (long long)m * n, alpha, beta, st);
    return 0;
}

// Resolve the co-resident pair count of every variant up front (not while a graph is being captured).
int ax_gemm_tc2_init(void) {
    int worst = 1 << 30;
    int v[6] = {pairs_for<0, 1, bf16>(0, 0), pairs_for<0, 1, float>(0, 1), pairs_for<0, 0, bf16>(1, 0),
                pairs_for<0, 0, float>(1, 1), pairs_for<1, 1, bf16>(2, 0), pairs_for<1, 1, float>(2, 1)};
    for (int i = 0; i < 6; i++) worst = v[i] < worst ? v[i] : worst;
    return worst;      // pairs that can run together (<= 0: the paired kernel is unavailable)
}

// Same argument meaning as ax_gemm_tc; returns -1 when the paired kernel cannot run here.
int ax_gemm_tc2(int out_bf16, int tb, const void* A, const void* B, void* C, const void* D,
                int m, int n, int k, float alpha, float beta, int* status, int ksplit, cudaStream_t st) {
    const void* Av[1] = {A}; const void* Bv[1] = {B}; void* Cv[1] = {C};
#define G2(AM, BMj, SL)                                                                                                        \
    (out_bf16 ? gemm2_launch<AM, BMj, bf16>(SL, 0, 1, Av, Bv, Cv, D, &m, &n, &k, alpha, beta, status, ksplit, st)             \
              : gemm2_launch<AM, BMj, float>(SL, 0, 1, Av, Bv, Cv, D, &m, &n, &k, alpha, beta, status, ksplit, st))
    if (tb == 0) return G2(0, 1, 0);
    if (tb == 1) return G2(0, 0, 1);
    return G2(1, 1, 2);
#undef G2
}

// Grouped launch (see GemmGroup).  mode 1: A[0] shared, B[g] / C[g] / n[g] per problem, m[0], k[0].  mode 2: A[s] / B[s] /
// k[s] per segment, C[0], m[0], n[0].  mode 3: A[g] / B[g] / C[g] / m[g] / n[g] per problem, k[0].  Returns -1 when this
// kernel cannot serve the request (the caller then runs the problems one by one).  mode 4: A[0], B[0] = gate weights,
// B[1] = up weights (both n[0] wide), C[0] = g, C[1] = u, C[2] = silu(g) * u; bf16 output only.  XA / XB / xk (mode 1):
// every problem's own extra K-segment.  Mode 2 takes up to 6 segments and an addend D (C = alpha * sum + beta * D).
int ax_gemm_tc2_group(int out_bf16, int tb, int mode, int count, const void* const* A, const void* const* B, void* const* C,
                      const int* m, const int* n, const int* k, float alpha, int* status, cudaStream_t st,
                      const void* const* XA, const void* const* XB, int xk, const void* D, float beta) {
    const int rope_mask = g_rope_req.rope_mask;
    const int maxc = mode == 2 ? 6 : 3;
    if (count < 2 || count > maxc || mode < 1 || mode > 4) { g_rope_req.rope_mask = 0; return -1; }
    if (mode == 4 && (!out_bf16 || count != 2 || !aligned16(C[2]))) { g_rope_req.rope_mask = 0; return -1; }
    if (rope_mask && (mode != 1 || !out_bf16 || tb != 0)) { g_rope_req.rope_mask = 0; return -1; }
    if (XA && (mode != 1 || tb == 2 || xk < 8 || xk % 8)) { g_rope_req.rope_mask = 0; return -1; }
    if (D && (mode != 2 || !aligned16(D))) { g_rope_req.rope_mask = 0; return -1; }
    for (int g = 0; g < count; g++) {
        bool bad = !aligned16(A[(mode == 2 || mode == 3) ? g : 0]) || !aligned16(B[g]);
        if (XA) bad = bad || !XA[g] || !XB[g] || !aligned16(XA[g]) || !aligned16(XB[g]);
        const int mg = m[mode == 3 ? g : 0], ng = n[(mode == 1 || mode == 3) ? g : 0], kg = k[mode == 2 ? g : 0];
        bad = bad || mg < 256 || ng < 8 || kg < 8;
        if (tb == 0) bad = bad || kg % 8 || ng % 8;
        else if (tb == 1) bad = bad || kg % 8;
        else bad = bad || mg % 8 || ng % 8;
        if (bad) { g_rope_req.rope_mask = 0; return -1; }
    }
#define G2(AM, BMj, SL)                                                                                                        \
    (out_bf16 ? gemm2_launch<AM, BMj, bf16>(SL, mode, count, A, B, C, D, m, n, k, alpha, D ? beta : 0.f, status, 1, st, XA, XB, xk)   \
              : gemm2_launch<AM, BMj, float>(SL, mode, count, A, B, C, D, m, n, k, alpha, D ? beta : 0.f, status, 1, st, XA, XB, xk))
    if (tb == 0) return G2(0, 1, 0);
    if (tb == 1) return G2(0, 0, 1);
    return G2(1, 1, 2);
#undef G2
}
