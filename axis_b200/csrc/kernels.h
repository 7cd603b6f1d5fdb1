// Internal launch interface between the dispatcher (axeng.cu) and the kernel
// translation units.  Every function enqueues on `st` and returns 0, or a
// non-zero code when the arguments cannot be served.
#pragma once
#include <cuda_runtime.h>

// dt: 0 = fp32 storage, 1 = bf16 storage (2 = bf16 in / fp32 out where stated)

// Code of the kernel variant the last multi-variant launcher chose (read through eng_last_variant; the parity
// tests assert with it that a shape really ran on the kernel they mean to check):
//   0x10 cross-entropy streaming rows, 0x11 cross-entropy register-resident rows,
//   0x20 general GEMM, 0x21 single-CTA tcgen05 GEMM, 0x22 paired-CTA tcgen05 GEMM (+ 0x100 * split-K factor)
extern int ax_variant;

// elementwise.cu
int ax_binary(int which, int dt, const void* a, const void* b, void* c, long long n, cudaStream_t st); // 0 add 1 mul 2 silu_mul
int ax_scale(int dt, const void* a, void* c, float alpha, long long n, cudaStream_t st);
int ax_copy(int dt, const void* a, void* c, long long n, cudaStream_t st);
int ax_cast(int to_f32, const void* a, void* c, long long n, cudaStream_t st);
int ax_transpose_bf16(int out_f32, const void* a, void* c, int rows, int cols, cudaStream_t st);
int ax_perm0213(int dt, const void* a, void* c, int d0, int d1, int d2, int d3, cudaStream_t st);
int ax_rope(int dt, const void* x, const float* cs, const float* sn, void* o, int T, int dh,
            long long rows, int heads_inner, int inverse, cudaStream_t st);
int ax_rope2(int dt, const void* x, const float* cs, const float* sn, void* o, int T, int dh, long long rows, int heads_inner,
             int inverse, const void* x2, void* o2, long long rows2, int heads_inner2, cudaStream_t st);
int ax_repeat_kv(int dt, const void* x, void* o, int B, int KV, int H, int T, int dh, cudaStream_t st);
int ax_repeat_kv_bwd(int dt, const void* g, void* o, int B, int KV, int H, int T, int dh, cudaStream_t st);
int ax_softmax_causal(int dt, const void* x, void* o, int rpb, int width, int qoff, long long rows, cudaStream_t st);
int ax_softmax_bwd(int dt, const void* p, const void* dp, void* ds, int width, long long rows, cudaStream_t st);
int ax_silu_bwd(int dt, const void* g, const void* u, const void* grad, void* dg, void* du, long long n, cudaStream_t st);
int ax_rowdot(int dt, const void* a, const void* b, float* c, long long rows, int dim, cudaStream_t st);

// norm.cu
int ax_rmsnorm(int dt, const void* x, const void* w, void* o, int rows, int dim, float eps, cudaStream_t st);
int ax_rmsnorm_bwd(int dt, const void* x, const void* w, const void* g, void* dx, void* tmp, int rows, int dim, float eps, cudaStream_t st);
int ax_colsum(int dt, const void* a, float* c, int rows, int n, cudaStream_t st);
// dx = (res ? res : 0) + rmsnorm_bwd; dw (fp32, may be null) written, or accumulated when dw_acc.
// scratch: >= ax_rmsnorm_bwd_acc_scratch(dim) bytes.
long long ax_rmsnorm_bwd_acc_scratch(int dim);
int ax_rmsnorm_bwd_acc(int dt, const void* x, const void* w, const void* g, const void* res, void* dx,
                       float* dw, float* scratch, int rows, int dim, float eps, cudaStream_t st, int defer = 0);
// Sums the partials that `count` deferred launches left in consecutive scratch areas (see norm.cu).
int ax_colsum_batch(const float* scratch, float* arena, const int* table, int first, int count, int dim, int chunk,
                    long long arena_elems, int* status, cudaStream_t st);

// loss.cu
// rows = rows of the table (derived from its buffer size by the caller): an id or target outside its range is
// skipped and recorded in the status word (0x401 gather, 0x402 scatter, 0x403 cross-entropy target)
int ax_embed(int dt, const void* table, const void* ids, int ids_i32, void* o, int N, int D, int rows, int* status, cudaStream_t st);
int ax_embed_bwd_atomic(int g_bf16, const void* g, const float* ids, float* dT, int N, int D, int rows, int* status, cudaStream_t st);
int ax_embed_bwd_det(int g_dt, const void* g, const int* ids, float* dT, int N, int D, int rows, int* status, cudaStream_t st);
int ax_countvalid(const float* tgt, float* acc, int N, cudaStream_t st);
int ax_ce(int dt, const void* logits, const float* tgt, void* dlogits, float* loss, const float* denom, int N, int V, int* status, cudaStream_t st);
// scratch: N + 8 floats. targets int32 (<0 ignored). loss[0] = mean NLL over valid, denom[0] = count.
int ax_ce_fused(int dt, const void* logits, const int* tgt, void* dlogits, float* loss, float* denom,
                float* scratch, int N, int V, int* status, cudaStream_t st);

// optim.cu
int ax_adamw(float* p, const float* g, float* m, float* v, const float* tbuf, void* pbf,
             const float* lrbuf, const float* gsbuf, float alpha, float beta, float gamma, long long n, cudaStream_t st);
int ax_l2acc(const float* g, float* acc, long long n, cudaStream_t st);
int ax_clipscale(const float* acc, float* scale, float max_norm, cudaStream_t st);
int ax_tick(float* t, cudaStream_t st);
#define AX_GNORM_CHUNK 8192          // elements per partial of the flat grad-norm
#define AX_ADAMW_CHUNK 1024          // granularity of the weight-decay flag table
// partials[i] = sum of squares of chunk i (fixed in-chunk order); tick (may be null) += 1;
// out (may be null) = sum of the partials in a fixed order.
int ax_gnorm_flat(const float* g, float* partials, long long n, float* tick, float* out, cudaStream_t st);
// One pass: scale = clip(sum(partials[0..np)) ), AdamW on n elements; wdflag[i] per AX_ADAMW_CHUNK.
int ax_adamw_flat(float* p, const float* g, float* m, float* v, void* pbf, const unsigned char* wdflag,
                  const float* tbuf, const float* lrbuf, const float* partials, int np, float* gnorm_out,
                  float max_norm, float wd, float eps, long long n, cudaStream_t st);

// gemm_simt.cu — general fp32-accumulate GEMM, any shape/stride; in: fp32|bf16, out: fp32|bf16
// C[m,n] = alpha * op(A) op(B) + beta * D   (D may alias C or be null when beta == 0)
int ax_gemm_simt(int in_bf16, int out_bf16, int tb, const void* A, const void* B, void* C, const void* D,
                 int m, int n, int k, int batch, long long sa, long long sb, long long sc,
                 float alpha, float beta, cudaStream_t st);

// gemm_tc.cu — tcgen05/TMEM/TMA bf16 GEMM. Returns -1 when the shape/alignment is not served.
int ax_gemm_tc_init(void);
int ax_gemm_tc(int out_bf16, int tb, const void* A, const void* B, void* C, const void* D,
               int m, int n, int k, float alpha, float beta, int* status, cudaStream_t st);

// gemm_tc2.cu — paired-CTA (cta_group::2) variant, 256 x 256 tile per two SMs
int ax_gemm_tc2_init(void);
int ax_gemm_tc2(int out_bf16, int tb, const void* A, const void* B, void* C, const void* D,
                int m, int n, int k, float alpha, float beta, int* status, int ksplit, cudaStream_t st);
void ax_gemm_set_mode(int mode);      // 0 auto, 1 single-CTA only, 2 paired whenever possible

// attn_simt.cu — exact-fp32 causal GQA attention on strided layouts.
struct AttnShape {
    int B, H, KV, T, DH;
    // element strides of q/o/dO/dq (per batch, head, token) and k/v/dk/dv
    long long qb, qh, qt, kb, kh, kt;
    // D (row dot) strides: D[b*db + h*dh_ + t*dtk]
    long long db, dh_, dtk;
    float scale;
};
int ax_attn_fwd_simt(int dt, const void* q, const void* k, const void* v, void* o, float* lse,
                     const AttnShape& s, cudaStream_t st);
// out_dt: storage type of dq/dk/dv (0 fp32, 1 bf16)
int ax_attn_bwd_simt(int dt, int out_dt, const void* q, const void* k, const void* v, const void* dO,
                     const float* lse, const float* Dv, void* dq, void* dk, void* dv,
                     const AttnShape& s, cudaStream_t st);

// gemm_tc2.cu — grouped launch of the paired-CTA GEMM (mode 1: shared A, per-problem B/C/n; mode 2: one C summed
// over per-segment A/B/k; mode 3: independent problems A/B/C/m/n of one depth k).  -1 when not served.
void ax_gemm_side(int on);
// Rotary request for the NEXT ax_gemm_tc2_group call (mode 1, bf16 output, tb 0): outputs g with bit g of `mask` set are
// [rows, heads * 64] projections and leave the launch rotated (tables fp32 [T, 32], row = batch * T + token).  The call
// either honours the request or returns -1; it never ignores it.
void ax_gemm_group_rope(const float* cs, const float* sn, int T, int mask);
// XA / XB / xk (mode 1, may be null): problem g adds XA[g] XB[g] of depth xk to its output.  Mode 2 takes up to six
// segments and an addend D: C = alpha * sum + beta * D.
int ax_gemm_tc2_group(int out_bf16, int tb, int mode, int count, const void* const* A, const void* const* B, void* const* C,
                      const int* m, const int* n, const int* k, float alpha, int* status, cudaStream_t st,
                      const void* const* XA = nullptr, const void* const* XB = nullptr, int xk = 0,
                      const void* D = nullptr, float beta = 0.f);

// fp32 scratch of the split-K GEMMs (main stream only), also used by the adapter-gradient kernel
float* ax_splitk_ws(size_t* bytes);

// lora.cu — adapter weight gradients out[g] = alpha * X[g]^T S[g] (X [N, F[g]], S [N, R] bf16; out fp32 [F, R], or
// [R, F] where layout[g] is 1) for up to sixteen products in one launch pair.  -1 when not served.
// out[g] [N, R] bf16 = alpha * X[g] [N, F[g]] W[g] with W [F, R] (tb 0) or [R, F] (tb 1): the skinny products of an adapter.
int ax_lora_proj(int count, int tb, const void* const* X, const void* const* W, void* const* out, const int* F, int N, int R,
                 float alpha, cudaStream_t st);
int ax_lora_grad(int count, const void* const* X, const void* const* S, float* const* out, const int* F, const int* layout,
                 int N, int R, float alpha, float* ws, size_t ws_bytes, cudaStream_t st);

// attn_tc.cu — tcgen05 flash attention (bf16, DH 64/128). -1 when not served.
int ax_attn_tc_init(void);
int ax_attn_tc128_init(void);
int ax_attn_fwd_tc(const void* q, const void* k, const void* v, void* o, float* lse,
                   const AttnShape& s, int* status, cudaStream_t st);
// dq_acc: fp32 accumulator of B*T*H*DH elements for the dQ reduce-add (null -> not served).
// rope_cos / rope_sin (fp32 [T, DH/2], may be null): when given, the inverse rotary is applied to dq and dk
// before they are rounded to bf16 (head_dim 64 only; -1 otherwise, the caller then runs the rotary op itself).
int ax_attn_bwd_tc(const void* q, const void* k, const void* v, const void* o, const void* dO,
                   const float* lse, float* Dscratch, float* dq_acc, void* dq, void* dk, void* dv,
                   const AttnShape& s, const float* rope_cos, const float* rope_sin, int* status, cudaStream_t st);
// attn_tc128.cu — the head_dim-128 kernels behind the two entry points above.
int ax_attn_fwd_tc128(const void* q, const void* k, const void* v, void* o, float* lse,
                      const AttnShape& s, int* status, cudaStream_t st);
int ax_attn_bwd_tc128(const void* q, const void* k, const void* v, const void* o, const void* dO,
                      const float* lse, float* Dscratch, float* dq_acc, void* dq, void* dk, void* dv,
                      const AttnShape& s, int* status, cudaStream_t st);
