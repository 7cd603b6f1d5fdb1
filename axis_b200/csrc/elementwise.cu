// Elementwise and small-reduction kernels: 16-byte vector accesses where the
// pointers allow it, scalar tails otherwise.  All arithmetic in fp32.
#include "common.cuh"
#include "kernels.h"

#define T256 256

// ── binary ops ──────────────────────────────────────────────────────────────
// exp for storage type T: full-precision expf in fp32 plans, __expf under bf16 storage
template <typename T> __device__ __forceinline__ float exp_t(float x) {
    return sizeof(T) == 4 ? expf(x) : __expf(x);
}
template <typename T, int OP> __device__ __forceinline__ float bin(float a, float b) {
    if (OP == 0) return a + b;
    if (OP == 1) return a * b;
    return (a / (1.f + exp_t<T>(-a))) * b;          // silu(a) * b
}
template <typename T, int OP>
__global__ void k_binary_vec(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c, long long n) {
    constexpr int N = Vec<T>::N;
    const long long nv = n / N;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
        float x[N], y[N];
        Vec<T>::ld(a + i * N, x);
        Vec<T>::ld(b + i * N, y);
#pragma unroll
        for (int j = 0; j < N; j++) x[j] = bin<T, OP>(x[j], y[j]);
        Vec<T>::st(c + i * N, x);
    }
    for (long long i = nv * N + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        stf(c, i, bin<T, OP>(ldf(a, i), ldf(b, i)));
}
template <typename T, int OP>
__global__ void k_binary(const T* a, const T* b, T* c, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        stf(c, i, bin<T, OP>(ldf(a, i), ldf(b, i)));
}
template <typename T, int OP>
static void launch_binary(const void* a, const void* b, void* c, long long n, cudaStream_t st) {
    if (aligned16(a) && aligned16(b) && aligned16(c))
        k_binary_vec<T, OP><<<ew_grid(n / Vec<T>::N + 1, T256), T256, 0, st>>>((const T*)a, (const T*)b, (T*)c, n);
    else
        k_binary<T, OP><<<ew_grid(n, T256), T256, 0, st>>>((const T*)a, (const T*)b, (T*)c, n);
}
int ax_binary(int which, int dt, const void* a, const void* b, void* c, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const bool h = dt == 1;
    switch (which) {
        case 0: h ? launch_binary<bf16, 0>(a, b, c, n, st) : launch_binary<float, 0>(a, b, c, n, st); break;
        case 1: h ? launch_binary<bf16, 1>(a, b, c, n, st) : launch_binary<float, 1>(a, b, c, n, st); break;
        default: h ? launch_binary<bf16, 2>(a, b, c, n, st) : launch_binary<float, 2>(a, b, c, n, st); break;
    }
    return 0;
}

// ── scale / zero / copy / cast ──────────────────────────────────────────────
template <typename T>
__global__ void k_scale(const T* a, T* c, float alpha, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        stf(c, i, ldf(a, i) * alpha);
}
int ax_scale(int dt, const void* a, void* c, float alpha, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const long long es = dt == 1 ? 2 : 4;
    // alpha == 0 is an explicit zero fill: the source is never read
    if (alpha == 0.f) return (int)cudaMemsetAsync(c, 0, n * es, st);
    if (dt == 1) k_scale<bf16><<<ew_grid(n, T256), T256, 0, st>>>((const bf16*)a, (bf16*)c, alpha, n);
    else k_scale<float><<<ew_grid(n, T256), T256, 0, st>>>((const float*)a, (float*)c, alpha, n);
    return 0;
}
int ax_copy(int dt, const void* a, void* c, long long n, cudaStream_t st) {
    if (n <= 0 || a == c) return 0;
    return (int)cudaMemcpyAsync(c, a, n * (dt == 1 ? 2 : 4), cudaMemcpyDeviceToDevice, st);
}
__global__ void k_cast_f2b(const float* __restrict__ a, bf16* __restrict__ c, long long n, int vec) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long start = 0;
    if (vec) {
        const long long nv = n / 8;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
            float f[8];
            Vec<float>::ld(a + i * 8, f);
            Vec<float>::ld(a + i * 8 + 4, f + 4);
            Vec<bf16>::st(c + i * 8, f);
        }
        start = nv * 8;
    }
    for (long long i = start + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        c[i] = __float2bfloat16(a[i]);
}
__global__ void k_cast_b2f(const bf16* __restrict__ a, float* __restrict__ c, long long n, int vec) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long start = 0;
    if (vec) {
        const long long nv = n / 8;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
            float f[8];
            Vec<bf16>::ld(a + i * 8, f);
            Vec<float>::st(c + i * 8, f);
            Vec<float>::st(c + i * 8 + 4, f + 4);
        }
        start = nv * 8;
    }
    for (long long i = start + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        c[i] = __bfloat162float(a[i]);
}
int ax_cast(int to_f32, const void* a, void* c, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const int vec = aligned16(a) && aligned16(c);
    if (!to_f32) k_cast_f2b<<<ew_grid(n / 8 + 1, T256), T256, 0, st>>>((const float*)a, (bf16*)c, n, vec);
    else k_cast_b2f<<<ew_grid(n / 8 + 1, T256), T256, 0, st>>>((const bf16*)a, (float*)c, n, vec);
    return 0;
}

// ── c[cols,rows] = a[rows,cols]^T, bf16 in, bf16 or fp32 out ───────────────
// Load-time layout change of checkpoint weights (stored [out,in]) to the [in,out] layout the GEMMs read:
// a 32 x 32 tile goes through shared memory so that both the reads and the writes are row-contiguous.
template <typename TO>
__global__ void __launch_bounds__(256) k_transpose_bf16(const bf16* __restrict__ a, TO* __restrict__ c, int rows, int cols) {
    __shared__ unsigned short tile[32][33];
    const unsigned short* ab = reinterpret_cast<const unsigned short*>(a);
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += 8)
        if (r0 + r < rows && c0 + threadIdx.x < cols) tile[r][threadIdx.x] = ab[(long long)(r0 + r) * cols + c0 + threadIdx.x];
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8)
        if (c0 + j < cols && r0 + threadIdx.x < rows) {
            const unsigned short v = tile[threadIdx.x][j];
            const long long o = (long long)(c0 + j) * rows + r0 + threadIdx.x;
            if constexpr (sizeof(TO) == 4) c[o] = __uint_as_float((unsigned)v << 16);
            else reinterpret_cast<unsigned short*>(c)[o] = v;
        }
}
int ax_transpose_bf16(int out_f32, const void* a, void* c, int rows, int cols, cudaStream_t st) {
    if (rows <= 0 || cols <= 0) return 0;
    const dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
    if (grid.y > 65535) return 121;
    if (out_f32) k_transpose_bf16<float><<<grid, block, 0, st>>>((const bf16*)a, (float*)c, rows, cols);
    else k_transpose_bf16<bf16><<<grid, block, 0, st>>>((const bf16*)a, (bf16*)c, rows, cols);
    return 0;
}

// ── [d0,d1,d2,d3] -> [d0,d2,d1,d3] ─────────────────────────────────────────
// One thread moves one 16-byte piece of a d3-row when d3 allows, else one element.
template <typename T, int W>
__global__ void k_perm0213(const T* __restrict__ x, T* __restrict__ o, int d0, int d1, int d2, int d3w) {
    const long long total = (long long)d0 * d1 * d2 * d3w;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int j3 = (int)(i % d3w);
        long long r = i / d3w;
        int j2 = (int)(r % d2); r /= d2;
        int j1 = (int)(r % d1); r /= d1;
        long long dst = ((r * d2 + j2) * d1 + j1) * d3w + j3;
        if (W == 1) o[dst] = x[i];
        else reinterpret_cast<uint4*>(o)[dst] = reinterpret_cast<const uint4*>(x)[i];
    }
}
int ax_perm0213(int dt, const void* a, void* c, int d0, int d1, int d2, int d3, cudaStream_t st) {
    const long long total = (long long)d0 * d1 * d2 * d3;
    if (total <= 0) return 0;
    const int per = dt == 1 ? 8 : 4;
    if (d3 % per == 0 && aligned16(a) && aligned16(c)) {
        if (dt == 1) k_perm0213<bf16, 8><<<ew_grid(total / per, T256), T256, 0, st>>>((const bf16*)a, (bf16*)c, d0, d1, d2, d3 / per);
        else k_perm0213<float, 4><<<ew_grid(total / per, T256), T256, 0, st>>>((const float*)a, (float*)c, d0, d1, d2, d3 / per);
    } else {
        if (dt == 1) k_perm0213<bf16, 1><<<ew_grid(total, T256), T256, 0, st>>>((const bf16*)a, (bf16*)c, d0, d1, d2, d3);
        else k_perm0213<float, 1><<<ew_grid(total, T256), T256, 0, st>>>((const float*)a, (float*)c, d0, d1, d2, d3);
    }
    return 0;
}

// ── rotary embedding (half split) ───────────────────────────────────────────
// Rows of dh elements; the token of row r is (r / heads_inner) % T, which
// covers both [B,H,T,dh] (heads_inner = 1) and [B,T,H,dh] (heads_inner = H).
// One thread handles the pair (j, j + dh/2); in place is safe.
template <typename T>
__global__ void k_rope(const T* x, const float* __restrict__ cs, const float* __restrict__ sn, T* o,
                       int T_, int dh, long long rows, int heads_inner, int inverse) {
    const int half = dh >> 1;
    const long long total = rows * half;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int j = (int)(i % half);
        const long long r = i / half;
        const int t = (int)((r / heads_inner) % T_);
        const float c = cs[t * half + j];
        const float s = inverse ? -sn[t * half + j] : sn[t * half + j];
        const float x1 = ldf(x, r * dh + j), x2 = ldf(x, r * dh + j + half);
        stf(o, r * dh + j, x1 * c - x2 * s);
        stf(o, r * dh + j + half, x1 * s + x2 * c);
    }
}
// 16-byte version: a thread rotates 8 (bf16) or 4 (fp32) consecutive pairs.  A second tensor with its own head count
// (the key projection next to the query projection) rides in the same launch.
template <typename T>
__global__ void k_rope_vec(const T* x, const float* __restrict__ cs, const float* __restrict__ sn, T* o,
                           int T_, int dh, long long rows, int heads_inner, int inverse,
                           const T* x2, T* o2, long long rows2, int heads_inner2) {
    constexpr int N = Vec<T>::N;
    const int half = dh >> 1, hv = half / N;
    const long long total1 = rows * hv, total = total1 + rows2 * hv;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const bool second = i >= total1;
        const long long ii = second ? i - total1 : i;
        const T* xs = second ? x2 : x;
        T* os = second ? o2 : o;
        const int hi = second ? heads_inner2 : heads_inner;
        const int j = (int)(ii % hv) * N;
        const long long r = ii / hv;
        const int t = (int)((r / hi) % T_);
        float x1[N], x2v[N], c[N], s[N], o1[N], o2v[N];
        Vec<T>::ld(xs + r * dh + j, x1);
        Vec<T>::ld(xs + r * dh + j + half, x2v);
#pragma unroll
        for (int q = 0; q < N; q += 4) {
            Vec<float>::ld(cs + t * half + j + q, c + q);
            Vec<float>::ld(sn + t * half + j + q, s + q);
        }
#pragma unroll
        for (int q = 0; q < N; q++) {
            const float sq = inverse ? -s[q] : s[q];
            o1[q] = x1[q] * c[q] - x2v[q] * sq;
            o2v[q] = x1[q] * sq + x2v[q] * c[q];
        }
        Vec<T>::st(os + r * dh + j, o1);
        Vec<T>::st(os + r * dh + j + half, o2v);
    }
}
int ax_rope(int dt, const void* x, const float* cs, const float* sn, void* o, int T_, int dh,
            long long rows, int heads_inner, int inverse, cudaStream_t st) {
    return ax_rope2(dt, x, cs, sn, o, T_, dh, rows, heads_inner, inverse, nullptr, nullptr, 0, 1, st);
}
// x2/o2 (optional): a second tensor of rows2 rows with heads_inner2 heads per token, rotated in the same launch
int ax_rope2(int dt, const void* x, const float* cs, const float* sn, void* o, int T_, int dh,
             long long rows, int heads_inner, int inverse, const void* x2, void* o2, long long rows2, int heads_inner2,
             cudaStream_t st) {
    if (rows <= 0 || dh < 2) return 0;
    if (heads_inner < 1) heads_inner = 1;
    if (heads_inner2 < 1) heads_inner2 = 1;
    if (!x2) rows2 = 0;
    const int half = dh / 2;
    const int N = dt == 1 ? 8 : 4;
    const bool vec = (half % N == 0) && aligned16(x) && aligned16(o) && aligned16(cs) && aligned16(sn) &&
                     (!x2 || (aligned16(x2) && aligned16(o2)));
    if (vec) {
        const long long items = (rows + rows2) * (half / N);
        if (dt == 1) k_rope_vec<bf16><<<ew_grid(items, T256), T256, 0, st>>>((const bf16*)x, cs, sn, (bf16*)o, T_, dh, rows, heads_inner, inverse,
                                                                              (const bf16*)x2, (bf16*)o2, rows2, heads_inner2);
        else k_rope_vec<float><<<ew_grid(items, T256), T256, 0, st>>>((const float*)x, cs, sn, (float*)o, T_, dh, rows, heads_inner, inverse,
                                                                        (const float*)x2, (float*)o2, rows2, heads_inner2);
    } else {
        for (int which = 0; which < (x2 ? 2 : 1); which++) {
            const void* xs = which ? x2 : x; void* os = which ? o2 : o;
            const long long rr = which ? rows2 : rows; const int hi = which ? heads_inner2 : heads_inner;
            const long long items = rr * half;
            if (dt == 1) k_rope<bf16><<<ew_grid(items, T256), T256, 0, st>>>((const bf16*)xs, cs, sn, (bf16*)os, T_, dh, rr, hi, inverse);
            else k_rope<float><<<ew_grid(items, T256), T256, 0, st>>>((const float*)xs, cs, sn, (float*)os, T_, dh, rr, hi, inverse);
        }
    }
    return 0;
}

// ── GQA expand / group-sum (kept for ABI completeness) ──────────────────────
template <typename T>
__global__ void k_repeat_kv(const T* x, T* o, int B, int KV, int H, int T_, int dh) {
    const long long total = (long long)B * H * T_ * dh;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const int rep = H / KV;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int j = (int)(i % dh);
        long long r = i / dh;
        int t = (int)(r % T_); r /= T_;
        int h = (int)(r % H); r /= H;
        o[i] = x[((r * KV + h / rep) * T_ + t) * dh + j];
    }
}
template <typename T>
__global__ void k_repeat_kv_bwd(const T* g, T* o, int B, int KV, int H, int T_, int dh) {
    const long long total = (long long)B * KV * T_ * dh;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const int rep = H / KV;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int j = (int)(i % dh);
        long long r = i / dh;
        int t = (int)(r % T_); r /= T_;
        int kv = (int)(r % KV); r /= KV;
        float acc = 0.f;
        for (int q = 0; q < rep; q++) acc += ldf(g, ((r * H + kv * rep + q) * T_ + t) * dh + j);
        stf(o, i, acc);
    }
}
int ax_repeat_kv(int dt, const void* x, void* o, int B, int KV, int H, int T_, int dh, cudaStream_t st) {
    const long long total = (long long)B * H * T_ * dh;
    if (total <= 0 || KV <= 0) return 0;
    if (dt == 1) k_repeat_kv<bf16><<<ew_grid(total, T256), T256, 0, st>>>((const bf16*)x, (bf16*)o, B, KV, H, T_, dh);
    else k_repeat_kv<float><<<ew_grid(total, T256), T256, 0, st>>>((const float*)x, (float*)o, B, KV, H, T_, dh);
    return 0;
}
int ax_repeat_kv_bwd(int dt, const void* g, void* o, int B, int KV, int H, int T_, int dh, cudaStream_t st) {
    const long long total = (long long)B * KV * T_ * dh;
    if (total <= 0 || KV <= 0) return 0;
    if (dt == 1) k_repeat_kv_bwd<bf16><<<ew_grid(total, T256), T256, 0, st>>>((const bf16*)g, (bf16*)o, B, KV, H, T_, dh);
    else k_repeat_kv_bwd<float><<<ew_grid(total, T256), T256, 0, st>>>((const float*)g, (float*)o, B, KV, H, T_, dh);
    return 0;
}

// ── tiled-attention softmax pair (fp32 / non-flash plans) ───────────────────
// Row r covers query qoff + (r % rpb); keys j <= that are kept.
template <typename T>
__global__ void k_softmax_causal(const T* x, T* o, int rpb, int width, int qoff, long long rows) {
    __shared__ float sh[40];
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        int t = qoff + (int)(r % rpb);
        if (t > width - 1) t = width - 1;
        const T* xr = x + r * width;
        float mx = -1e30f;
        for (int j = threadIdx.x; j <= t; j += blockDim.x) mx = fmaxf(mx, ldf(xr, j));
        mx = block_max(mx, sh);
        float acc = 0.f;
        for (int j = threadIdx.x; j <= t; j += blockDim.x) acc += expf(ldf(xr, j) - mx);
        const float denom = block_sum(acc, sh);
        T* orow = o + r * width;
        for (int j = threadIdx.x; j < width; j += blockDim.x)
            stf(orow, j, (j <= t) ? expf(ldf(xr, j) - mx) / denom : 0.f);
        __syncthreads();
    }
}
template <typename T>
__global__ void k_softmax_bwd(const T* p, const T* dp, T* ds, int width, long long rows) {
    __shared__ float sh[40];
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        float dot = 0.f;
        for (int j = threadIdx.x; j < width; j += blockDim.x) dot += ldf(dp, r * width + j) * ldf(p, r * width + j);
        dot = block_sum(dot, sh);
        for (int j = threadIdx.x; j < width; j += blockDim.x)
            stf(ds, r * width + j, ldf(p, r * width + j) * (ldf(dp, r * width + j) - dot));
        __syncthreads();
    }
}
int ax_softmax_causal(int dt, const void* x, void* o, int rpb, int width, int qoff, long long rows, cudaStream_t st) {
    if (rows <= 0 || width <= 0) return 0;
    const int grid = (int)(rows < 65535LL * 16 ? rows : 65535LL * 16);
    const int thr = width >= 256 ? 256 : (width >= 64 ? 64 : 32);
    if (dt == 1) k_softmax_causal<bf16><<<grid, thr, 0, st>>>((const bf16*)x, (bf16*)o, rpb, width, qoff, rows);
    else k_softmax_causal<float><<<grid, thr, 0, st>>>((const float*)x, (float*)o, rpb, width, qoff, rows);
    return 0;
}
int ax_softmax_bwd(int dt, const void* p, const void* dp, void* ds, int width, long long rows, cudaStream_t st) {
    if (rows <= 0 || width <= 0) return 0;
    const int grid = (int)(rows < 65535LL * 16 ? rows : 65535LL * 16);
    const int thr = width >= 256 ? 256 : (width >= 64 ? 64 : 32);
    if (dt == 1) k_softmax_bwd<bf16><<<grid, thr, 0, st>>>((const bf16*)p, (const bf16*)dp, (bf16*)ds, width, rows);
    else k_softmax_bwd<float><<<grid, thr, 0, st>>>((const float*)p, (const float*)dp, (float*)ds, width, rows);
    return 0;
}

// ── SwiGLU backward: dg = grad*u*silu'(g), du = grad*silu(g) ───────────────
template <typename T>
__global__ void k_silu_bwd(const T* __restrict__ g, const T* __restrict__ u, const T* __restrict__ grad,
                           T* __restrict__ dg, T* __restrict__ du, long long n, int vec) {
    constexpr int N = Vec<T>::N;
    pdl_enter();
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long start = 0;
    if (vec) {
        const long long nv = n / N;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
            float x[N], uu[N], gr[N], a[N], b[N];
            Vec<T>::ld(g + i * N, x);
            Vec<T>::ld(u + i * N, uu);
            Vec<T>::ld(grad + i * N, gr);
#pragma unroll
            for (int j = 0; j < N; j++) {
                const float sig = 1.f / (1.f + exp_t<T>(-x[j]));
                a[j] = gr[j] * uu[j] * (sig * (1.f + x[j] * (1.f - sig)));
                b[j] = gr[j] * (x[j] * sig);
            }
            Vec<T>::st(dg + i * N, a);
            Vec<T>::st(du + i * N, b);
        }
        start = nv * N;
    }
    for (long long i = start + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float x = ldf(g, i), sig = 1.f / (1.f + expf(-x)), gr = ldf(grad, i);
        stf(dg, i, gr * ldf(u, i) * (sig * (1.f + x * (1.f - sig))));
        stf(du, i, gr * (x * sig));
    }
}
int ax_silu_bwd(int dt, const void* g, const void* u, const void* grad, void* dg, void* du, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const int vec = aligned16(g) && aligned16(u) && aligned16(grad) && aligned16(dg) && aligned16(du);
    if (dt == 1) ax_launch_chain(k_silu_bwd<bf16>, dim3(ew_grid(n / 8 + 1, T256)), dim3(T256), 0, st, (const bf16*)g, (const bf16*)u, (const bf16*)grad, (bf16*)dg, (bf16*)du, n, vec);
    else k_silu_bwd<float><<<ew_grid(n / 4 + 1, T256), T256, 0, st>>>((const float*)g, (const float*)u, (const float*)grad, (float*)dg, (float*)du, n, vec);
    return 0;
}

// ── row dot: c[r] = sum_d a[r,d] * b[r,d], one warp per row ────────────────
template <typename T>
__global__ void k_rowdot(const T* a, const T* b, float* c, long long rows, int dim) {
    const int lane = threadIdx.x & 31;
    const long long wstride = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += wstride) {
        float acc = 0.f;
        for (int d = lane; d < dim; d += 32) acc += ldf(a, r * dim + d) * ldf(b, r * dim + d);
        acc = warp_sum(acc);
        if (!lane) c[r] = acc;
    }
}
int ax_rowdot(int dt, const void* a, const void* b, float* c, long long rows, int dim, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (dt >= 1) k_rowdot<bf16><<<ew_grid(rows * 32, T256), T256, 0, st>>>((const bf16*)a, (const bf16*)b, c, rows, dim);
    else k_rowdot<float><<<ew_grid(rows * 32, T256), T256, 0, st>>>((const float*)a, (const float*)b, c, rows, dim);
    return 0;
}
