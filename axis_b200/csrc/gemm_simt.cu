// General GEMM on CUDA cores: true fp32 FMA accumulation, any shape, stride or
// alignment, fp32 or bf16 operands and output, strided-batched.  It serves the
// fp32 parity mode and every shape the tensor-core path does not take.
//
//   C[b][i,j] = alpha * sum_k A(i,k) * B(k,j) + beta * D[b][i,j]
//   tb = 0: A [m,k] row-major, B [k,n] row-major
//   tb = 1: A [m,k] row-major, B [n,k] row-major (C = A B^T)
//   tb = 2: A [k,m] row-major, B [k,n] row-major (C = A^T B)
#include "common.cuh"
#include "kernels.h"

#define GT 64      // C tile edge
#define GK 16      // k step

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
k_gemm_simt(const TI* __restrict__ A, const TI* __restrict__ B, TO* C, const TO* D,
            int m, int n, int k, long long as_m, long long as_k, long long bs_k, long long bs_n,
            long long sa, long long sb, long long sc, float alpha, float beta) {
    __shared__ float As[GK][GT + 4];
    __shared__ float Bs[GK][GT + 4];
    const int bz = blockIdx.z;
    A += (long long)bz * sa;
    B += (long long)bz * sb;
    C += (long long)bz * sc;
    if (D) D += (long long)bz * sc;
    const int i0 = blockIdx.y * GT, j0 = blockIdx.x * GT;
    const int tid = threadIdx.x;
    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] = 0.f;

    const bool a_kfast = as_k == 1;      // consecutive threads along k when k is contiguous
    const bool b_nfast = bs_n == 1;
    for (int k0 = 0; k0 < k; k0 += GK) {
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const int e = tid + l * 256;                 // 0..1023
            int ii, kk;
            if (a_kfast) { kk = e & (GK - 1); ii = e >> 4; } else { ii = e & (GT - 1); kk = e >> 6; }
            const int gi = i0 + ii, gk = k0 + kk;
            As[kk][ii] = (gi < m && gk < k) ? ldf(A, gi * as_m + gk * as_k) : 0.f;
            int jj, k2;
            if (b_nfast) { jj = e & (GT - 1); k2 = e >> 6; } else { k2 = e & (GK - 1); jj = e >> 4; }
            const int gj = j0 + jj, gk2 = k0 + k2;
            Bs[k2][jj] = (gj < n && gk2 < k) ? ldf(B, gk2 * bs_k + gj * bs_n) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int q = 0; q < 4; q++) { a[q] = As[kk][ty * 4 + q]; b[q] = Bs[kk][tx * 4 + q]; }
#pragma unroll
            for (int p = 0; p < 4; p++)
#pragma unroll
                for (int q = 0; q < 4; q++) acc[p][q] = fmaf(a[p], b[q], acc[p][q]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const int gi = i0 + ty * 4 + p;
        if (gi >= m) continue;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int gj = j0 + tx * 4 + q;
            if (gj >= n) continue;
            const long long idx = (long long)gi * n + gj;
            float r = alpha * acc[p][q];
            if (beta != 0.f) r += beta * ldf(D, idx);
            stf(C, idx, r);
        }
    }
}

int ax_gemm_simt(int in_bf16, int out_bf16, int tb, const void* A, const void* B, void* C, const void* D,
                 int m, int n, int k, int batch, long long sa, long long sb, long long sc,
                 float alpha, float beta, cudaStream_t st) {
    if (m <= 0 || n <= 0) return 0;
    if (batch < 1) batch = 1;
    long long as_m, as_k, bs_k, bs_n;
    if (tb == 0) { as_m = k; as_k = 1; bs_k = n; bs_n = 1; }
    else if (tb == 1) { as_m = k; as_k = 1; bs_k = 1; bs_n = k; }
    else { as_m = 1; as_k = m; bs_k = n; bs_n = 1; }
    if (beta != 0.f && !D) D = C;
    dim3 grid((n + GT - 1) / GT, (m + GT - 1) / GT, batch);
    if (grid.y > 65535 || grid.z > 65535) return 123;
    if (in_bf16 && out_bf16)
        k_gemm_simt<bf16, bf16><<<grid, 256, 0, st>>>((const bf16*)A, (const bf16*)B, (bf16*)C, (const bf16*)D, m, n, k, as_m, as_k, bs_k, bs_n, sa, sb, sc, alpha, beta);
    else if (in_bf16)
        k_gemm_simt<bf16, float><<<grid, 256, 0, st>>>((const bf16*)A, (const bf16*)B, (float*)C, (const float*)D, m, n, k, as_m, as_k, bs_k, bs_n, sa, sb, sc, alpha, beta);
    else if (!out_bf16)
        k_gemm_simt<float, float><<<grid, 256, 0, st>>>((const float*)A, (const float*)B, (float*)C, (const float*)D, m, n, k, as_m, as_k, bs_k, bs_n, sa, sb, sc, alpha, beta);
    else
        return 124;
    return 0;
}
