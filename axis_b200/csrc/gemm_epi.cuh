// GEMM epilogue helper shared by the tcgen05 GEMM kernels: one thread owns 32
// consecutive fp32 accumulator columns of one output row and writes
// alpha * acc + beta * addend, as 16-byte stores when alignment allows.
#pragma once
#include "common.cuh"

template <typename TO> __device__ __forceinline__ void epi_store(TO* crow, const TO* drow, const uint32_t* acc, int col0,
                                                                  int ncols_valid, float alpha, float beta, bool vec_ok);
template <> __device__ __forceinline__ void epi_store<bf16>(bf16* crow, const bf16* drow, const uint32_t* acc, int col0,
                                                            int nvalid, float alpha, float beta, bool vec_ok) {
    if (vec_ok && nvalid >= 32) {
#pragma unroll
        for (int v = 0; v < 4; v++) {
            float f[8];
#pragma unroll
            for (int q = 0; q < 8; q++) f[q] = alpha * __uint_as_float(acc[v * 8 + q]);
            if (drow) {
                float d[8];
                Vec<bf16>::ld(drow + col0 + v * 8, d);
#pragma unroll
                for (int q = 0; q < 8; q++) f[q] += beta * d[q];
            }
            Vec<bf16>::st(crow + col0 + v * 8, f);
        }
    } else {
        for (int q = 0; q < 32 && q < nvalid; q++) {
            float f = alpha * __uint_as_float(acc[q]);
            if (drow) f += beta * __bfloat162float(drow[col0 + q]);
            crow[col0 + q] = __float2bfloat16(f);
        }
    }
}
template <> __device__ __forceinline__ void epi_store<float>(float* crow, const float* drow, const uint32_t* acc, int col0,
                                                             int nvalid, float alpha, float beta, bool vec_ok) {
    if (vec_ok && nvalid >= 32) {
#pragma unroll
        for (int v = 0; v < 8; v++) {
            float f[4];
#pragma unroll
            for (int q = 0; q < 4; q++) f[q] = alpha * __uint_as_float(acc[v * 4 + q]);
            if (drow) {
                float d[4];
                Vec<float>::ld(drow + col0 + v * 4, d);
#pragma unroll
                for (int q = 0; q < 4; q++) f[q] += beta * d[q];
            }
            Vec<float>::st(crow + col0 + v * 4, f);
        }
    } else {
        for (int q = 0; q < 32 && q < nvalid; q++) {
            float f = alpha * __uint_as_float(acc[q]);
            if (drow) f += beta * drow[col0 + q];
            crow[col0 + q] = f;
        }
    }
}

