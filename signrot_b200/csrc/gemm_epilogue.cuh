// Epilogue shared by the int4 GEMM kernels.
//
// mode 0: store the exact int32 accumulator (what signrot/kernels/gemm.cu returns).
// mode 1: the dequant chain of Linear4bit.forward (signrot/nn/linear.py:36-50) fused
//         into the GEMM, so the int32 [M,N] matrix never goes to HBM:
//           acc -= int32(zero[row]) * wsum[col]                 (asym only; nn/linear.py:39-43)
//           out  = rn_h((float(acc) * s_row[row]) * s_col[col]) (kernels/quant.cu:84-87)
//           out  = rn_h(out + bias[col])                        (nn/linear.py:47-48)
//         With expert_ids, the per-column tables are [E, N] and indexed by
//         expert_ids[row] (signrot/kernels/moe.cu:216-225).
#pragma once
#include "common.cuh"

namespace sr {

struct Epilogue {
    int mode;
    int32_t *c;              // mode 0: [M, ldc]
    int64_t ldc;
    __half *out;             // mode 1: [M, N]
    const __half *a_scale;   // [M]
    const __half *w_scale;   // [N] or [E, N]
    const int8_t *a_zero;    // [M] or null
    const int32_t *w_sum;    // [N] or [E, N], required when a_zero is set
    const __half *bias;      // [N] or null
    const int32_t *expert_ids;  // [M] or null

    __device__ __forceinline__ __half dequant(uint32_t row, uint32_t col, int acc, uint32_t N) const {
        const size_t e = expert_ids ? (size_t)expert_ids[row] * N : 0;
        if (a_zero) acc -= (int)a_zero[row] * w_sum[e + col];
        __half o = __float2half_rn(((float)acc * __half2float(a_scale[row])) * __half2float(w_scale[e + col]));
        if (bias) o = __float2half_rn(__half2float(o) + __half2float(bias[col]));
        return o;
    }

    __device__ __forceinline__ void store(uint32_t row, uint32_t col, int acc, uint32_t N) const {
        if (mode == 0) c[(size_t)row * ldc + col] = acc;
        else out[(size_t)row * N + col] = dequant(row, col, acc, N);
    }
};

int launch_gemm_small(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                      const Epilogue &ep, cudaStream_t st);
int launch_gemm_tc(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                   const Epilogue &ep, cudaStream_t st);

}  // namespace sr
