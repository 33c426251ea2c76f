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
    uint32_t lda;            // bytes between rows of A; 0 = K / 2 (dense).  A may be a column range of a wider code matrix

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

// int32 -> fp32 without the conversion pipe: exact for |x| < 2^22 (magic-number add on the
// integer and floating-point pipes); larger magnitudes take the ordinary conversion.
__device__ __forceinline__ float int_to_float_fast(int x, bool small) {
    return small ? (__int_as_float(0x4B400000 + x) - 12582912.f) : (float)x;
}

// Stores one lane's 32 consecutive accumulator columns (values still carry the factor 256).
// `small` = every |acc >> 8| of this problem is below 2^22.
__device__ __forceinline__ void store_acc_chunk(const Epilogue &ep, uint32_t row, uint32_t col0, const int (&v)[32],
                                                uint32_t M, uint32_t N, bool small) {
    if (row >= M || col0 >= N) return;
    const bool full = (col0 + 32 <= N);
    if (ep.mode == 0) {
        int32_t *dst = ep.c + (size_t)row * ep.ldc + col0;
        if (full && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<int4 *>(dst + j) = make_int4(v[j] >> 8, v[j + 1] >> 8, v[j + 2] >> 8, v[j + 3] >> 8);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < N) dst[j] = v[j] >> 8;
        }
        return;
    }
    __half *dst = ep.out + (size_t)row * N + col0;
    const size_t e = ep.expert_ids ? (size_t)ep.expert_ids[row] * N : 0;
    const __half *ws = ep.w_scale + e + col0;
    const bool vec = full && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0 && (reinterpret_cast<uintptr_t>(ws) & 15u) == 0 &&
                     !ep.a_zero && !ep.bias;
    if (vec) {
        const float sr_ = __half2float(ep.a_scale[row]);
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            Vec16 s, o;
            s.u = __ldg(reinterpret_cast<const uint4 *>(ws + j));
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float2 sc = __half22float2(s.h2[t]);
                const float a = (int_to_float_fast(v[j + 2 * t] >> 8, small) * sr_) * sc.x;
                const float b = (int_to_float_fast(v[j + 2 * t + 1] >> 8, small) * sr_) * sc.y;
                o.h2[t] = __floats2half2_rn(a, b);
            }
            *reinterpret_cast<uint4 *>(dst + j) = o.u;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < N) dst[j] = ep.dequant(row, col0 + j, v[j] >> 8, N);
    }
}

// Warp-collective variant of the dequant path for the tcgen05 epilogues: lane l holds 32 consecutive columns
// of row row0 + l.  When the plain symmetric case applies to the whole chunk (uniform across the warp), the 64
// output bytes of every row go through a 32 x 80-byte staging area in shared memory and leave as 64-byte runs,
// four lanes per row: whole 32-byte sectors instead of the half sectors a lane-per-row store writes.
// `stage` = 2560 bytes private to the warp.  Falls back to store_acc_chunk otherwise.
__device__ __forceinline__ void store_acc_chunk_warp(const Epilogue &ep, uint32_t row0, int lane, uint32_t col0,
                                                     const int (&v)[32], uint32_t row_end, uint32_t N, bool small,
                                                     uint8_t *stage) {
    if (row0 >= row_end) return;   // warp-uniform: none of the 32 rows exists
    const uint32_t row = row0 + lane;
    bool vec = false;
    if (ep.mode == 1 && col0 + 32 <= N && !ep.a_zero && !ep.bias) {
        const size_t e = ep.expert_ids ? (size_t)ep.expert_ids[row < row_end ? row : row0] * N : 0;
        const __half *ws = ep.w_scale + e + col0;
        vec = ((reinterpret_cast<uintptr_t>(ep.out + (size_t)row0 * N + col0) | reinterpret_cast<uintptr_t>(ws) |
                (uintptr_t)(N * 2)) & 15u) == 0;
        vec = __all_sync(0xffffffffu, vec);
        if (vec) {
            const float sr_ = row < row_end ? __half2float(ep.a_scale[row]) : 0.f;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                Vec16 s, o;
                s.u = __ldg(reinterpret_cast<const uint4 *>(ws + j));
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float2 sc = __half22float2(s.h2[t]);
                    const float a = (int_to_float_fast(v[j + 2 * t] >> 8, small) * sr_) * sc.x;
                    const float b = (int_to_float_fast(v[j + 2 * t + 1] >> 8, small) * sr_) * sc.y;
                    o.h2[t] = __floats2half2_rn(a, b);
                }
                *reinterpret_cast<uint4 *>(stage + lane * 80 + j * 2) = o.u;
            }
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int r = it * 8 + (lane >> 2), piece = lane & 3;
                const uint4 val = *reinterpret_cast<const uint4 *>(stage + r * 80 + piece * 16);
                if (row0 + r < row_end)
                    *reinterpret_cast<uint4 *>(ep.out + (size_t)(row0 + r) * N + col0 + piece * 8) = val;
            }
            __syncwarp();
        }
    }
    if (!vec) store_acc_chunk(ep, row, col0, v, row_end, N, small);
}

int launch_gemm_skinny(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                       const Epilogue &ep, cudaStream_t st);
int launch_gemm_skinny_swiglu(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                              const Epilogue &ep, cudaStream_t st);
int launch_gemm_skinny_grouped(const uint8_t *A, const uint8_t *B, int64_t rows, int64_t N, int64_t K, bool a_unsigned,
                               const Epilogue &ep, const int32_t *row_off, int num_experts, cudaStream_t st);
// ws / ws_bytes / split_cnt: optional split-K workspace (gemm_tc3_splitk_bytes) and its zeroed, self-resetting counters
int launch_gemm_tc3(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                    const Epilogue &ep, cudaStream_t st, int32_t *ws = nullptr, int64_t ws_bytes = 0,
                    int32_t *split_cnt = nullptr);
int64_t gemm_tc3_splitk_bytes(int64_t M, int64_t N, int64_t K);   // 0: the launch would not split K
int launch_gemm_tc3_grouped(const uint8_t *A, const uint8_t *B, int64_t rows, int64_t N, int64_t K, bool a_unsigned,
                            const Epilogue &ep, const int32_t *row_off, int num_experts, cudaStream_t st);
int launch_gemm_tc3_ptr_array(const int32_t *sizes, int64_t P, const int64_t *ptr_a, const int64_t *ptr_b,
                              const int64_t *ptr_c, const int64_t *lda, const int64_t *ldb, const int64_t *ldc,
                              bool a_unsigned, int64_t k_limit, const int32_t **use_tc_flag, cudaStream_t st);

}  // namespace sr
