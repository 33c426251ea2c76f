// Internal interface between the rotation kernels and their C ABI.
#pragma once
#include "common.cuh"

namespace sr {

struct RotateArgs {
    const void *x;              // [rows, n] in_dtype
    const void *hadk;           // [K, K] fp16 (fp32 in fp32 mode); null when K == 1
    const int8_t *sign;         // [n] or [E, n] of +-1; may be null
    const int32_t *expert_ids;  // [rows] or null: row r uses sign[expert_ids[r]]
    void *out;                  // rotated rows in out_dtype; may be null
    uint8_t *q;                 // packed codes [rows, n/2]; may be null
    __half *q_scale;            // [rows]
    __half *q_zero;             // [rows] (asym only)
    uint32_t rows, n, S, K, stride;
    float scale;                // multiplies the Walsh-Hadamard sums (1/sqrt(n))
    float clip;
    int in_dtype, out_dtype;    // SR_F16 / SR_BF16 / SR_F32
    int fp32_mode;              // no intermediate rounding (OnlineHadamard force_fp32)
    int cast_in_to_f16;         // bf16 input is first rounded to fp16 (the reference's x.to(float16))
    int asym;
};

int launch_rotate_generic(const RotateArgs &a, cudaStream_t st);
// Returns SR_OK when a specialised kernel took the call, SR_ERR_UNSUPPORTED when the
// shape has none (the caller then uses the generic kernel).
int launch_rotate_fast(const RotateArgs &a, cudaStream_t st);
int launch_rotate_had28(const RotateArgs &a, cudaStream_t st);
int launch_rotate_tc4096(const RotateArgs &a, cudaStream_t st);   // tensor-core transform (mma.sync), rows of 4096
int launch_rotate_umma4096(const RotateArgs &a, cudaStream_t st); // tcgen05 + TMA, rows of 4096, symmetric codes
int launch_rotate_had28_umma(const RotateArgs &a, cudaStream_t st); // tcgen05 + TMA, rows of 14336, symmetric codes
int launch_rotate_heads32(const RotateArgs &a, cudaStream_t st);  // head-wise H32 (x) I128 on the tensor cores

// ---- packed fp32 arithmetic on register pairs (add.f32x2 / sub.f32x2 / mul.f32x2, sm_100)
typedef unsigned long long u64;

__device__ __forceinline__ u64 pack2(float lo, float hi) {
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(u64 v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ u64 add2(u64 a, u64 b) {
    u64 r;
    asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ u64 sub2(u64 a, u64 b) {
    u64 r;
    asm("sub.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
    u64 r;
    asm("mul.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// Walsh-Hadamard transform of 2*NP values held as NP register pairs: one stage inside the
// pairs, then stages between pairs at distances 1 .. HMAX/2 (HMAX = NP for a full transform).
template <int NP, int HMAX>
__device__ __forceinline__ void fwht_pairs(u64 (&v)[NP]) {
#pragma unroll
    for (int a = 0; a < NP; ++a) {
        float lo, hi;
        unpack2(v[a], lo, hi);
        v[a] = pack2(lo + hi, lo - hi);
    }
#pragma unroll
    for (int h = 1; h < HMAX; h <<= 1) {
#pragma unroll
        for (int a = 0; a < NP; ++a) {
            if ((a & h) == 0) {
                const u64 x = v[a], y = v[a + h];
                v[a] = add2(x, y);
                v[a + h] = sub2(x, y);
            }
        }
    }
}

}  // namespace sr
