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

}  // namespace sr
