// C ABI of the W4A4 GEMMs: argument validation and the choice of kernel by shape (weight-streaming
// mma.sync kernel for the decode regime, the CTA-pair tcgen05 kernel above it and for MoE prefill).
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include <cstdlib>
#include <cstring>

namespace sr {

// Kernel choice by shape.  The weight-streaming kernel's mma.sync rate bounds it at about 32 rows.  With 33 .. 64 rows
// it runs two CTAs per SM, one block of 16 weight rows each, and still wins while all blocks are one round of the grid
// (measured at 64 rows, K = 4096: N = 4096 11.6 us against 15.0 us on the tensor-core kernel; N = 5120, two rounds,
// 20.3 against 15.6 us).
static bool decode_regime(int64_t M, int64_t N) { return M <= 32 || (M <= 64 && N <= 32ll * current_sm_count()); }

// |a * b| <= 64 for signed codes and <= 120 for unsigned activation codes; the tensor-core kernel carries every product
// times 256 in its int32 accumulator, so K is bounded by 2^31 / (256 * 64) resp. 2^31 / (256 * 120).
static int64_t max_k(bool a_unsigned) { return a_unsigned ? 65536 : 131040; }

static int run_gemm(const void *A, const void *B, int64_t M, int64_t N, int64_t K, int a_unsigned,
                    const Epilogue &ep, void *stream, const char *who, void *ws = nullptr, int64_t ws_bytes = 0,
                    void *split_cnt = nullptr) {
    SR_REQUIRE(M >= 0 && N >= 0 && K >= 0, SR_ERR_INVALID, "%s: negative size", who);
    SR_REQUIRE(K % 32 == 0, SR_ERR_INVALID, "%s: A.shape[-1]: %lld must be multiplication of 32", who, (long long)K);
    if (M == 0 || N == 0) return SR_OK;
    SR_REQUIRE(K > 0, SR_ERR_INVALID, "%s: K must be positive", who);
    SR_REQUIRE(A && B, SR_ERR_INVALID, "%s: null pointer", who);
    SR_REQUIRE(M < (1ll << 31) && N < (1ll << 31), SR_ERR_UNSUPPORTED, "%s: size out of range", who);
    SR_REQUIRE(K <= max_k(a_unsigned != 0), SR_ERR_UNSUPPORTED, "%s: K = %lld exceeds %lld (int32 accumulator range)", who,
               (long long)K, (long long)max_k(a_unsigned != 0));
    SR_REQUIRE(aligned16(A) && aligned16(B), SR_ERR_INVALID, "%s: operands must be 16-byte aligned", who);
    if (decode_regime(M, N))
        return launch_gemm_skinny((const uint8_t *)A, (const uint8_t *)B, M, N, K, a_unsigned != 0, ep, as_stream(stream));
    return launch_gemm_tc3((const uint8_t *)A, (const uint8_t *)B, M, N, K, a_unsigned != 0, ep, as_stream(stream),
                           (int32_t *)ws, ws_bytes, (int32_t *)split_cnt);
}

}  // namespace sr

using namespace sr;

extern "C" {

int sr_matmul_i4(const void *A, const void *B, int64_t M, int64_t N, int64_t K, int a_unsigned, void *C,
                 void *stream) {
    SR_REQUIRE(M == 0 || N == 0 || C != nullptr, SR_ERR_INVALID, "matmul: null output");
    Epilogue ep = {};
    ep.mode = 0;
    ep.c = (int32_t *)C;
    ep.ldc = N;
    return run_gemm(A, B, M, N, K, a_unsigned, ep, stream, "matmul");
}

int sr_matmul_i4_ld(const void *A, int64_t lda_bytes, const void *B, int64_t M, int64_t N, int64_t K, int a_unsigned,
                    void *C, void *stream) {
    SR_REQUIRE(M == 0 || N == 0 || C != nullptr, SR_ERR_INVALID, "matmul: null output");
    SR_REQUIRE(lda_bytes >= K / 2 && lda_bytes % 16 == 0 && lda_bytes < (1ll << 31), SR_ERR_INVALID,
               "matmul: row stride of %lld bytes for rows of %lld packed bytes (must cover a row and be a multiple of 16)",
               (long long)lda_bytes, (long long)(K / 2));
    Epilogue ep = {};
    ep.mode = 0;
    ep.c = (int32_t *)C;
    ep.ldc = N;
    ep.lda = (uint32_t)lda_bytes;
    return run_gemm(A, B, M, N, K, a_unsigned, ep, stream, "matmul");
}

int sr_w4a4_linear(const void *A, const void *a_scale, const void *a_zero, const void *W, const void *w_scale,
                   const void *w_sum, const void *bias, int64_t M, int64_t N, int64_t K, void *out, void *stream) {
    SR_REQUIRE(M == 0 || N == 0 || (out && a_scale && w_scale), SR_ERR_INVALID, "w4a4_linear: null pointer");
    SR_REQUIRE(a_zero == nullptr || w_sum != nullptr, SR_ERR_INVALID,
               "w4a4_linear: asymmetric activations need the int4 row sums of the weight");
    Epilogue ep = {};
    ep.mode = 1;
    ep.out = (__half *)out;
    ep.a_scale = (const __half *)a_scale;
    ep.w_scale = (const __half *)w_scale;
    ep.a_zero = (const int8_t *)a_zero;
    ep.w_sum = a_zero ? (const int32_t *)w_sum : nullptr;
    ep.bias = (const __half *)bias;
    return run_gemm(A, W, M, N, K, a_zero != nullptr, ep, stream, "w4a4_linear");
}

int sr_w4a4_linear_ws_bytes(int64_t M, int64_t N, int64_t K, int64_t *bytes) {
    SR_REQUIRE(bytes != nullptr, SR_ERR_INVALID, "w4a4_linear_ws_bytes: null pointer");
    *bytes = (M <= 0 || N <= 0 || K <= 0 || decode_regime(M, N)) ? 0 : gemm_tc3_splitk_bytes(M, N, K);
    return SR_OK;
}

int sr_w4a4_linear_ws(const void *A, const void *a_scale, const void *a_zero, const void *W, const void *w_scale,
                      const void *w_sum, const void *bias, int64_t M, int64_t N, int64_t K, void *out, void *ws,
                      int64_t ws_bytes, void *counters, void *stream) {
    SR_REQUIRE(M == 0 || N == 0 || (out && a_scale && w_scale), SR_ERR_INVALID, "w4a4_linear: null pointer");
    SR_REQUIRE(a_zero == nullptr || w_sum != nullptr, SR_ERR_INVALID,
               "w4a4_linear: asymmetric activations need the int4 row sums of the weight");
    SR_REQUIRE(ws_bytes >= 0 && (ws_bytes == 0 || (ws && counters)), SR_ERR_INVALID, "w4a4_linear: workspace without counters");
    Epilogue ep = {};
    ep.mode = 1;
    ep.out = (__half *)out;
    ep.a_scale = (const __half *)a_scale;
    ep.w_scale = (const __half *)w_scale;
    ep.a_zero = (const int8_t *)a_zero;
    ep.w_sum = a_zero ? (const int32_t *)w_sum : nullptr;
    ep.bias = (const __half *)bias;
    return run_gemm(A, W, M, N, K, a_zero != nullptr, ep, stream, "w4a4_linear", ws, ws_bytes, counters);
}

int sr_w4a4_swiglu(const void *A, const void *a_scale, const void *a_zero, const void *W, const void *w_scale,
                   const void *w_sum, const void *bias, int64_t M, int64_t N, int64_t K, void *out, void *stream) {
    SR_REQUIRE(M >= 0 && N >= 0 && K >= 0, SR_ERR_INVALID, "w4a4_swiglu: negative size");
    if (M == 0 || N == 0) return SR_OK;
    SR_REQUIRE(out && A && W && a_scale && w_scale, SR_ERR_INVALID, "w4a4_swiglu: null pointer");
    SR_REQUIRE(a_zero == nullptr || w_sum != nullptr, SR_ERR_INVALID,
               "w4a4_swiglu: asymmetric activations need the int4 row sums of the weight");
    SR_REQUIRE(K > 0 && 2 * N < (1ll << 31), SR_ERR_INVALID, "w4a4_swiglu: size out of range");
    Epilogue ep = {};
    ep.mode = 1;
    ep.out = (__half *)out;
    ep.a_scale = (const __half *)a_scale;
    ep.w_scale = (const __half *)w_scale;
    ep.a_zero = (const int8_t *)a_zero;
    ep.w_sum = a_zero ? (const int32_t *)w_sum : nullptr;
    ep.bias = (const __half *)bias;
    return launch_gemm_skinny_swiglu((const uint8_t *)A, (const uint8_t *)W, M, N, K, a_zero != nullptr, ep,
                                     as_stream(stream));
}

int sr_grouped_linear(const void *A, const void *a_scale, const void *a_zero, const void *expert_ids,
                      const void *row_offsets, const void *W, const void *w_scale, const void *w_sum, int64_t rows,
                      int64_t num_experts, int64_t N, int64_t K, int64_t expected_rows, void *out, void *stream) {
    SR_REQUIRE(rows >= 0 && N >= 0 && K >= 0 && num_experts >= 1, SR_ERR_INVALID, "grouped_linear: bad size");
    if (rows == 0 || N == 0) return SR_OK;
    SR_REQUIRE(K > 0 && K % 32 == 0, SR_ERR_INVALID, "grouped_linear: K = %lld must be a positive multiple of 32",
               (long long)K);
    SR_REQUIRE(A && W && out && a_scale && w_scale && expert_ids && row_offsets, SR_ERR_INVALID,
               "grouped_linear: null pointer");
    SR_REQUIRE(a_zero == nullptr || w_sum != nullptr, SR_ERR_INVALID,
               "grouped_linear: asymmetric activations need the int4 row sums of the weights");
    SR_REQUIRE(K <= max_k(a_zero != nullptr), SR_ERR_UNSUPPORTED, "grouped_linear: K = %lld exceeds %lld (int32 accumulator range)",
               (long long)K, (long long)max_k(a_zero != nullptr));
    Epilogue ep = {};
    ep.mode = 1;
    ep.out = (__half *)out;
    ep.a_scale = (const __half *)a_scale;
    ep.w_scale = (const __half *)w_scale;
    ep.a_zero = (const int8_t *)a_zero;
    ep.w_sum = a_zero ? (const int32_t *)w_sum : nullptr;
    ep.expert_ids = (const int32_t *)expert_ids;
    // few rows per expert (decode): the weight-streaming kernel; otherwise the CTA-pair tensor-core kernel
    const int64_t covered = expected_rows > 0 && expected_rows < rows ? expected_rows : rows;
    if (covered <= 16 * num_experts)
        return launch_gemm_skinny_grouped((const uint8_t *)A, (const uint8_t *)W, rows, N, K, a_zero != nullptr, ep,
                                          (const int32_t *)row_offsets, (int)num_experts, as_stream(stream));
    return launch_gemm_tc3_grouped((const uint8_t *)A, (const uint8_t *)W, rows, N, K, a_zero != nullptr, ep,
                                   (const int32_t *)row_offsets, (int)num_experts, as_stream(stream));
}

}  // extern "C"
