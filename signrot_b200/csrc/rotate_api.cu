// C ABI of the online rotation: argument checks and kernel selection.
#include "rotate.cuh"

namespace sr {

static bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }

static int dtype_ok(int d) { return d == SR_F16 || d == SR_BF16 || d == SR_F32; }

static int run_rotate(RotateArgs &a, void *stream, const char *who) {
    if (a.rows == 0 || a.n == 0) return SR_OK;
    cudaStream_t st = as_stream(stream);
    int rc = launch_rotate_fast(a, st);
    if (rc != SR_ERR_UNSUPPORTED) return rc;
    return launch_rotate_generic(a, st);
}

}  // namespace sr

using namespace sr;

extern "C" {

int sr_hadamard(const void *x, int dtype, int64_t rows, int64_t n, const void *hadk, int64_t K, float scale,
                const void *sign, int fp32_mode, void *out, int out_dtype, void *stream) {
    SR_REQUIRE(rows >= 0 && n >= 0 && K >= 1, SR_ERR_INVALID, "hadamard: bad size");
    SR_REQUIRE(dtype_ok(dtype) && dtype_ok(out_dtype), SR_ERR_INVALID, "hadamard: unknown dtype");
    if (rows == 0 || n == 0) return SR_OK;
    SR_REQUIRE(n % K == 0 && is_pow2(n / K), SR_ERR_INVALID,
               "hadamard: n = %lld must be K = %lld times a power of two", (long long)n, (long long)K);
    SR_REQUIRE(K == 1 || hadk != nullptr, SR_ERR_INVALID, "hadamard: K > 1 needs the K x K matrix");
    SR_REQUIRE(x && out, SR_ERR_INVALID, "hadamard: null pointer");
    SR_REQUIRE(rows < (1ll << 31) && n <= 65536, SR_ERR_UNSUPPORTED, "hadamard: size out of range");
    RotateArgs a = {};
    a.x = x; a.hadk = hadk; a.sign = (const int8_t *)sign; a.out = out;
    a.rows = (uint32_t)rows; a.n = (uint32_t)n; a.K = (uint32_t)K; a.S = (uint32_t)(n / K); a.stride = 1;
    a.scale = scale; a.clip = 1.f; a.in_dtype = dtype; a.out_dtype = out_dtype; a.fp32_mode = fp32_mode;
    return run_rotate(a, stream, "hadamard");
}

int sr_hadamard_heads(const void *x, int dtype, int64_t rows, int64_t heads, int64_t head_dim, float scale,
                      int fp32_mode, void *out, int out_dtype, void *stream) {
    SR_REQUIRE(rows >= 0 && heads >= 1 && head_dim >= 1, SR_ERR_INVALID, "hadamard_heads: bad size");
    SR_REQUIRE(dtype_ok(dtype) && dtype_ok(out_dtype), SR_ERR_INVALID, "hadamard_heads: unknown dtype");
    SR_REQUIRE(is_pow2(heads), SR_ERR_UNSUPPORTED, "hadamard_heads: the number of heads must be a power of two");
    if (rows == 0) return SR_OK;
    SR_REQUIRE(x && out, SR_ERR_INVALID, "hadamard_heads: null pointer");
    SR_REQUIRE(rows < (1ll << 31) && heads * head_dim <= 65536, SR_ERR_UNSUPPORTED, "hadamard_heads: size out of range");
    RotateArgs a = {};
    a.x = x; a.out = out;
    a.rows = (uint32_t)rows; a.n = (uint32_t)(heads * head_dim); a.K = 1; a.S = (uint32_t)heads;
    a.stride = (uint32_t)head_dim;
    a.scale = scale; a.clip = 1.f; a.in_dtype = dtype; a.out_dtype = out_dtype; a.fp32_mode = fp32_mode;
    return run_rotate(a, stream, "hadamard_heads");
}

int sr_rotate_quant(const void *x, int dtype, int64_t rows, int64_t n, const void *hadk, int64_t K, float scale,
                    const void *sign, const void *expert_ids, int64_t heads, float clip_ratio, int asym, void *q,
                    void *q_scale, void *q_zero, void *rotated, void *stream) {
    SR_REQUIRE(rows >= 0 && n >= 0 && K >= 1 && heads >= 0, SR_ERR_INVALID, "rotate_quant: bad size");
    SR_REQUIRE(dtype == SR_F16 || dtype == SR_BF16, SR_ERR_INVALID, "rotate_quant: activations must be fp16 or bf16");
    if (rows == 0 || n == 0) return SR_OK;
    SR_REQUIRE(n % 8 == 0, SR_ERR_INVALID, "rotate_quant: n must be a multiple of 8");
    SR_REQUIRE(x && q && q_scale && (!asym || q_zero), SR_ERR_INVALID, "rotate_quant: null pointer");
    SR_REQUIRE(rows < (1ll << 31) && n <= 65536, SR_ERR_UNSUPPORTED, "rotate_quant: size out of range");
    RotateArgs a = {};
    a.x = x; a.hadk = hadk; a.sign = (const int8_t *)sign; a.expert_ids = (const int32_t *)expert_ids;
    a.out = rotated; a.q = (uint8_t *)q; a.q_scale = (__half *)q_scale; a.q_zero = (__half *)q_zero;
    a.rows = (uint32_t)rows; a.n = (uint32_t)n; a.scale = scale; a.clip = clip_ratio;
    a.in_dtype = dtype; a.out_dtype = SR_F16; a.cast_in_to_f16 = 1; a.asym = asym;
    if (heads > 0) {
        // head-wise transform (H_heads (x) I_head_dim), the o_proj input rotation
        SR_REQUIRE(K == 1 && is_pow2(heads) && n % heads == 0, SR_ERR_UNSUPPORTED,
                   "rotate_quant: head-wise rotation needs a power-of-two head count dividing n");
        a.K = 1; a.S = (uint32_t)heads; a.stride = (uint32_t)(n / heads);
    } else {
        SR_REQUIRE(n % K == 0 && is_pow2(n / K), SR_ERR_INVALID,
                   "rotate_quant: n = %lld must be K = %lld times a power of two", (long long)n, (long long)K);
        SR_REQUIRE(K == 1 || hadk != nullptr, SR_ERR_INVALID, "rotate_quant: K > 1 needs the K x K matrix");
        a.K = (uint32_t)K; a.S = (uint32_t)(n / K); a.stride = 1;
    }
    return run_rotate(a, stream, "rotate_quant");
}

}  // extern "C"
