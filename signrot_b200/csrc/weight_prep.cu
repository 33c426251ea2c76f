// Offline weight preparation on the GPU: per-channel symmetric int4 round-to-nearest with the
// SignRot sign unfold/refold, straight to packed codes.
//
// Follows rtn_fwrd (fake_quant/gptq_utils.py:411-465) with WeightQuantizer.find_params
// (fake_quant/quant_utils.py:453-520) and the packing of Linear4bit.from_float
// (signrot/nn/linear.py:52-73):
//   Wu      = W * sign                       (unfold; exact, sign is +-1)
//   xmax    = max(|min(Wu, 0)|, max(Wu, 0)) clamped to >= 1e-5, fp32
//   scale   = xmax / 7                       (optionally the best of 80 shrunk candidates, `mse`)
//   q       = clamp(rint(Wu / scale), minq, 7)   minq = -7 when a sign is refolded, else -8
//   code    = q * sign                       (refold), two codes per byte, element 2j in the low nibble
// The reference materialises scale * q in the model dtype and divides by the fp16 scale again when
// it packs; |q| <= 8 keeps that round trip exact, so the codes are the same.
#include "common.cuh"
#include <cfloat>

namespace sr {

namespace {

constexpr int WP_THREADS = 256;

__device__ __forceinline__ float wp_load(const __half *p) { return __half2float(*p); }
__device__ __forceinline__ float wp_load(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
__device__ __forceinline__ float wp_load(const float *p) { return *p; }

__device__ __forceinline__ double block_sum(double v, double *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double s = 0.0;
#pragma unroll
    for (int w = 0; w < WP_THREADS / 32; ++w) s += red[w];
    return s;
}

// One CTA per weight row; the row (with the sign unfolded) lives in shared memory as fp32.
template <typename T>
__global__ void __launch_bounds__(WP_THREADS)
rtn_pack_kernel(const T *__restrict__ W, const int8_t *__restrict__ sign, uint32_t N, uint32_t K, int mse,
                uint8_t *__restrict__ packed, __half *__restrict__ scale_out) {
    extern __shared__ __align__(16) float wp_row[];
    __shared__ float redf[2][WP_THREADS / 32];
    __shared__ double redd[WP_THREADS / 32];
    const uint32_t n = blockIdx.x;
    const int tid = threadIdx.x;
    const T *wr = W + (size_t)n * K;
    float vmin = FLT_MAX, vmax = -FLT_MAX;
    for (uint32_t k = tid; k < K; k += WP_THREADS) {
        float v = wp_load(wr + k);
        if (sign && sign[k] < 0) v = -v;
        wp_row[k] = v;
        vmin = fminf(vmin, v);
        vmax = fmaxf(vmax, v);
    }
    vmin = warp_min(vmin);
    vmax = warp_max(vmax);
    if ((tid & 31) == 0) {
        redf[0][tid >> 5] = vmin;
        redf[1][tid >> 5] = vmax;
    }
    __syncthreads();
    vmin = redf[0][0];
    vmax = redf[1][0];
#pragma unroll
    for (int w = 1; w < WP_THREADS / 32; ++w) {
        vmin = fminf(vmin, redf[0][w]);
        vmax = fmaxf(vmax, redf[1][w]);
    }
    vmin = fminf(vmin, 0.f);
    vmax = fmaxf(vmax, 0.f);
    const float xmax = fmaxf(fmaxf(fabsf(vmin), vmax), 1e-5f);
    const float minq = sign ? -7.f : -8.f;
    float scale = __fdiv_rn(xmax, 7.f);
    if (mse) {
        // candidates p = 1 - i/100, i = 0..79; error sum |scale q - w|^2.4; the first best wins
        double best = 1.0 / 0.0;
        for (int i = 0; i < 80; ++i) {
            const float p = (float)(1.0 - (double)i / 100.0);
            const float s1 = __fdiv_rn(__fmul_rn(p, xmax), 7.f);
            double err = 0.0;
            for (uint32_t k = tid; k < K; k += WP_THREADS) {
                const float w = wp_row[k];
                const float qv = __fmul_rn(s1, fminf(fmaxf(rintf(__fdiv_rn(w, s1)), minq), 7.f));
                err += (double)powf(fabsf(qv - w), 2.4f);
            }
            err = block_sum(err, redd);
            if (err < best) {
                best = err;
                scale = s1;
            }
        }
    }
    if (tid == 0) scale_out[n] = __float2half_rn(scale);
    uint8_t *pr = packed + (size_t)n * (K >> 1);
    for (uint32_t j = tid; j < (K >> 1); j += WP_THREADS) {
        uint32_t byte = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t k = 2 * j + h;
            int qi = (int)fminf(fmaxf(rintf(__fdiv_rn(wp_row[k], scale)), minq), 7.f);
            if (sign && sign[k] < 0) qi = -qi;
            byte |= (uint32_t)(qi & 15) << (4 * h);
        }
        pr[j] = (uint8_t)byte;
    }
}

template <typename T>
int launch_rtn_pack(const void *W, const int8_t *sign, int64_t N, int64_t K, int mse, uint8_t *packed, __half *scale,
                    cudaStream_t st) {
    const size_t smem = (size_t)K * sizeof(float);
    auto kfn = rtn_pack_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "rtn_pack: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    kfn<<<(unsigned)N, WP_THREADS, smem, st>>>((const T *)W, sign, (uint32_t)N, (uint32_t)K, mse, packed, scale);
    return check_launch("rtn_pack");
}

}  // namespace

}  // namespace sr

using namespace sr;

extern "C" {

int sr_rtn_pack(const void *W, int dtype, int64_t N, int64_t K, const void *sign, int mse, void *packed, void *scale,
                void *stream) {
    SR_REQUIRE(N >= 0 && K >= 0, SR_ERR_INVALID, "rtn_pack: negative size");
    if (N == 0 || K == 0) return SR_OK;
    SR_REQUIRE(W && packed && scale, SR_ERR_INVALID, "rtn_pack: null pointer");
    SR_REQUIRE(K % 2 == 0, SR_ERR_INVALID, "rtn_pack: K = %lld must be even", (long long)K);
    SR_REQUIRE(K <= 56 * 1024 && N < (1ll << 31), SR_ERR_UNSUPPORTED, "rtn_pack: rows of at most 57344 values");
    cudaStream_t st = as_stream(stream);
    switch (dtype) {
        case SR_F16: return launch_rtn_pack<__half>(W, (const int8_t *)sign, N, K, mse, (uint8_t *)packed, (__half *)scale, st);
        case SR_BF16: return launch_rtn_pack<__nv_bfloat16>(W, (const int8_t *)sign, N, K, mse, (uint8_t *)packed, (__half *)scale, st);
        case SR_F32: return launch_rtn_pack<float>(W, (const int8_t *)sign, N, K, mse, (uint8_t *)packed, (__half *)scale, st);
        default: return fail(SR_ERR_INVALID, "rtn_pack: unknown dtype tag %d", dtype);
    }
}

}  // extern "C"
