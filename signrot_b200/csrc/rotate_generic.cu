// Online rotation, general shapes: y = ((hadK (x) H_S) x) / sqrt(n) * sign, optionally
// fused with the per-token int4 quantizer.
//
// Replaces, for one row per CTA and in one launch,
//   fast_hadamard_transform.hadamard_transform  (signrot/functional/hadamard.py:81,85)
//   the fp16 had-K matmul                       (signrot/functional/hadamard.py:86)
//   the had_adj_sign multiply                   (signrot/nn/hadamard.py:39)
//   the o_proj head-wise Hadamard H_heads (x) I (fake_quant/quant_utils.py:287-291)
//   sym/asym_quant_dynamic                      (signrot/kernels/fused.cu:68-198)
// Rounding points are the reference's: the Walsh-Hadamard stage accumulates in
// fp32 and is rounded to the tensor dtype, the had-K stage accumulates fp32 and
// is rounded again, the sign is exact.  With fp32 mode nothing is rounded until
// the final cast.
//
// This is the shape-generic kernel (any power-of-two S up to 16384/K, any K with a
// table, strided head-wise transform).  The row lives in shared memory as fp32 and
// is transformed by radix-8 register passes.  The 8B-model shapes have dedicated
// kernels in rotate_fast.cu.
#include "rotate.cuh"
#include <cfloat>

namespace sr {


__device__ __forceinline__ float round_to(float v, int dtype) {
    if (dtype == SR_F16) return __half2float(__float2half_rn(v));
    if (dtype == SR_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}

__device__ __forceinline__ void fwht8(float (&a)[8]) {
#pragma unroll
    for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if ((i & h) == 0) {
                const float u = a[i], w = a[i + h];
                a[i] = u + w;
                a[i + h] = u - w;
            }
        }
    }
}

__global__ void __launch_bounds__(256)
rotate_generic_kernel(RotateArgs p) {
    extern __shared__ float buf[];
    __shared__ float red[2][8];
    const uint32_t row = blockIdx.x;
    const int tid = threadIdx.x;
    const uint32_t n = p.n;

    // ---- load row as fp32
    if (p.in_dtype == SR_F16) {
        const __half *xr = (const __half *)p.x + (size_t)row * n;
        for (uint32_t i = tid; i < n; i += 256) buf[i] = __half2float(xr[i]);
    } else if (p.in_dtype == SR_BF16) {
        const __nv_bfloat16 *xr = (const __nv_bfloat16 *)p.x + (size_t)row * n;
        for (uint32_t i = tid; i < n; i += 256) {
            float f = __bfloat162float(xr[i]);
            if (p.cast_in_to_f16) f = __half2float(__float2half_rn(f));
            buf[i] = f;
        }
    } else {
        const float *xr = (const float *)p.x + (size_t)row * n;
        for (uint32_t i = tid; i < n; i += 256) buf[i] = xr[i];
    }
    __syncthreads();

    // ---- Walsh-Hadamard over index bits [stride, stride * S): radix-8 passes
    uint32_t h = p.stride;
    const uint32_t hend = p.stride * p.S;
    while (h < hend) {
        const uint32_t left = hend / h;  // remaining factor, a power of two >= 2
        if (left >= 8) {
            const uint32_t groups = n >> 3;
            for (uint32_t g = tid; g < groups; g += 256) {
                const uint32_t base = (g / h) * (8 * h) + (g % h);
                float a[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) a[j] = buf[base + j * h];
                fwht8(a);
#pragma unroll
                for (int j = 0; j < 8; ++j) buf[base + j * h] = a[j];
            }
            h <<= 3;
        } else {
            // one radix-2 pass (left is 2 or 4: at most two of these)
            const uint32_t pairs = n >> 1;
            for (uint32_t g = tid; g < pairs; g += 256) {
                const uint32_t base = (g / h) * (2 * h) + (g % h);
                const float u = buf[base], w = buf[base + h];
                buf[base] = u + w;
                buf[base + h] = u - w;
            }
            h <<= 1;
        }
        __syncthreads();
    }

    const int mid_dtype = p.fp32_mode ? SR_F32 : (p.in_dtype == SR_BF16 && !p.cast_in_to_f16 ? SR_BF16 : (p.in_dtype == SR_F32 ? SR_F32 : SR_F16));
    // scale, first rounding point
    for (uint32_t i = tid; i < n; i += 256) buf[i] = round_to(buf[i] * p.scale, mid_dtype);
    __syncthreads();

    // ---- had-K stage over the major index: y[k', j] = sum_k hadK[k', k] z[k, j]
    if (p.K > 1) {
        const uint32_t K = p.K, S = n / K;  // stride == 1 on this path
        float *tmp = buf + n;                // second row buffer
        for (uint32_t o = tid; o < n; o += 256) {
            const uint32_t kp = o / S, j = o % S;
            float acc = 0.f;
            if (p.fp32_mode) {
                const float *hk = (const float *)p.hadk + (size_t)kp * K;
                for (uint32_t k = 0; k < K; ++k) acc = fmaf(__ldg(hk + k), buf[k * S + j], acc);
            } else {
                const __half *hk = (const __half *)p.hadk + (size_t)kp * K;
                for (uint32_t k = 0; k < K; ++k) acc = fmaf(__half2float(__ldg(hk + k)), buf[k * S + j], acc);
            }
            tmp[o] = round_to(acc, mid_dtype);
        }
        __syncthreads();
        for (uint32_t i = tid; i < n; i += 256) buf[i] = tmp[i];
        __syncthreads();
    }

    // ---- sign (exact), final cast
    const int8_t *sg = p.sign ? p.sign + (size_t)(p.expert_ids ? p.expert_ids[row] : 0) * n : nullptr;
    const int final_dtype = p.q ? SR_F16 : p.out_dtype;
    float vmax = p.asym ? -FLT_MAX : 0.f, vmin = FLT_MAX;
    for (uint32_t i = tid; i < n; i += 256) {
        float v = buf[i];
        if (sg && sg[i] < 0) v = -v;
        v = round_to(v, final_dtype);
        buf[i] = v;
        if (p.asym) {
            vmax = fmaxf(vmax, v);
            vmin = fminf(vmin, v);
        } else {
            vmax = fmaxf(vmax, fabsf(v));
        }
    }
    if (p.out) {
        // the sign multiply and the cast happen before the store, as in OnlineHadamard.forward
        if (p.out_dtype == SR_F16) {
            __half *orow = (__half *)p.out + (size_t)row * n;
            for (uint32_t i = tid; i < n; i += 256) orow[i] = __float2half_rn(buf[i]);
        } else if (p.out_dtype == SR_BF16) {
            __nv_bfloat16 *orow = (__nv_bfloat16 *)p.out + (size_t)row * n;
            for (uint32_t i = tid; i < n; i += 256) orow[i] = __float2bfloat16_rn(buf[i]);
        } else {
            float *orow = (float *)p.out + (size_t)row * n;
            for (uint32_t i = tid; i < n; i += 256) orow[i] = buf[i];
        }
    }
    if (!p.q) return;

    // ---- per-token quantizer on the fp16 row (fused.cu:83-110 / 156-198)
    vmax = warp_max(vmax);
    vmin = warp_min(vmin);
    if ((tid & 31) == 0) {
        red[0][tid >> 5] = vmax;
        red[1][tid >> 5] = vmin;
    }
    __syncthreads();
    vmax = red[0][0];
    vmin = red[1][0];
#pragma unroll
    for (int w = 1; w < 8; ++w) {
        vmax = fmaxf(vmax, red[0][w]);
        vmin = fminf(vmin, red[1][w]);
    }
    float rcp;
    int zero_i = 0;
    if (!p.asym) {
        __half scale = __float2half(vmax / 7.f);
        if (p.clip != 1.f) scale = __float2half(__half2float(scale) * p.clip);
        if (tid == 0) p.q_scale[row] = scale;
        rcp = rcp_approx_ftz(__half2float(scale));
    } else {
        __half hmin = __float2half(vmin), hmax = __float2half(vmax);
        if (p.clip != 1.f) {
            hmin = __float2half(__half2float(hmin) * p.clip);
            hmax = __float2half(__half2float(hmax) * p.clip);
        }
        const __half diff = __float2half(__half2float(hmax) - __half2float(hmin));
        const __half scale = __float2half(__half2float(diff) / 15.f);
        const __half ratio = __float2half(-__half2float(hmin) / __half2float(scale));
        const __half zero = __float2half(nearbyintf(__half2float(ratio)));
        if (tid == 0) {
            p.q_scale[row] = scale;
            p.q_zero[row] = zero;
        }
        zero_i = __half2int_rn(zero);
        rcp = rcp_approx_ftz(__half2float(scale));
    }
    uint32_t *qr = reinterpret_cast<uint32_t *>(p.q + (size_t)row * (n >> 1));
    for (uint32_t w = tid; w < (n >> 3); w += 256) {
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const __half hv = __float2half_rn(buf[w * 8 + j]);
            const int c = p.asym ? asym_code(hv, rcp, zero_i, 0, 15) : sym_code(hv, rcp);
            packed |= (uint32_t)(c & 15) << (4 * j);
        }
        qr[w] = packed;
    }
}

int launch_rotate_generic(const RotateArgs &a, cudaStream_t st) {
    const size_t smem = (size_t)a.n * sizeof(float) * (a.K > 1 ? 2 : 1);
    SR_REQUIRE(smem <= 200 * 1024, SR_ERR_UNSUPPORTED, "rotate: row of %u elements does not fit in shared memory",
               a.n);
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(rotate_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             200 * 1024);
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "rotate: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    rotate_generic_kernel<<<a.rows, 256, smem, st>>>(a);
    return check_launch("rotate_generic");
}

}  // namespace sr
