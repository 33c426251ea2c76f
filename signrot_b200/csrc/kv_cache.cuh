// Paged int4 KV cache descriptor shared by the cache kernels.
//
// Cache layout (signrot/transformers/kv_cache.py:185-196, kernels/include/flashinfer/page.cuh:60-95):
//   data  uint8 [pages, layers, 2 (k,v), heads, page_size, head_dim/2]   two 4-bit codes per byte
//   param fp16  [pages, layers, 2,       heads, page_size, 2]            (scale, zero) per vector
//   dequant: float(code) * scale - zero                                  (quantization.cuh:76)
#pragma once
#include "common.cuh"

namespace sr {

struct PagedKV {
    uint8_t *data;
    __half2 *param;
    const int32_t *indptr, *indices, *last_page_offset;
    uint32_t num_layers, layer, heads, page_size;  // head_dim fixed to 128

    __device__ __forceinline__ size_t vec_index(uint32_t page, uint32_t kv, uint32_t head, uint32_t entry) const {
        return ((((size_t)page * num_layers + layer) * 2 + kv) * heads + head) * page_size + entry;
    }
    __device__ __forceinline__ uint32_t seq_len(uint32_t b) const {
        return (uint32_t)(indptr[b + 1] - indptr[b] - 1) * page_size + (uint32_t)last_page_offset[b];
    }
};

constexpr int HD = 128;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- per-vector arithmetic shared by the append kernels and the decode kernel that appends by itself.  One warp
// per 128-wide head vector; lane l holds dims 4 l .. 4 l + 3.

// signrot/kernels/fused.cu:236-247
__device__ __forceinline__ void kv_params_dev(float vmin, float vmax, __half &scale, __half &zero) {
    const __half hmin = __float2half(vmin), hmax = __float2half(vmax);
    __half diff = __float2half(__half2float(hmax) - __half2float(hmin));
    diff = __float2half(fmaxf(__half2float(diff), 1e-5f));
    scale = __float2half(__half2float(diff) / 15.f);
    zero = __hneg(hmin);
}

// Rotary embedding of one head vector in place (the arithmetic of rope_qk_kernel: both products rounded to fp16
// before the add, signrot/kernels/fused.cu:316-349).  `raw` = the lane's four values as loaded, `ct` = offset of the
// lane's four cos / sin entries; the rotate-half partner of dims 4 l .. lives in lane l ^ 16.
__device__ __forceinline__ void rope_vec(__half (&h)[4], uint2 raw, const __half *__restrict__ cosv,
                                         const __half *__restrict__ sinv, size_t ct, int lane) {
    const uint32_t p0 = __shfl_xor_sync(0xffffffffu, raw.x, 16), p1 = __shfl_xor_sync(0xffffffffu, raw.y, 16);
    __half pb[4];
    *reinterpret_cast<uint2 *>(pb) = make_uint2(p0, p1);
    __half c[4], sn[4];
    *reinterpret_cast<uint2 *>(c) = __ldg(reinterpret_cast<const uint2 *>(cosv + ct));
    *reinterpret_cast<uint2 *>(sn) = __ldg(reinterpret_cast<const uint2 *>(sinv + ct));
    const bool first_half = lane < 16;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __half p = __float2half(__half2float(h[j]) * __half2float(c[j]));
        const float bf = first_half ? -__half2float(pb[j]) : __half2float(pb[j]);
        const __half r = __float2half(bf * __half2float(sn[j]));
        h[j] = __float2half(__half2float(p) + __half2float(r));
    }
}

// One new K (which = 0, optionally through H_128 / sqrt(128)) or V (which = 1) vector: quantizer of
// kv_append_quant_kernel (fused.cu:214-265) and the store into the page slot of token `pos` of request b.
__device__ __forceinline__ void kv_quant_store(const PagedKV &kv, const __half (&h)[4], uint32_t which, bool had,
                                               float had_scale, uint32_t b, uint32_t head, uint32_t pos, int lane) {
    float a[4] = {__half2float(h[0]), __half2float(h[1]), __half2float(h[2]), __half2float(h[3])};
    if (had) {
        const float t0 = a[0] + a[1], t1 = a[0] - a[1], t2 = a[2] + a[3], t3 = a[2] - a[3];
        a[0] = t0 + t2; a[1] = t1 + t3; a[2] = t0 - t2; a[3] = t1 - t3;
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float o = __shfl_xor_sync(0xffffffffu, a[j], m);
                a[j] = (lane & m) ? (o - a[j]) : (a[j] + o);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) a[j] = __half2float(__float2half_rn(a[j] * had_scale));
    }
    float vmax = fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3]));
    float vmin = fminf(fminf(a[0], a[1]), fminf(a[2], a[3]));
    vmax = warp_max(vmax);
    vmin = warp_min(vmin);
    __half scale, zero;
    kv_params_dev(vmin, vmax, scale, zero);
    const float fs = __half2float(scale), fz = __half2float(zero);
    uint32_t code = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __half shifted = __float2half(a[j] + fz);
        const __half scaled = __float2half(__half2float(shifted) / fs);
        code |= (uint32_t)clampi((int)nearbyintf(__half2float(scaled)), 0, 15) << (4 * j);
    }
    const uint32_t page = (uint32_t)kv.indices[kv.indptr[b] + pos / kv.page_size];
    const uint32_t entry = pos % kv.page_size;
    const size_t vi = kv.vec_index(page, which, head, entry);
    reinterpret_cast<uint16_t *>(kv.data + vi * 64)[lane] = (uint16_t)code;
    if (lane == 0) {
        __half2 pr;
        pr.x = scale;
        pr.y = zero;
        kv.param[vi] = pr;
    }
}

// Projections of the one new token per request, for the decode kernel that applies the rotary embedding and
// appends K / V itself (k == null: q is already rotated and the cache already holds the token).
struct RopeIn {
    const __half *q, *k, *v;            // base + request * stride + head * 128 (column ranges of a fused projection are fine)
    long long q_stride, k_stride, v_stride;
    const __half *cosv, *sinv;          // [cos_seqs (1 or batch), 1, 128]
    uint32_t cos_seqs;
    int had_k;
};

// Tensor-core decode kernel (kv_decode_tc.cu): same arguments and workspace format as decode_kernel.
// Returns 0 when the geometry is not one it handles (page_size % 16 != 0), 1 when the split-KV states are left in tmp
// for decode_merge_kernel, 2 when the output is complete (one chunk, merged in the cluster, or merged through counters).
int launch_decode_tc(int G, dim3 grid, const __half *q, const PagedKV &kv, __half *o, float *tmp, uint32_t num_chunks,
                     int had_q, float had_scale, cudaStream_t st, int32_t *counters = nullptr, const RopeIn *rope = nullptr);

}  // namespace sr
