// int4 paged KV cache: append, prefill scatter, fused Hadamard+quantize+append, and
// GQA-native split-KV decode attention with in-register dequantisation.
//
// Cache layout (signrot/transformers/kv_cache.py:185-196, kernels/include/flashinfer/page.cuh:60-95):
//   data  uint8 [pages, layers, 2 (k,v), heads, page_size, head_dim/2]   two 4-bit codes per byte
//   param fp16  [pages, layers, 2,       heads, page_size, 2]            (scale, zero) per vector
//   dequant: float(code) * scale - zero                                  (quantization.cuh:76)
// Request b owns pages indices[indptr[b] .. indptr[b+1]); its last page holds
// last_page_offset[b] valid entries.
//
// Replaces kernels/flashinfer.cu:11-106 + include/flashinfer/decode.cuh:481-751 and
// page.cuh:119-219.  Differences in design, not in results:
//  * one CTA serves all q heads that share a KV head, so a GQA cache is stored once
//    (the reference repeats every KV head group_size times, kv_cache.py:346-353);
//  * the dot products use  sum_d q_d (c_d s - z) = s sum_d q_d c_d - z sum_d q_d,
//    so codes are consumed as integers and the affine part is applied per vector;
//  * quantisation of new K/V (with the Hadamard on K) happens in the kernel that
//    writes the page slot.
#include "common.cuh"
#include "kv_cache.cuh"
#include <atomic>
#include <cfloat>
#include <cstdlib>
#include <cstring>

namespace sr {

// ------------------------------------------------------------------ scatter of pre-quantised vectors

// One warp per (token, head): lanes 0-3 copy K (64 B), 4-7 copy V, 8/9 the params.
// k/v: [tokens, heads, 64] uint8, k_param/v_param: [tokens, heads] half2.
// seqlen_indptr == nullptr: decode append, one token per request (page.cuh:119-164);
// otherwise prefill, request b appends tokens seqlen_indptr[b]..seqlen_indptr[b+1] (page.cuh:166-219).
__global__ void __launch_bounds__(256)
kv_scatter_kernel(PagedKV kv, const uint8_t *__restrict__ k, const uint8_t *__restrict__ v,
                  const __half2 *__restrict__ k_param, const __half2 *__restrict__ v_param,
                  const int32_t *__restrict__ seqlen_indptr, uint32_t batch, uint32_t total_tokens) {
    const uint32_t w = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= total_tokens * kv.heads) return;
    const uint32_t tok = w / kv.heads, head = w % kv.heads;
    uint32_t b, pos;
    if (seqlen_indptr == nullptr) {
        b = tok;
        pos = kv.seq_len(b) - 1;
    } else {
        b = 0;
        while (b + 1 < batch && (uint32_t)seqlen_indptr[b + 1] <= tok) ++b;
        const uint32_t n_app = (uint32_t)(seqlen_indptr[b + 1] - seqlen_indptr[b]);
        pos = kv.seq_len(b) - n_app + (tok - (uint32_t)seqlen_indptr[b]);
    }
    const uint32_t page = (uint32_t)kv.indices[kv.indptr[b] + pos / kv.page_size];
    const uint32_t entry = pos % kv.page_size;
    const size_t src = ((size_t)tok * kv.heads + head);
    if (lane < 8) {
        const uint32_t which = lane >> 2, part = lane & 3;
        const uint4 val = *reinterpret_cast<const uint4 *>((which ? v : k) + src * 64 + part * 16);
        *reinterpret_cast<uint4 *>(kv.data + kv.vec_index(page, which, head, entry) * 64 + part * 16) = val;
    } else if (lane == 8) {
        kv.param[kv.vec_index(page, 0, head, entry)] = k_param[src];
    } else if (lane == 9) {
        kv.param[kv.vec_index(page, 1, head, entry)] = v_param[src];
    }
}

// ------------------------------------------------------------------ fused Hadamard + quantise + append

// A warp takes KV_VPW consecutive (token, head, k|v) vectors of 128 at a time (lane holds 4 consecutive values
// of each; the loads and the shuffle butterflies of the KV_VPW vectors are independent, which is what hides
// their latency).  k, v: [B, T, heads, 128] fp16.  K goes through H_128 / sqrt(128) (fp32 butterflies,
// rounded to fp16: kv_cache.py:70-73,308-309) when had_k is set, then both are quantised (fused.cu:214-265)
// straight into their page slots.
constexpr int KV_VPW = 4;

__global__ void __launch_bounds__(256)
kv_append_quant_kernel(PagedKV kv, const __half *__restrict__ k, const __half *__restrict__ v, uint32_t batch,
                       uint32_t T, int had_k, float had_scale) {
    const int lane = threadIdx.x & 31;
    const uint32_t total = batch * T * kv.heads * 2;
    const uint32_t warps = gridDim.x * 8;
    for (uint32_t w0 = (blockIdx.x * 8 + (threadIdx.x >> 5)) * KV_VPW; w0 < total; w0 += warps * KV_VPW) {
        float a[KV_VPW][4];
        bool live[KV_VPW];
#pragma unroll
        for (int u = 0; u < KV_VPW; ++u) {
            const uint32_t w = w0 + u;
            live[u] = w < total;
            uint2 raw = make_uint2(0, 0);
            if (live[u]) raw = __ldg(reinterpret_cast<const uint2 *>(((w & 1) ? v : k) + (size_t)(w >> 1) * HD + lane * 4));
            const __half2 h01 = *reinterpret_cast<const __half2 *>(&raw.x), h23 = *reinterpret_cast<const __half2 *>(&raw.y);
            a[u][0] = __half2float(h01.x); a[u][1] = __half2float(h01.y);
            a[u][2] = __half2float(h23.x); a[u][3] = __half2float(h23.y);
        }
        if (had_k) {
#pragma unroll
            for (int u = 0; u < KV_VPW; ++u) {
                if (((w0 + u) & 1) == 0) {   // K vectors only (uniform across the warp)
                    const float t0 = a[u][0] + a[u][1], t1 = a[u][0] - a[u][1], t2 = a[u][2] + a[u][3], t3 = a[u][2] - a[u][3];
                    a[u][0] = t0 + t2; a[u][1] = t1 + t3; a[u][2] = t0 - t2; a[u][3] = t1 - t3;
                }
            }
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
                for (int u = 0; u < KV_VPW; ++u) {
                    if (((w0 + u) & 1) == 0) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float o = __shfl_xor_sync(0xffffffffu, a[u][j], m);
                            a[u][j] = (lane & m) ? (o - a[u][j]) : (a[u][j] + o);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < KV_VPW; ++u)
                if (((w0 + u) & 1) == 0)
#pragma unroll
                    for (int j = 0; j < 4; ++j) a[u][j] = __half2float(__float2half_rn(a[u][j] * had_scale));
        }
#pragma unroll
        for (int u = 0; u < KV_VPW; ++u) {
            float vmax = fmaxf(fmaxf(a[u][0], a[u][1]), fmaxf(a[u][2], a[u][3]));
            float vmin = fminf(fminf(a[u][0], a[u][1]), fminf(a[u][2], a[u][3]));
            vmax = warp_max(vmax);
            vmin = warp_min(vmin);
            __half scale, zero;
            kv_params_dev(vmin, vmax, scale, zero);
            const float fs = __half2float(scale), fz = __half2float(zero);
            uint32_t code = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half shifted = __float2half(a[u][j] + fz);
                const __half scaled = __float2half(__half2float(shifted) / fs);
                code |= (uint32_t)clampi((int)nearbyintf(__half2float(scaled)), 0, 15) << (4 * j);
            }
            if (live[u]) {
                const uint32_t w = w0 + u, which = w & 1, vec = w >> 1;
                const uint32_t head = vec % kv.heads;
                const uint32_t t = (vec / kv.heads) % T, b = vec / (kv.heads * T);
                const uint32_t pos = kv.seq_len(b) - T + t;
                const uint32_t page = (uint32_t)kv.indices[kv.indptr[b] + pos / kv.page_size];
                const uint32_t entry = pos % kv.page_size;
                const size_t vi = kv.vec_index(page, which, head, entry);
                reinterpret_cast<uint16_t *>(kv.data + vi * 64)[lane] = (uint16_t)code;
                if (lane == 0) {
                    __half2 p;
                    p.x = scale;
                    p.y = zero;
                    kv.param[vi] = p;
                }
            }
        }
    }
}

// ------------------------------------------------------------------ fused RoPE + append
//
// One pass over the projections of the new tokens: rotary embedding on q and k (the arithmetic of
// rope_qk_kernel: both products rounded to fp16 before the add, signrot/kernels/fused.cu:316-349),
// roped q written to q_out (and roped k to k_out when the caller needs it for a dense prefill
// attention), roped K rotated by the head_dim Hadamard and quantized, V quantized, both written to
// their page slots (the arithmetic of kv_append_quant_kernel).  q, k, v are addressed as
// base + token * stride + head * 128, so they may be column ranges of one fused q/k/v projection.
// One warp per 128-wide head vector; lane l holds dims 4l .. 4l+3, whose rotate-half partner lives
// in lane l ^ 16.
__global__ void __launch_bounds__(256)
rope_kv_append_kernel(PagedKV kv, const __half *__restrict__ q, const __half *__restrict__ k,
                      const __half *__restrict__ v, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                      const __half *__restrict__ cosv, const __half *__restrict__ sinv, uint32_t cos_seqs,
                      __half *__restrict__ q_out, __half *__restrict__ k_out, uint32_t batch, uint32_t T, uint32_t hq,
                      int had_k, float had_scale) {
    pdl_trigger();   // launched with programmatic serialization: see launch_pdl
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const uint32_t per_tok = hq + 2 * kv.heads;
    const uint32_t total = batch * T * per_tok;
    const uint32_t warps = gridDim.x * 8;
    for (uint32_t w = blockIdx.x * 8 + (threadIdx.x >> 5); w < total; w += warps) {
        const uint32_t token = w / per_tok, slot = w % per_tok;
        const int type = slot < hq ? 0 : (slot < hq + kv.heads ? 1 : 2);   // q, k, v (uniform across the warp)
        const uint32_t head = type == 0 ? slot : (type == 1 ? slot - hq : slot - hq - kv.heads);
        const __half *src = type == 0 ? q + (size_t)token * q_stride : (type == 1 ? k + (size_t)token * k_stride
                                                                                   : v + (size_t)token * v_stride);
        const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(src + (size_t)head * HD + lane * 4));
        __half h[4];
        *reinterpret_cast<uint2 *>(h) = raw;
        if (type < 2) {
            rope_vec(h, raw, cosv, sinv, (size_t)(cos_seqs == 1 ? token % T : token) * HD + lane * 4, lane);
            __half *dst = type == 0 ? q_out + ((size_t)token * hq + head) * HD : (k_out ? k_out + ((size_t)token * kv.heads + head) * HD : nullptr);
            if (dst) *reinterpret_cast<uint2 *>(dst + lane * 4) = *reinterpret_cast<const uint2 *>(h);
            if (type == 0) continue;
        }
        const uint32_t t = token % T, b = token / T;
        kv_quant_store(kv, h, (uint32_t)(type - 1), type == 1 && had_k, had_scale, b, head, kv.seq_len(b) - T + t, lane);
    }
}

// ------------------------------------------------------------------ decode attention

// 4-bit code -> fp32 without the conversion pipe (2^23 + n has n in its low mantissa bits).
__device__ __forceinline__ float nib2f(uint32_t w) { return __uint_as_float(0x4B000000u | (w & 15u)) - 8388608.f; }

// grid (batch, kv_heads, chunks), 128 threads.  G = q heads per KV head.  Eight lanes
// share one cached token (16 dims each); a warp covers four tokens per step, the CTA 16.
template <int G>
__global__ void __launch_bounds__(128)
decode_kernel(const __half *__restrict__ q, PagedKV kv, __half *__restrict__ o, float *__restrict__ tmp,
              uint32_t num_chunks, int had_q, float had_scale) {
    const uint32_t b = blockIdx.x, hk = blockIdx.y, chunk = blockIdx.z;
    const uint32_t hq_total = gridDim.y * G;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane & 7;        // which 16-dim slice
    const int slot = (warp << 2) | (lane >> 3);  // token slot 0..15

    __shared__ float sh_q[G][HD];
    __shared__ float sh_o[4][G][HD];
    __shared__ float sh_md[4][G][2];

    // ---- load q (optionally Hadamard-rotated, kv_cache.py:157-158), one warp per q head
    const float sm_scale = 1.44269504088896340736f * 0.08838834764831845f;  // log2(e) / sqrt(128)
    for (int g = warp; g < G; g += 4) {
        const uint32_t hq = hk * G + g;
        const __half *qp = q + ((size_t)b * hq_total + hq) * HD + lane * 4;
        const uint2 raw = *reinterpret_cast<const uint2 *>(qp);
        const __half2 h01 = *reinterpret_cast<const __half2 *>(&raw.x), h23 = *reinterpret_cast<const __half2 *>(&raw.y);
        float a[4] = {__half2float(h01.x), __half2float(h01.y), __half2float(h23.x), __half2float(h23.y)};
        if (had_q) {
            float t0 = a[0] + a[1], t1 = a[0] - a[1], t2 = a[2] + a[3], t3 = a[2] - a[3];
            a[0] = t0 + t2; a[1] = t1 + t3; a[2] = t0 - t2; a[3] = t1 - t3;
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float ot = __shfl_xor_sync(0xffffffffu, a[j], m);
                    a[j] = (lane & m) ? (ot - a[j]) : (a[j] + ot);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) a[j] = __half2float(__float2half_rn(a[j] * had_scale));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) sh_q[g][lane * 4 + j] = a[j];
    }
    __syncthreads();

    float qv[G][16], qsum[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            qv[g][j] = sh_q[g][sub * 16 + j] * sm_scale;
            s += qv[g][j];
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        qsum[g] = s;
    }

    // ---- this chunk's token range
    const uint32_t page_begin = (uint32_t)kv.indptr[b], page_end = (uint32_t)kv.indptr[b + 1];
    const uint32_t pages_total = page_end - page_begin;
    const uint32_t per_chunk = (pages_total + num_chunks - 1) / num_chunks;
    const uint32_t cp_begin = min(chunk * per_chunk, pages_total), cp_end = min(cp_begin + per_chunk, pages_total);
    const uint32_t last_valid = (uint32_t)kv.last_page_offset[b];

    float m[G], d[G], acc[G][16], accz[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -5e4f;
        d[g] = 0.f;
        accz[g] = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[g][j] = 0.f;
    }

    for (uint32_t pi = cp_begin; pi < cp_end; ++pi) {
        const uint32_t page = (uint32_t)kv.indices[page_begin + pi];
        const uint32_t valid = (pi == pages_total - 1) ? last_valid : kv.page_size;
        const size_t kbase = kv.vec_index(page, 0, hk, 0), vbase = kv.vec_index(page, 1, hk, 0);
        // the trip count is uniform across the warp (the shuffles below need every lane);
        // lanes whose token slot is past the end of the page compute on zeros and skip the update
        for (uint32_t e0 = 0; e0 < valid; e0 += 16) {
            const uint32_t e = e0 + slot;
            const bool live = e < valid;
            uint2 kc = make_uint2(0, 0), vc = make_uint2(0, 0);
            float2 kp = make_float2(0.f, 0.f), vp = make_float2(0.f, 0.f);
            if (live) {
                kc = __ldg(reinterpret_cast<const uint2 *>(kv.data + (kbase + e) * 64) + sub);
                vc = __ldg(reinterpret_cast<const uint2 *>(kv.data + (vbase + e) * 64) + sub);
                kp = __half22float2(kv.param[kbase + e]);
                vp = __half22float2(kv.param[vbase + e]);
            }
            float kf[16], vf[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                kf[j] = nib2f(kc.x >> (4 * j));
                kf[8 + j] = nib2f(kc.y >> (4 * j));
                vf[j] = nib2f(vc.x >> (4 * j));
                vf[8 + j] = nib2f(vc.y >> (4 * j));
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float dot = 0.f;
#pragma unroll
                for (int j = 0; j < 16; ++j) dot = fmaf(qv[g][j], kf[j], dot);
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                dot += __shfl_xor_sync(0xffffffffu, dot, 4);
                if (live) {
                    const float x = dot * kp.x - kp.y * qsum[g];
                    const float m_new = fmaxf(m[g], x);
                    const float alpha = ex2(m[g] - m_new);
                    const float p = ex2(x - m_new);
                    m[g] = m_new;
                    d[g] = d[g] * alpha + p;
                    const float ps = p * vp.x;
                    accz[g] = accz[g] * alpha + p * vp.y;
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[g][j] = fmaf(ps, vf[j], acc[g][j] * alpha);
                }
            }
        }
    }

    // ---- merge the 16 token slots (same dim slice `sub`)
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[g][j] -= accz[g];
        // within the warp: lanes sub, sub+8, sub+16, sub+24
#pragma unroll
        for (int off = 8; off < 32; off <<= 1) {
            const float m_o = __shfl_xor_sync(0xffffffffu, m[g], off);
            const float d_o = __shfl_xor_sync(0xffffffffu, d[g], off);
            const float m_new = fmaxf(m[g], m_o);
            const float a = ex2(m[g] - m_new), bsc = ex2(m_o - m_new);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float o_o = __shfl_xor_sync(0xffffffffu, acc[g][j], off);
                acc[g][j] = acc[g][j] * a + o_o * bsc;
            }
            d[g] = d[g] * a + d_o * bsc;
            m[g] = m_new;
        }
    }
    // across warps through shared memory (warp w's lanes 0..7 hold its merged state)
    float *so = &sh_o[0][0][0];
    if (lane < 8) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int j = 0; j < 16; ++j) so[((warp * G + g) * HD) + sub * 16 + j] = acc[g][j];
            if (sub == 0) {
                sh_md[warp][g][0] = m[g];
                sh_md[warp][g][1] = d[g];
            }
        }
    }
    __syncthreads();
    // thread t finalises dim t (HD == blockDim) for every g
    for (int g = 0; g < G; ++g) {
        float mm = sh_md[0][g][0];
#pragma unroll
        for (int w = 1; w < 4; ++w) mm = fmaxf(mm, sh_md[w][g][0]);
        float dd = 0.f, oo = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float sc = ex2(sh_md[w][g][0] - mm);
            dd += sh_md[w][g][1] * sc;
            oo += so[((w * G + g) * HD) + tid] * sc;
        }
        const uint32_t hq = hk * G + g;
        if (num_chunks == 1) {
            o[((size_t)b * hq_total + hq) * HD + tid] = __float2half_rn(__fdividef(oo, dd));
        } else {
            float *dst = tmp + (((size_t)b * hq_total + hq) * num_chunks + chunk) * (HD + 4);
            dst[tid] = oo;
            if (tid == 0) {
                dst[HD] = mm;
                dst[HD + 1] = dd;
            }
        }
    }
}

// grid (batch, q heads), 128 threads: combine the per-chunk states (decode.cuh:726-751).
__global__ void __launch_bounds__(128)
decode_merge_kernel(const float *__restrict__ tmp, __half *__restrict__ o, uint32_t num_chunks) {
    pdl_trigger();   // launched with programmatic serialization: see launch_pdl
    pdl_wait();
    const uint32_t b = blockIdx.x, h = blockIdx.y, H = gridDim.y;
    const int tid = threadIdx.x;
    const float *src = tmp + ((size_t)b * H + h) * num_chunks * (HD + 4);
    float mm = -5e4f;
    for (uint32_t c = 0; c < num_chunks; ++c) mm = fmaxf(mm, src[c * (HD + 4) + HD]);
    float dd = 0.f, oo = 0.f;
    for (uint32_t c = 0; c < num_chunks; ++c) {
        const float sc = ex2(src[c * (HD + 4) + HD] - mm);
        dd += src[c * (HD + 4) + HD + 1] * sc;
        oo += src[c * (HD + 4) + tid] * sc;
    }
    o[((size_t)b * H + h) * HD + tid] = __float2half_rn(__fdividef(oo, dd));
}

}  // namespace sr

using namespace sr;

static int fill_kv(PagedKV &kv, void *kv_data, void *kv_param, const void *indptr, const void *indices,
                   const void *last_page_offset, int64_t num_layers, int64_t layer_idx, int64_t heads,
                   int64_t page_size, const char *who) {
    SR_REQUIRE(kv_data && kv_param && indptr && indices && last_page_offset, SR_ERR_INVALID, "%s: null pointer", who);
    SR_REQUIRE(num_layers > 0 && layer_idx >= 0 && layer_idx < num_layers, SR_ERR_INVALID, "%s: bad layer index", who);
    SR_REQUIRE(heads > 0 && page_size > 0, SR_ERR_INVALID, "%s: bad cache geometry", who);
    SR_REQUIRE(aligned16(kv_data) && aligned4(kv_param), SR_ERR_INVALID, "%s: cache buffers are misaligned", who);
    kv.data = (uint8_t *)kv_data;
    kv.param = (__half2 *)kv_param;
    kv.indptr = (const int32_t *)indptr;
    kv.indices = (const int32_t *)indices;
    kv.last_page_offset = (const int32_t *)last_page_offset;
    kv.num_layers = (uint32_t)num_layers;
    kv.layer = (uint32_t)layer_idx;
    kv.heads = (uint32_t)heads;
    kv.page_size = (uint32_t)page_size;
    return SR_OK;
}

extern "C" {

int sr_append_kv_i4(void *kv_data, void *kv_param, const void *kv_indptr, const void *kv_indices,
                    const void *last_page_offset, const void *k, const void *v, const void *k_param,
                    const void *v_param, int64_t num_layers, int64_t layer_idx, int64_t num_heads, int64_t page_size,
                    int64_t head_dim, int64_t batch_size, void *stream) {
    SR_REQUIRE(head_dim == 128, SR_ERR_INVALID, "append_kv_i4: CHECK_EQ(head_dim, 128) failed. %lld vs 128", (long long)head_dim);
    if (batch_size == 0) return SR_OK;
    PagedKV kv;
    int rc = fill_kv(kv, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, num_layers, layer_idx, num_heads,
                     page_size, "append_kv_i4");
    if (rc) return rc;
    SR_REQUIRE(k && v && k_param && v_param, SR_ERR_INVALID, "append_kv_i4: null pointer");
    const uint32_t warps = (uint32_t)(batch_size * num_heads);
    kv_scatter_kernel<<<cdiv<uint32_t>(warps, 8), 256, 0, as_stream(stream)>>>(
        kv, (const uint8_t *)k, (const uint8_t *)v, (const __half2 *)k_param, (const __half2 *)v_param, nullptr,
        (uint32_t)batch_size, (uint32_t)batch_size);
    return check_launch("append_kv_i4");
}

int sr_init_kv_i4(void *kv_data, void *kv_param, const void *kv_indptr, const void *kv_indices,
                  const void *last_page_offset, const void *k, const void *v, const void *k_param,
                  const void *v_param, const void *seqlen_indptr, int64_t total_tokens, int64_t num_layers,
                  int64_t layer_idx, int64_t num_heads, int64_t page_size, int64_t head_dim, int64_t batch_size,
                  void *stream) {
    SR_REQUIRE(head_dim == 128, SR_ERR_INVALID, "init_kv_i4: CHECK_EQ(head_dim, 128) failed. %lld vs 128", (long long)head_dim);
    if (batch_size == 0 || total_tokens == 0) return SR_OK;
    PagedKV kv;
    int rc = fill_kv(kv, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, num_layers, layer_idx, num_heads,
                     page_size, "init_kv_i4");
    if (rc) return rc;
    SR_REQUIRE(k && v && k_param && v_param && seqlen_indptr, SR_ERR_INVALID, "init_kv_i4: null pointer");
    const int64_t warps = total_tokens * num_heads;
    SR_REQUIRE(warps < (1ll << 31), SR_ERR_UNSUPPORTED, "init_kv_i4: too many tokens");
    kv_scatter_kernel<<<(unsigned)cdiv<int64_t>(warps, 8), 256, 0, as_stream(stream)>>>(
        kv, (const uint8_t *)k, (const uint8_t *)v, (const __half2 *)k_param, (const __half2 *)v_param,
        (const int32_t *)seqlen_indptr, (uint32_t)batch_size, (uint32_t)total_tokens);
    return check_launch("init_kv_i4");
}

int sr_kv_append_quant(void *kv_data, void *kv_param, const void *kv_indptr, const void *kv_indices,
                       const void *last_page_offset, const void *k, const void *v, int64_t batch_size,
                       int64_t new_tokens, int64_t num_layers, int64_t layer_idx, int64_t num_heads,
                       int64_t page_size, int64_t head_dim, int hadamard_k, void *stream) {
    SR_REQUIRE(head_dim == 128, SR_ERR_INVALID, "kv_append_quant: head_dim must be 128, got %lld", (long long)head_dim);
    if (batch_size == 0 || new_tokens == 0) return SR_OK;
    PagedKV kv;
    int rc = fill_kv(kv, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, num_layers, layer_idx, num_heads,
                     page_size, "kv_append_quant");
    if (rc) return rc;
    SR_REQUIRE(k && v, SR_ERR_INVALID, "kv_append_quant: null pointer");
    const int64_t warps = batch_size * new_tokens * num_heads * 2;
    SR_REQUIRE(warps < (1ll << 31), SR_ERR_UNSUPPORTED, "kv_append_quant: too many tokens");
    const float had_scale = (float)(1.0 / sqrt(128.0));
    // persistent over groups of KV_VPW vectors per warp; small launches keep one group per warp
    int64_t ctas = cdiv<int64_t>(cdiv<int64_t>(warps, KV_VPW), 8);
    if (ctas > 148 * 8) ctas = 148 * 8;
    kv_append_quant_kernel<<<(unsigned)ctas, 256, 0, as_stream(stream)>>>(
        kv, (const __half *)k, (const __half *)v, (uint32_t)batch_size, (uint32_t)new_tokens, hadamard_k, had_scale);
    return check_launch("kv_append_quant");
}

int sr_rope_kv_append(void *kv_data, void *kv_param, const void *kv_indptr, const void *kv_indices,
                      const void *last_page_offset, const void *q, const void *k, const void *v, int64_t q_stride,
                      int64_t k_stride, int64_t v_stride, const void *cos, const void *sin, int64_t cos_seqs,
                      void *q_out, void *k_out, int64_t batch_size, int64_t new_tokens, int64_t num_layers,
                      int64_t layer_idx, int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size,
                      int64_t head_dim, int hadamard_k, void *stream) {
    SR_REQUIRE(head_dim == 128, SR_ERR_INVALID, "rope_kv_append: head_dim must be 128, got %lld", (long long)head_dim);
    if (batch_size == 0 || new_tokens == 0) return SR_OK;
    PagedKV kv;
    int rc = fill_kv(kv, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, num_layers, layer_idx,
                     num_kv_heads, page_size, "rope_kv_append");
    if (rc) return rc;
    SR_REQUIRE(q && k && v && cos && sin && q_out, SR_ERR_INVALID, "rope_kv_append: null pointer");
    SR_REQUIRE(num_qo_heads >= 1, SR_ERR_INVALID, "rope_kv_append: no q heads");
    SR_REQUIRE(cos_seqs == 1 || cos_seqs == batch_size, SR_ERR_INVALID, "rope_kv_append: cos/sin must be [1 or batch, T, 128]");
    SR_REQUIRE(q_stride % 4 == 0 && k_stride % 4 == 0 && v_stride % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                     reinterpret_cast<uintptr_t>(cos) | reinterpret_cast<uintptr_t>(sin) | reinterpret_cast<uintptr_t>(q_out) |
                     reinterpret_cast<uintptr_t>(k_out)) & 7u) == 0,
               SR_ERR_INVALID, "rope_kv_append: rows must be 8-byte aligned");
    const int64_t warps = batch_size * new_tokens * (num_qo_heads + 2 * num_kv_heads);
    SR_REQUIRE(warps < (1ll << 31), SR_ERR_UNSUPPORTED, "rope_kv_append: too many tokens");
    int64_t ctas = cdiv<int64_t>(warps, 8);
    if (ctas > 148 * 8) ctas = 148 * 8;
    launch_pdl(rope_kv_append_kernel, dim3((unsigned)ctas), dim3(256), 0, as_stream(stream),
        kv, (const __half *)q, (const __half *)k, (const __half *)v, q_stride, k_stride, v_stride, (const __half *)cos,
        (const __half *)sin, (uint32_t)cos_seqs, (__half *)q_out, (__half *)k_out, (uint32_t)batch_size,
        (uint32_t)new_tokens, (uint32_t)num_qo_heads, hadamard_k, (float)(1.0 / sqrt(128.0)));
    return check_launch("rope_kv_append");
}

static int batch_decode_impl(void *o, const void *q, void *kv_data, void *kv_param, const void *kv_indptr,
                             const void *kv_indices, const void *last_page_offset, int64_t num_layers, int64_t layer_idx,
                             int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size, int64_t head_dim,
                             int64_t batch_size, void *tmp, int64_t num_chunks, int hadamard_q, void *stream,
                             int32_t *counters, const RopeIn *rope = nullptr) {
    SR_REQUIRE(head_dim == 128, SR_ERR_INVALID, "batch_decode_i4: CHECK_EQ(head_dim, 128) failed. %lld vs 128", (long long)head_dim);
    if (batch_size == 0) return SR_OK;
    PagedKV kv;
    int rc = fill_kv(kv, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, num_layers, layer_idx,
                     num_kv_heads, page_size, "batch_decode_i4");
    if (rc) return rc;
    SR_REQUIRE(o && q, SR_ERR_INVALID, "batch_decode_i4: null pointer");
    SR_REQUIRE(num_qo_heads > 0 && num_qo_heads % num_kv_heads == 0, SR_ERR_INVALID,
               "batch_decode_i4: %lld q heads cannot share %lld kv heads", (long long)num_qo_heads, (long long)num_kv_heads);
    const int64_t G = num_qo_heads / num_kv_heads;
    SR_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, SR_ERR_UNSUPPORTED, "batch_decode_i4: group size %lld not supported", (long long)G);
    if (tmp == nullptr || num_chunks < 1) num_chunks = 1;
    SR_REQUIRE(num_chunks <= 65535, SR_ERR_INVALID, "batch_decode_i4: too many chunks");
    SR_REQUIRE(aligned4(q) && aligned4(o), SR_ERR_INVALID, "batch_decode_i4: q/o misaligned");
    cudaStream_t st = as_stream(stream);
    dim3 grid((unsigned)batch_size, (unsigned)num_kv_heads, (unsigned)num_chunks);
    const float had_scale = (float)(1.0 / sqrt(128.0));
    const __half *qp = (const __half *)q;
    __half *op = (__half *)o;
    float *tp = (float *)tmp;
    const uint32_t nc = (uint32_t)num_chunks;
    // the tensor-core kernel takes page sizes that are multiples of 16; the CUDA-core kernel the rest
    // 0: not this kernel's geometry; 1: split-KV states left in tmp; 2: output complete
    const int took = launch_decode_tc((int)G, grid, qp, kv, op, tp, nc, hadamard_q, had_scale, st, counters, rope);
    SR_REQUIRE(took != 0 || rope == nullptr, SR_ERR_UNSUPPORTED,
               "rope_decode_i4: the page size must be a multiple of 16 (use rope_kv_append and batch_decode_i4)");
    if (!took) switch (G) {
        case 1: decode_kernel<1><<<grid, 128, 0, st>>>(qp, kv, op, tp, nc, hadamard_q, had_scale); break;
        case 2: decode_kernel<2><<<grid, 128, 0, st>>>(qp, kv, op, tp, nc, hadamard_q, had_scale); break;
        case 4: decode_kernel<4><<<grid, 128, 0, st>>>(qp, kv, op, tp, nc, hadamard_q, had_scale); break;
        default: decode_kernel<8><<<grid, 128, 0, st>>>(qp, kv, op, tp, nc, hadamard_q, had_scale); break;
    }
    rc = check_launch("batch_decode_i4");
    if (rc) return rc;
    if (num_chunks > 1 && took != 2) {   // the tensor-core kernel merges by itself inside a cluster, or when it has counters
        dim3 mgrid((unsigned)batch_size, (unsigned)num_qo_heads);
        launch_pdl(decode_merge_kernel, mgrid, dim3(128), 0, st, (const float *)tp, op, nc);
        rc = check_launch("batch_decode_i4 (merge)");
    }
    return rc;
}

int sr_batch_decode_i4(void *o, const void *q, void *kv_data, void *kv_param, const void *kv_indptr,
                       const void *kv_indices, const void *last_page_offset, int64_t num_layers, int64_t layer_idx,
                       int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size, int64_t head_dim,
                       int64_t batch_size, void *tmp, int64_t num_chunks, int hadamard_q, void *stream) {
    return batch_decode_impl(o, q, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, num_layers, layer_idx,
                             num_qo_heads, num_kv_heads, page_size, head_dim, batch_size, tmp, num_chunks, hadamard_q,
                             stream, nullptr);
}

int sr_batch_decode_i4_merged(void *o, const void *q, void *kv_data, void *kv_param, const void *kv_indptr,
                              const void *kv_indices, const void *last_page_offset, int64_t num_layers,
                              int64_t layer_idx, int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size,
                              int64_t head_dim, int64_t batch_size, void *tmp, int64_t num_chunks, void *counters,
                              int hadamard_q, void *stream) {
    SR_REQUIRE(counters != nullptr || num_chunks <= 1 || tmp == nullptr, SR_ERR_INVALID,
               "batch_decode_i4_merged: the arrival counters are missing");
    return batch_decode_impl(o, q, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, num_layers, layer_idx,
                             num_qo_heads, num_kv_heads, page_size, head_dim, batch_size, tmp, num_chunks, hadamard_q,
                             stream, (int32_t *)counters);
}

int sr_rope_decode_i4(void *o, const void *q, const void *k, const void *v, int64_t q_stride, int64_t k_stride,
                      int64_t v_stride, const void *cos, const void *sin, int64_t cos_seqs, void *kv_data, void *kv_param,
                      const void *kv_indptr, const void *kv_indices, const void *last_page_offset, int64_t num_layers,
                      int64_t layer_idx, int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size, int64_t head_dim,
                      int64_t batch_size, void *tmp, int64_t num_chunks, int hadamard_q, int hadamard_k, void *stream) {
    SR_REQUIRE(q && k && v && cos && sin, SR_ERR_INVALID, "rope_decode_i4: null pointer");
    SR_REQUIRE(cos_seqs == 1 || cos_seqs == batch_size, SR_ERR_INVALID, "rope_decode_i4: cos/sin for 1 or batch sequences");
    SR_REQUIRE(q_stride >= num_qo_heads * 128 && k_stride >= num_kv_heads * 128 && v_stride >= num_kv_heads * 128 &&
                   q_stride % 4 == 0 && k_stride % 4 == 0 && v_stride % 4 == 0,
               SR_ERR_INVALID, "rope_decode_i4: bad request stride");
    SR_REQUIRE(((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)cos | (uintptr_t)sin) % 8 == 0, SR_ERR_INVALID,
               "rope_decode_i4: q, k, v, cos and sin must be 8-byte aligned");
    RopeIn rope;
    rope.q = (const __half *)q;
    rope.k = (const __half *)k;
    rope.v = (const __half *)v;
    rope.q_stride = q_stride;
    rope.k_stride = k_stride;
    rope.v_stride = v_stride;
    rope.cosv = (const __half *)cos;
    rope.sinv = (const __half *)sin;
    rope.cos_seqs = (uint32_t)cos_seqs;
    rope.had_k = hadamard_k;
    return batch_decode_impl(o, q, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, num_layers, layer_idx,
                             num_qo_heads, num_kv_heads, page_size, head_dim, batch_size, tmp, num_chunks, hadamard_q,
                             stream, nullptr, &rope);
}

// ------------------------------------------------------------------ decode-step bookkeeping on the device
//
// One CTA.  Reads the token count of the (uniform-length) batch, publishes the position of the token
// this step appends and the page tables of the sequence INCLUDING that token, then stores the new count.
// Page of (request b, logical page j) = j * batch + b; a request's pages are listed contiguously.
__global__ void decode_advance_kernel(int32_t *__restrict__ length, int64_t *__restrict__ position,
                                      int32_t *__restrict__ kv_indptr, int32_t *__restrict__ kv_indices,
                                      int32_t *__restrict__ last_page_offset, int batch, int page_size, int max_pages) {
    pdl_trigger();
    pdl_wait();
    const int len = *length;
    __syncthreads();                       // every thread has read the count before thread 0 replaces it
    const int new_len = min(len + 1, max_pages * page_size);
    const int pages = (new_len + page_size - 1) / page_size;
    const int last = new_len - (pages - 1) * page_size;
    for (int i = threadIdx.x; i <= batch; i += blockDim.x) {
        kv_indptr[i] = i * pages;
        if (i < batch) last_page_offset[i] = last;
    }
    for (int i = threadIdx.x; i < pages * batch; i += blockDim.x) kv_indices[i] = (i % pages) * batch + i / pages;
    if (threadIdx.x == 0) {
        *position = new_len - 1;
        *length = new_len;
    }
}

int sr_decode_advance(void *length, void *position, void *kv_indptr, void *kv_indices, void *last_page_offset,
                      int64_t batch_size, int64_t page_size, int64_t max_pages, void *stream) {
    SR_REQUIRE(length && position && kv_indptr && kv_indices && last_page_offset, SR_ERR_INVALID,
               "decode_advance: null pointer");
    SR_REQUIRE(batch_size > 0 && page_size > 0 && max_pages > 0 && batch_size * max_pages < (1ll << 30), SR_ERR_INVALID,
               "decode_advance: bad geometry (batch %lld, page %lld, pages %lld)", (long long)batch_size,
               (long long)page_size, (long long)max_pages);
    launch_pdl(decode_advance_kernel, dim3(1), dim3(256), 0, as_stream(stream), (int32_t *)length, (int64_t *)position,
               (int32_t *)kv_indptr, (int32_t *)kv_indices, (int32_t *)last_page_offset, (int)batch_size,
               (int)page_size, (int)max_pages);
    return check_launch("decode_advance");
}

// ------------------------------------------------------------------ decode without a caller workspace
//
// Built-in split-KV workspace for callers that have no way to allocate device memory: a
// fixed array in the library's own data segment.  Every GPU that loads the library carries
// these 4.1 MiB until the process exits.
#define SR_DECODE_STATIC_FLOATS (16ll * 32 * 16 * 132)  /* batch 16 x 32 q heads x 16 chunks x (128 + 4) */
static __device__ __align__(256) float g_decode_workspace[SR_DECODE_STATIC_FLOATS];

// In host code `g_decode_workspace` is only a handle for the runtime, not an address a kernel
// may dereference.  The device address is looked up once per device (with that device current).
static float *decode_workspace_for_current_device(int *rc) {
    static std::atomic<float *> cached[64];   // zero-initialised; a racing first call stores the same address
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        *rc = fail(SR_ERR_CUDA, "batch_decode_i4_static: cudaGetDevice: %s", cudaGetErrorString(e));
        return nullptr;
    }
    float *p = cached[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        e = cudaGetSymbolAddress((void **)&p, g_decode_workspace);
        if (e != cudaSuccess || p == nullptr) {
            *rc = fail(SR_ERR_CUDA, "batch_decode_i4_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return nullptr;
        }
        cached[dev].store(p, std::memory_order_release);
    }
    *rc = SR_OK;
    return p;
}

int sr_batch_decode_i4_static(void *o, const void *q, void *kv_data, void *kv_param, const void *kv_indptr,
                              const void *kv_indices, const void *last_page_offset, int64_t num_layers,
                              int64_t layer_idx, int64_t num_qo_heads, int64_t num_kv_heads, int64_t page_size,
                              int64_t head_dim, int64_t batch_size, int64_t num_chunks, int hadamard_q,
                              void *stream) {
    SR_REQUIRE(batch_size >= 0 && num_qo_heads >= 0, SR_ERR_INVALID, "batch_decode_i4_static: negative size");
    if (num_chunks < 1) num_chunks = 1;
    float *ws = nullptr;
    if (num_chunks > 1 && batch_size > 0) {
        const long long need = (long long)batch_size * num_qo_heads * num_chunks * (128 + 4);
        SR_REQUIRE(need <= SR_DECODE_STATIC_FLOATS, SR_ERR_UNSUPPORTED,
                   "batch_decode_i4_static: batch %lld x %lld q heads x %lld chunks needs %lld floats of workspace, "
                   "the built-in one holds %lld; use fewer chunks or sr_batch_decode_i4 with your own buffer",
                   (long long)batch_size, (long long)num_qo_heads, (long long)num_chunks, need,
                   (long long)SR_DECODE_STATIC_FLOATS);
        int rc = SR_OK;
        ws = decode_workspace_for_current_device(&rc);
        if (rc != SR_OK) return rc;
    }
    // Every chunk writes its whole record before the merge kernel reads it, so nothing in the
    // workspace has to start at zero; what the previous call left there is simply overwritten.
    return sr_batch_decode_i4(o, q, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, num_layers, layer_idx,
                              num_qo_heads, num_kv_heads, page_size, head_dim, batch_size, ws, num_chunks, hadamard_q,
                              stream);
}

}  // extern "C"
