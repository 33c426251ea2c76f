// Adjacent fused ops of the decode graph: RMSNorm, rotary embedding, SwiGLU and
// the KV-cache quantize+pack.  Arithmetic (operation order and every fp16
// rounding point) follows signrot/kernels/fused.cu:214-390; the memory access
// is vectorised (128-bit) and rows are held in registers.
#include "common.cuh"
#include <cfloat>
#include <cstdlib>

namespace sr {

bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("SIGNROT_B200_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

// ------------------------------------------------------------------ RMSNorm
// out = rn_h(x * rsqrtf(sum(x^2) / mean_dim + eps)), fp32 accumulation (fused.cu:278-302)
template <int NV>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const __half *__restrict__ x, uint32_t rows, uint32_t cols, float eps, float mean_dim,
               __half *__restrict__ out) {
    const uint32_t row = blockIdx.x;
    const int tid = threadIdx.x;
    const uint32_t nvec = cols >> 3;
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * cols);
    __shared__ float red[8];
    Vec16 v[NV];
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const uint32_t vi = tid + i * 256;
        if (vi < nvec) {
            v[i].u = __ldg(xr + vi);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float f = __half2float(v[i].h[j]);
                acc += f * f;
            }
        }
    }
    acc = warp_sum(acc);
    if ((tid & 31) == 0) red[tid >> 5] = acc;
    __syncthreads();
    acc = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) acc += red[w];
    const float inv = rsqrtf(acc / mean_dim + eps);
    uint4 *orow = reinterpret_cast<uint4 *>(out + (size_t)row * cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const uint32_t vi = tid + i * 256;
        if (vi < nvec) {
            Vec16 o;
#pragma unroll
            for (int j = 0; j < 8; ++j) o.h[j] = __float2half(__half2float(v[i].h[j]) * inv);
            orow[vi] = o.u;
        }
    }
}

__global__ void __launch_bounds__(256)
rmsnorm_generic_kernel(const __half *__restrict__ x, uint32_t rows, uint32_t cols, float eps, float mean_dim,
                       __half *__restrict__ out) {
    const uint32_t row = blockIdx.x;
    const int tid = threadIdx.x;
    const __half *xr = x + (size_t)row * cols;
    __shared__ float red[8];
    float acc = 0.f;
    for (uint32_t i = tid; i < cols; i += 256) {
        const float f = __half2float(xr[i]);
        acc += f * f;
    }
    acc = warp_sum(acc);
    if ((tid & 31) == 0) red[tid >> 5] = acc;
    __syncthreads();
    acc = 0.f;
    for (int w = 0; w < 8; ++w) acc += red[w];
    const float inv = rsqrtf(acc / mean_dim + eps);
    __half *orow = out + (size_t)row * cols;
    for (uint32_t i = tid; i < cols; i += 256) orow[i] = __float2half(__half2float(xr[i]) * inv);
}

// ------------------------------------------------------------------ RoPE
// In-place HF rotate-half rotary embedding on q [B,T,Hq,D] and k [B,T,Hk,D]; both
// products are rounded to fp16 before the add (fused.cu:316-349).
__global__ void __launch_bounds__(128)
rope_qk_kernel(__half *__restrict__ q, __half *__restrict__ k, const __half *__restrict__ cosv,
               const __half *__restrict__ sinv, uint32_t seq_len, uint32_t cos_seqs, uint32_t hq, uint32_t hk,
               uint32_t head_dim, uint32_t total_pairs) {
    // one thread per (token, head, pair-of-2 channels in the first half): two
    // pairs per thread so that loads are 32-bit
    const uint32_t half_dim = head_dim >> 1;
    const uint32_t per_head = half_dim >> 1;  // threads per head (head_dim % 4 == 0 here)
    const size_t gid = (size_t)blockIdx.x * 128 + threadIdx.x;
    if (gid >= total_pairs) return;
    const uint32_t i = (gid % per_head) * 2;
    const size_t th = gid / per_head;
    const uint32_t heads = hq + hk;
    const uint32_t head = th % heads;
    const size_t token = th / heads;
    __half *base = head < hq ? q + (token * hq + head) * head_dim : k + (token * hk + (head - hq)) * head_dim;
    const size_t ct = cos_seqs == 1 ? token % seq_len : token;
    const __half *c = cosv + ct * head_dim, *s = sinv + ct * head_dim;
    const __half2 x0 = *reinterpret_cast<const __half2 *>(base + i);
    const __half2 x1 = *reinterpret_cast<const __half2 *>(base + i + half_dim);
    const __half2 c0 = *reinterpret_cast<const __half2 *>(c + i), c1 = *reinterpret_cast<const __half2 *>(c + i + half_dim);
    const __half2 s0 = *reinterpret_cast<const __half2 *>(s + i), s1 = *reinterpret_cast<const __half2 *>(s + i + half_dim);
    auto rot = [](__half a, __half ca, __half b, __half sb, bool neg) {
        const __half p = __float2half(__half2float(a) * __half2float(ca));
        const float bf = neg ? -__half2float(b) : __half2float(b);
        const __half r = __float2half(bf * __half2float(sb));
        return __float2half(__half2float(p) + __half2float(r));
    };
    __half2 o0, o1;
    o0.x = rot(x0.x, c0.x, x1.x, s0.x, true);
    o0.y = rot(x0.y, c0.y, x1.y, s0.y, true);
    o1.x = rot(x1.x, c1.x, x0.x, s1.x, false);
    o1.y = rot(x1.y, c1.y, x0.y, s1.y, false);
    *reinterpret_cast<__half2 *>(base + i) = o0;
    *reinterpret_cast<__half2 *>(base + i + half_dim) = o1;
}

__global__ void __launch_bounds__(128)
rope_qk_generic_kernel(__half *__restrict__ q, __half *__restrict__ k, const __half *__restrict__ cosv,
                       const __half *__restrict__ sinv, uint32_t seq_len, uint32_t cos_seqs, uint32_t hq,
                       uint32_t hk, uint32_t head_dim) {
    const uint32_t half_dim = head_dim >> 1;
    const uint32_t heads = hq + hk;
    const size_t token = blockIdx.x / heads;
    const uint32_t head = blockIdx.x % heads;
    __half *base = head < hq ? q + (token * hq + head) * head_dim : k + (token * hk + (head - hq)) * head_dim;
    const size_t ct = cos_seqs == 1 ? token % seq_len : token;
    const __half *c = cosv + ct * head_dim, *s = sinv + ct * head_dim;
    for (uint32_t i = threadIdx.x; i < half_dim; i += blockDim.x) {
        const float x0 = __half2float(base[i]), x1 = __half2float(base[i + half_dim]);
        const __half a0 = __float2half(x0 * __half2float(c[i]));
        const __half b0 = __float2half(-x1 * __half2float(s[i]));
        const __half a1 = __float2half(x1 * __half2float(c[i + half_dim]));
        const __half b1 = __float2half(x0 * __half2float(s[i + half_dim]));
        base[i] = __float2half(__half2float(a0) + __half2float(b0));
        base[i + half_dim] = __float2half(__half2float(a1) + __half2float(b1));
    }
}

// ------------------------------------------------------------------ SwiGLU
// rn_h(rn_h(g / (1 + expf(-g))) * u)   (fused.cu:367-381)
__device__ __forceinline__ __half swiglu1(__half g, __half u) {
    const float gf = __half2float(g);
    const __half s = __float2half(gf / (1.f + expf(-gf)));
    return __float2half(__half2float(s) * __half2float(u));
}

__global__ void __launch_bounds__(256)
swiglu_kernel(const __half *__restrict__ gate, const __half *__restrict__ up, size_t numel, __half *__restrict__ out,
              bool vec) {
    const size_t gid = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (vec) {
        const size_t nvec = numel >> 3;
        if (gid < nvec) {
            Vec16 g, u, o;
            g.u = __ldg(reinterpret_cast<const uint4 *>(gate) + gid);
            u.u = __ldg(reinterpret_cast<const uint4 *>(up) + gid);
#pragma unroll
            for (int j = 0; j < 8; ++j) o.h[j] = swiglu1(g.h[j], u.h[j]);
            reinterpret_cast<uint4 *>(out)[gid] = o.u;
        }
        // tail (numel % 8) handled by the first few threads
        const size_t tail = (nvec << 3) + gid;
        if (gid < 8 && tail < numel) out[tail] = swiglu1(gate[tail], up[tail]);
    } else {
        if (gid < numel) out[gid] = swiglu1(gate[gid], up[gid]);
    }
}

// ------------------------------------------------------------------ KV quantize + pack
// Per row (one head vector): asymmetric uint4 with params [scale, zero = -min]
// (fused.cu:214-265; Python twin signrot/transformers/kv_cache.py:47-58):
//   diff = rn_h(max(rn_h(hmax - hmin), 1e-5)); scale = rn_h(diff / 15); zero = -hmin
//   q = clamp(rint(rn_h(rn_h(x + zero) / scale)), 0, 15)      (true division)
// The quantize step is shared with the fused KV append in kv_cache.cu.
__device__ __forceinline__ void kv_params(float vmin, float vmax, __half &scale, __half &zero) {
    const __half hmin = __float2half(vmin), hmax = __float2half(vmax);
    __half diff = __float2half(__half2float(hmax) - __half2float(hmin));
    diff = __float2half(fmaxf(__half2float(diff), 1e-5f));
    scale = __float2half(__half2float(diff) / 15.f);
    zero = __hneg(hmin);
}
__device__ __forceinline__ uint32_t kv_code(__half x, float fscale, float fzero) {
    const __half shifted = __float2half(__half2float(x) + fzero);
    const __half scaled = __float2half(__half2float(shifted) / fscale);
    return (uint32_t)clampi((int)nearbyintf(__half2float(scaled)), 0, 15);
}

// TPR threads per row, 8 elements each (cols == TPR * 8)
template <int TPR>
__global__ void __launch_bounds__(256)
kv_quant_pack_kernel(const __half *__restrict__ x, uint32_t rows, uint32_t cols, __half *__restrict__ param,
                     uint8_t *__restrict__ q) {
    const int tid = threadIdx.x;
    const int sub = tid % TPR;
    const uint32_t row = blockIdx.x * (256 / TPR) + tid / TPR;
    const bool live = row < rows;
    Vec16 v;
    float vmax = -FLT_MAX, vmin = FLT_MAX;
    if (live) {
        v.u = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)row * cols) + sub);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float f = __half2float(v.h[j]);
            vmax = fmaxf(vmax, f);
            vmin = fminf(vmin, f);
        }
    }
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) {
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
        vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
    }
    if (!live) return;
    __half scale, zero;
    kv_params(vmin, vmax, scale, zero);
    if (sub == 0) {
        __half2 p;
        p.x = scale;
        p.y = zero;
        *reinterpret_cast<__half2 *>(param + (size_t)row * 2) = p;
    }
    const float fs = __half2float(scale), fz = __half2float(zero);
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) packed |= kv_code(v.h[j], fs, fz) << (4 * j);
    reinterpret_cast<uint32_t *>(q + (size_t)row * (cols >> 1))[sub] = packed;
}

__global__ void __launch_bounds__(128)
kv_quant_pack_generic_kernel(const __half *__restrict__ x, uint32_t rows, uint32_t cols, __half *__restrict__ param,
                             uint8_t *__restrict__ q) {
    const uint32_t row = blockIdx.x;
    const int tid = threadIdx.x;
    const __half *xr = x + (size_t)row * cols;
    __shared__ float red[2][4];
    float vmax = -FLT_MAX, vmin = FLT_MAX;
    for (uint32_t i = tid; i < cols; i += 128) {
        const float f = __half2float(xr[i]);
        vmax = fmaxf(vmax, f);
        vmin = fminf(vmin, f);
    }
    vmax = warp_max(vmax);
    vmin = warp_min(vmin);
    if ((tid & 31) == 0) {
        red[0][tid >> 5] = vmax;
        red[1][tid >> 5] = vmin;
    }
    __syncthreads();
    vmax = fmaxf(fmaxf(red[0][0], red[0][1]), fmaxf(red[0][2], red[0][3]));
    vmin = fminf(fminf(red[1][0], red[1][1]), fminf(red[1][2], red[1][3]));
    __half scale, zero;
    kv_params(vmin, vmax, scale, zero);
    if (tid == 0) {
        param[(size_t)row * 2] = scale;
        param[(size_t)row * 2 + 1] = zero;
    }
    const float fs = __half2float(scale), fz = __half2float(zero);
    uint8_t *qr = q + (size_t)row * (cols >> 1);
    for (uint32_t c = tid; c < (cols >> 1); c += 128)
        qr[c] = (uint8_t)(kv_code(xr[2 * c], fs, fz) | (kv_code(xr[2 * c + 1], fs, fz) << 4));
}

}  // namespace sr

using namespace sr;

extern "C" {

int sr_rmsnorm(const void *x, int64_t rows, int64_t cols, float eps, int64_t mean_dim, void *out, void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "rmsnorm: negative size");
    if (rows == 0 || cols == 0) return SR_OK;
    SR_REQUIRE(x && out, SR_ERR_INVALID, "rmsnorm: null pointer");
    cudaStream_t st = as_stream(stream);
    const __half *xp = (const __half *)x;
    __half *op = (__half *)out;
    const uint32_t r = (uint32_t)rows, c = (uint32_t)cols;
    const float md = (float)(uint32_t)mean_dim;
    if (cols % 8 == 0 && cols <= 16384 && aligned16(x) && aligned16(out)) {
        const int64_t nvec = cols / 8;
        if (nvec <= 256) rmsnorm_kernel<1><<<r, 256, 0, st>>>(xp, r, c, eps, md, op);
        else if (nvec <= 512) rmsnorm_kernel<2><<<r, 256, 0, st>>>(xp, r, c, eps, md, op);
        else if (nvec <= 1024) rmsnorm_kernel<4><<<r, 256, 0, st>>>(xp, r, c, eps, md, op);
        else rmsnorm_kernel<8><<<r, 256, 0, st>>>(xp, r, c, eps, md, op);
    } else {
        rmsnorm_generic_kernel<<<r, 256, 0, st>>>(xp, r, c, eps, md, op);
    }
    return check_launch("rmsnorm");
}

int sr_rope_qk(void *q, void *k, const void *cosv, const void *sinv, int64_t n_seqs, int64_t seq_len,
               int64_t cos_seqs, int64_t n_q_heads, int64_t n_k_heads, int64_t head_dim, void *stream) {
    SR_REQUIRE(n_seqs >= 0 && seq_len >= 0 && n_q_heads >= 0 && n_k_heads >= 0 && head_dim >= 0, SR_ERR_INVALID,
               "rope_qk: negative size");
    SR_REQUIRE(head_dim % 2 == 0, SR_ERR_INVALID, "rope_qk expects an even head_dim");
    SR_REQUIRE(cos_seqs == 1 || cos_seqs == n_seqs, SR_ERR_INVALID, "rope_qk: cos/sin batch must be 1 or match q");
    const int64_t blocks = n_seqs * seq_len * (n_q_heads + n_k_heads);
    if (blocks == 0 || head_dim == 0) return SR_OK;
    SR_REQUIRE(q && k && cosv && sinv, SR_ERR_INVALID, "rope_qk: null pointer");
    cudaStream_t st = as_stream(stream);
    if (head_dim % 4 == 0 && aligned4(q) && aligned4(k) && aligned4(cosv) && aligned4(sinv)) {
        const int64_t total = blocks * (head_dim / 4);
        SR_REQUIRE(total < (int64_t)1 << 32, SR_ERR_UNSUPPORTED, "rope_qk: problem too large");
        rope_qk_kernel<<<(unsigned)cdiv<int64_t>(total, 128), 128, 0, st>>>(
            (__half *)q, (__half *)k, (const __half *)cosv, (const __half *)sinv, (uint32_t)seq_len,
            (uint32_t)cos_seqs, (uint32_t)n_q_heads, (uint32_t)n_k_heads, (uint32_t)head_dim, (uint32_t)total);
    } else {
        rope_qk_generic_kernel<<<(unsigned)blocks, 128, 0, st>>>((__half *)q, (__half *)k, (const __half *)cosv,
                                                                 (const __half *)sinv, (uint32_t)seq_len,
                                                                 (uint32_t)cos_seqs, (uint32_t)n_q_heads,
                                                                 (uint32_t)n_k_heads, (uint32_t)head_dim);
    }
    return check_launch("rope_qk");
}

int sr_swiglu(const void *gate, const void *up, int64_t numel, void *out, void *stream) {
    SR_REQUIRE(numel >= 0, SR_ERR_INVALID, "swiglu: negative size");
    if (numel == 0) return SR_OK;
    SR_REQUIRE(gate && up && out, SR_ERR_INVALID, "swiglu: null pointer");
    const bool vec = aligned16(gate) && aligned16(up) && aligned16(out) && numel >= 8;
    const size_t work = vec ? (size_t)numel / 8 : (size_t)numel;
    swiglu_kernel<<<(unsigned)cdiv<size_t>(work, 256), 256, 0, as_stream(stream)>>>(
        (const __half *)gate, (const __half *)up, (size_t)numel, (__half *)out, vec);
    return check_launch("swiglu");
}

int sr_kv_quant_pack(const void *x, int64_t rows, int64_t cols, void *q, void *param, void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "kv_quant_pack: negative size");
    SR_REQUIRE(cols % 2 == 0, SR_ERR_INVALID, "kv_quant_pack expects an even last dimension");
    if (rows == 0 || cols == 0) return SR_OK;
    SR_REQUIRE(x && q && param, SR_ERR_INVALID, "kv_quant_pack: null pointer");
    cudaStream_t st = as_stream(stream);
    const uint32_t r = (uint32_t)rows, c = (uint32_t)cols;
    const bool al = aligned16(x) && aligned4(q) && aligned4(param);
    if (al && cols == 128)
        kv_quant_pack_kernel<16><<<cdiv<uint32_t>(r, 16), 256, 0, st>>>((const __half *)x, r, c, (__half *)param,
                                                                        (uint8_t *)q);
    else if (al && cols == 64)
        kv_quant_pack_kernel<8><<<cdiv<uint32_t>(r, 32), 256, 0, st>>>((const __half *)x, r, c, (__half *)param,
                                                                       (uint8_t *)q);
    else if (al && cols == 256)
        kv_quant_pack_kernel<32><<<cdiv<uint32_t>(r, 8), 256, 0, st>>>((const __half *)x, r, c, (__half *)param,
                                                                       (uint8_t *)q);
    else
        kv_quant_pack_generic_kernel<<<r, 128, 0, st>>>((const __half *)x, r, c, (__half *)param, (uint8_t *)q);
    return check_launch("kv_quant_pack");
}

}  // extern "C"
