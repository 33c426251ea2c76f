// Routing of a sparse MoE block as three launches instead of some forty small tensor-library ones
// (signrot/nn/moe.py:159-236 of the reference: softmax, top-k, renormalisation, counting, stable
// sort by expert, gathers, un-permute and weighted sum).
//
//   moe_route_kernel    router logits [T, E] fp16 -> fp32 softmax, top-k (ties: lowest index),
//                       optional renormalisation, fp16 routing weights [T, k]; rows (t, j) sorted by
//                       expert, token order kept inside an expert: tok[R], eid[R], inv[R] (position
//                       of row t*k+j in the sorted order), row_off[E + 1].   R = T * k.
//   moe_gather_kernel   packed codes / scales / zeros of every token -> one copy per routed row.
//   moe_combine_kernel  out[t] = sum_j rn_h(y[inv[t*k+j]] * w[t, j]), fp32 sum, one fp16 rounding.
//
// The route kernel is one CTA: T * E and T * k are small next to the expert GEMMs it feeds (decode:
// 64 tokens; prefill: a few thousand), and a single CTA needs no grid-wide ordering to be
// deterministic.  Nothing here synchronises with the host or depends on data-dependent shapes.
#include "common.cuh"
#include <cfloat>

namespace sr {

namespace {

constexpr int RT_THREADS = 1024;
constexpr int RT_MAX_EXPERTS = 512;
constexpr int RT_MAX_TOPK = 8;

// softmax + top-k of one token by one warp; lane l owns experts l, l + 32, ... (EPL of them).  Result j of the top-k
// lives in lane j until the end, so nothing is indexed at run time.  `stage`: shared-memory copy of the chosen ids, or null.
template <int EPL>
__device__ __forceinline__ void route_token_n(const __half *__restrict__ logits, uint32_t t, uint32_t E, uint32_t k,
                                              int renorm, __half *__restrict__ weights, int32_t *__restrict__ chosen,
                                              uint16_t *stage, int lane) {
    float p[EPL];
    float mx = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const uint32_t e = lane + 32 * i;
        float v = e < E ? __half2float(logits[(size_t)t * E + e]) : -FLT_MAX;
        // non-finite logits (an overflowed router) must still give k valid expert ids: NaN ranks highest, as in
        // the tensor library's top-k, infinities become the largest finite values
        v = (v != v) ? FLT_MAX : fminf(fmaxf(v, -FLT_MAX), FLT_MAX);
        p[i] = v;
        mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const uint32_t e = lane + 32 * i;
        p[i] = e < E ? expf(p[i] - mx) : 0.f;
        sum += p[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < EPL; ++i) p[i] = (lane + 32 * i) < E ? p[i] / sum : -1.f;
    float my_v = 0.f, tot = 0.f;
    int my_i = 0;
    for (uint32_t j = 0; j < k; ++j) {
        // this lane's best, then the warp's best; equal values: the lower expert index wins
        float bv = -1.f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < EPL; ++i)
            if (p[i] > bv) {
                bv = p[i];
                bi = lane + 32 * i;
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        bi = min(bi, (int)E - 1);               // always an id a weight stack has
        if (lane == (int)j) {
            my_v = bv;
            my_i = bi;
        }
        tot += bv;
#pragma unroll
        for (int i = 0; i < EPL; ++i)
            if (lane + 32 * i == bi) p[i] = -1.f;   // taken
    }
    if ((uint32_t)lane < k) {
        const float w = renorm ? my_v / tot : my_v;
        weights[(size_t)t * k + lane] = __float2half_rn(w);
        chosen[(size_t)t * k + lane] = my_i;
        if (stage != nullptr) stage[(size_t)t * k + lane] = (uint16_t)my_i;
    }
}

__device__ __forceinline__ void route_token(const __half *__restrict__ logits, uint32_t t, uint32_t E, uint32_t k,
                                            int renorm, __half *__restrict__ weights, int32_t *__restrict__ chosen,
                                            uint16_t *stage, int lane) {
    if (E <= 32) route_token_n<1>(logits, t, E, k, renorm, weights, chosen, stage, lane);
    else if (E <= 128) route_token_n<4>(logits, t, E, k, renorm, weights, chosen, stage, lane);
    else route_token_n<RT_MAX_EXPERTS / 32>(logits, t, E, k, renorm, weights, chosen, stage, lane);
}

// many tokens: the per-token part on a grid of its own (8 tokens per CTA)
__global__ void __launch_bounds__(256)
moe_topk_kernel(const __half *__restrict__ logits, uint32_t T, uint32_t E, uint32_t k, int renorm,
                __half *__restrict__ weights, int32_t *__restrict__ chosen) {
    pdl_trigger();
    pdl_wait();
    const uint32_t t = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t < T) route_token(logits, t, E, k, renorm, weights, chosen, nullptr, threadIdx.x & 31);
}

__global__ void __launch_bounds__(RT_THREADS)
moe_route_kernel(const __half *__restrict__ logits, uint32_t T, uint32_t E, uint32_t k, int renorm, int do_topk,
                 int staged, __half *__restrict__ weights, int32_t *__restrict__ chosen, int32_t *__restrict__ tok,
                 int32_t *__restrict__ eid, int32_t *__restrict__ inv, int32_t *__restrict__ row_off) {
    extern __shared__ uint16_t chosen_sh[];   // the routed rows' experts, when they fit (staged)
    __shared__ int32_t counts[RT_MAX_EXPERTS];
    __shared__ int32_t start[RT_MAX_EXPERTS + 1];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int WARPS = RT_THREADS / 32;
    const uint32_t R = T * k;

    if (do_topk)
        for (uint32_t t = warp; t < T; t += WARPS)
            route_token(logits, t, E, k, renorm, weights, chosen, staged ? chosen_sh : nullptr, lane);
    for (uint32_t e = tid; e < E; e += RT_THREADS) counts[e] = 0;
    __syncthreads();   // also orders the global writes of `chosen` before the reads below (one CTA)
    if (staged && !do_topk) {     // the ids come from the top-k kernel: stage them (with do_topk they already are)
        for (uint32_t r = tid; r < R; r += RT_THREADS) chosen_sh[r] = (uint16_t)chosen[r];
        __syncthreads();
    }
    auto expert_of = [&](uint32_t r) { return staged ? (int32_t)chosen_sh[r] : chosen[r]; };

    // ---- rows per expert: warp w counts experts w, w + WARPS, ... with ballots over the rows in order
    for (uint32_t e = warp; e < E; e += WARPS) {
        int c = 0;
        for (uint32_t i = 0; i < R; i += 32) {
            const bool mine = i + lane < R && expert_of(i + lane) == (int32_t)e;
            c += __popc(__ballot_sync(0xffffffffu, mine));
        }
        if (lane == 0) counts[e] = c;
    }
    __syncthreads();
    if (warp == 0) {   // exclusive scan over at most 512 experts: 16 per lane
        int local[RT_MAX_EXPERTS / 32];
        int s = 0;
#pragma unroll
        for (int i = 0; i < RT_MAX_EXPERTS / 32; ++i) {
            const uint32_t e = lane * (RT_MAX_EXPERTS / 32) + i;
            local[i] = e < E ? counts[e] : 0;
            s += local[i];
        }
        int incl = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        int run = incl - s;
#pragma unroll
        for (int i = 0; i < RT_MAX_EXPERTS / 32; ++i) {
            const uint32_t e = lane * (RT_MAX_EXPERTS / 32) + i;
            if (e < E) {
                start[e] = run;
                row_off[e] = run;
            }
            run += local[i];
        }
        if (lane == 31) {
            start[E] = incl;
            row_off[E] = incl;
        }
    }
    __syncthreads();

    // ---- placement, token order kept inside an expert
    for (uint32_t e = warp; e < E; e += WARPS) {
        int base = start[e];
        for (uint32_t i = 0; i < R; i += 32) {
            const uint32_t r = i + lane;
            const bool mine = r < R && expert_of(r) == (int32_t)e;
            const uint32_t mask = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int pos = base + __popc(mask & ((1u << lane) - 1u));
                tok[pos] = (int32_t)(r / k);
                eid[pos] = (int32_t)e;
                inv[r] = pos;
            }
            base += __popc(mask);
        }
    }
}

// one warp per routed row: 16-byte pieces of the packed codes, lane 0 the scale (and zero)
__global__ void __launch_bounds__(256)
moe_gather_kernel(const uint8_t *__restrict__ q, const __half *__restrict__ scale, const int8_t *__restrict__ zero,
                  const int32_t *__restrict__ tok, uint32_t R, uint32_t row_bytes, uint8_t *__restrict__ q_out,
                  __half *__restrict__ scale_out, int8_t *__restrict__ zero_out) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const uint32_t r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= R) return;
    const uint32_t t = (uint32_t)tok[r];
    const uint4 *src = reinterpret_cast<const uint4 *>(q + (size_t)t * row_bytes);
    uint4 *dst = reinterpret_cast<uint4 *>(q_out + (size_t)r * row_bytes);
    for (uint32_t i = lane; i < row_bytes / 16; i += 32) dst[i] = __ldg(src + i);
    if (lane == 0) {
        scale_out[r] = scale[t];
        if (zero) zero_out[r] = zero[t];
    }
}

// one CTA per token, 8 values per thread and step.  row_range (optional, two int32 on the device): only sorted rows
// lo <= r < hi contribute (an expert-parallel rank owns a contiguous range of the sorted rows); OUT32: the fp32 sum
// is written unrounded, for a sum across ranks.
template <bool OUT32>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __half *__restrict__ y, const __half *__restrict__ weights, const int32_t *__restrict__ inv,
                   const int32_t *__restrict__ row_range, uint32_t T, uint32_t k, uint32_t hid, void *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const uint32_t t = blockIdx.x;
    const int32_t lo = row_range ? row_range[0] : 0, hi = row_range ? row_range[1] : 0x7fffffff;
    for (uint32_t c = threadIdx.x * 8; c < hid; c += 256 * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (uint32_t j = 0; j < k; ++j) {
            const int32_t r = inv[(size_t)t * k + j];
            if (r < lo || r >= hi) continue;
            const float w = __half2float(weights[(size_t)t * k + j]);
            Vec16 v;
            v.u = __ldg(reinterpret_cast<const uint4 *>(y + (size_t)r * hid + c));
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += __half2float(__float2half_rn(__half2float(v.h[i]) * w));
        }
        if (OUT32) {
            float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + (size_t)t * hid + c);
            dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        } else {
            Vec16 o;
#pragma unroll
            for (int i = 0; i < 8; ++i) o.h[i] = __float2half_rn(acc[i]);
            *reinterpret_cast<uint4 *>(reinterpret_cast<__half *>(out) + (size_t)t * hid + c) = o.u;
        }
    }
}

}  // namespace

}  // namespace sr

using namespace sr;

extern "C" {

int sr_moe_route(const void *logits, int64_t tokens, int64_t num_experts, int64_t top_k, int renormalize,
                 void *weights, void *chosen, void *tok, void *eid, void *inv, void *row_offsets, void *stream) {
    SR_REQUIRE(tokens >= 0 && num_experts >= 1 && top_k >= 1, SR_ERR_INVALID, "moe_route: bad size");
    SR_REQUIRE(num_experts <= RT_MAX_EXPERTS && top_k <= RT_MAX_TOPK && top_k <= num_experts, SR_ERR_UNSUPPORTED,
               "moe_route: at most %d experts and top-%d", RT_MAX_EXPERTS, RT_MAX_TOPK);
    SR_REQUIRE(tokens * top_k < (1ll << 31), SR_ERR_UNSUPPORTED, "moe_route: too many routed rows");
    SR_REQUIRE(row_offsets && (tokens == 0 || (logits && weights && chosen && tok && eid && inv)), SR_ERR_INVALID,
               "moe_route: null pointer");
    cudaStream_t st = as_stream(stream);
    const int64_t R = tokens * top_k;
    const int do_topk = tokens <= 256;                  // few tokens: everything in the one CTA
    if (!do_topk)
        launch_pdl(moe_topk_kernel, dim3((unsigned)cdiv<int64_t>(tokens, 8)), dim3(256), 0, st, (const __half *)logits,
                   (uint32_t)tokens, (uint32_t)num_experts, (uint32_t)top_k, renormalize, (__half *)weights,
                   (int32_t *)chosen);
    const int staged = R * 2 <= 200 * 1024;
    const size_t smem = staged ? (size_t)R * 2 : 0;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "moe_route: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    launch_pdl(moe_route_kernel, dim3(1), dim3(RT_THREADS), smem, st, (const __half *)logits, (uint32_t)tokens,
               (uint32_t)num_experts, (uint32_t)top_k, renormalize, do_topk, staged, (__half *)weights, (int32_t *)chosen,
               (int32_t *)tok, (int32_t *)eid, (int32_t *)inv, (int32_t *)row_offsets);
    return check_launch("moe_route");
}

int sr_moe_gather(const void *q, const void *scale, const void *zero, const void *tok, int64_t rows, int64_t row_bytes,
                  void *q_out, void *scale_out, void *zero_out, void *stream) {
    SR_REQUIRE(rows >= 0 && row_bytes >= 0, SR_ERR_INVALID, "moe_gather: negative size");
    if (rows == 0) return SR_OK;
    SR_REQUIRE(q && scale && tok && q_out && scale_out && (!zero || zero_out), SR_ERR_INVALID, "moe_gather: null pointer");
    SR_REQUIRE(row_bytes % 16 == 0 && aligned16(q) && aligned16(q_out), SR_ERR_UNSUPPORTED,
               "moe_gather: packed rows must be multiples of 16 bytes");
    launch_pdl(moe_gather_kernel, dim3((unsigned)cdiv<int64_t>(rows, 8)), dim3(256), 0, as_stream(stream),
               (const uint8_t *)q, (const __half *)scale, (const int8_t *)zero, (const int32_t *)tok, (uint32_t)rows,
               (uint32_t)row_bytes, (uint8_t *)q_out, (__half *)scale_out, (int8_t *)zero_out);
    return check_launch("moe_gather");
}

int sr_moe_combine(const void *y, const void *weights, const void *inv, const void *row_range, int64_t tokens,
                   int64_t top_k, int64_t hidden, int out_f32, void *out, void *stream) {
    SR_REQUIRE(tokens >= 0 && top_k >= 1 && hidden >= 0, SR_ERR_INVALID, "moe_combine: bad size");
    if (tokens == 0 || hidden == 0) return SR_OK;
    SR_REQUIRE(y && weights && inv && out, SR_ERR_INVALID, "moe_combine: null pointer");
    SR_REQUIRE(hidden % 8 == 0 && aligned16(y) && aligned16(out), SR_ERR_UNSUPPORTED,
               "moe_combine: hidden must be a multiple of 8 and rows 16-byte aligned");
    if (out_f32)
        launch_pdl(moe_combine_kernel<true>, dim3((unsigned)tokens), dim3(256), 0, as_stream(stream), (const __half *)y,
                   (const __half *)weights, (const int32_t *)inv, (const int32_t *)row_range, (uint32_t)tokens,
                   (uint32_t)top_k, (uint32_t)hidden, out);
    else
        launch_pdl(moe_combine_kernel<false>, dim3((unsigned)tokens), dim3(256), 0, as_stream(stream), (const __half *)y,
                   (const __half *)weights, (const int32_t *)inv, (const int32_t *)row_range, (uint32_t)tokens,
                   (uint32_t)top_k, (uint32_t)hidden, out);
    return check_launch("moe_combine");
}

}  // extern "C"
