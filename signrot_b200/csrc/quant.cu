// Activation / weight quantization kernels (memory-bound, CUDA cores).
//
// Numerics follow the reference kernels op for op:
//   symmetric per-token int4   signrot/kernels/fused.cu:68-112, quant.cu:13-63
//   asymmetric per-token uint4 signrot/kernels/fused.cu:143-198, quant.cu:133-231
//   dequant epilogue           signrot/kernels/quant.cu:66-131
//   expert-indexed variants    signrot/kernels/moe.cu:60-238
//   int4 row sums, rank-1 term signrot/kernels/quant.cu:233-383
// but the data movement is new: every row is read from HBM exactly once with
// 128-bit loads, kept in registers between the range reduction and the code
// decision, and the packed codes leave with 32-bit (or wider) stores.
#include "common.cuh"
#include <cfloat>

namespace sr {

// ------------------------------------------------------------------ dynamic quant

// One row is owned by TPR threads (TPR <= 32: part of a warp, several rows per
// warp; TPR == 256: the whole CTA).  Each thread keeps NV 16-byte vectors.
// NORM (whole-CTA rows only): the row is first formed as x (+ delta, one fp16 addition, stored to
// sum_out) and normalised as rmsnorm_kernel does it (same thread-to-vector mapping, same summation
// order, so the codes equal those of the separate add / RMSNorm / quantizer launches bit for bit).
struct NormArgs {
    const __half *delta;   // optional addend (the residual branch)
    __half *sum_out;       // optional: x + delta
    __half *normed_out;    // optional: the normalised row
    float eps, mean_dim;
};

template <int TPR, int NV, bool ASYM, bool NORM = false>
__global__ void __launch_bounds__(256)
act_quant_dynamic_kernel(const __half *__restrict__ x, const int8_t *__restrict__ sign,
                         const int32_t *__restrict__ expert_ids, uint32_t rows, uint32_t cols,
                         float clip, __half *__restrict__ scale_out, __half *__restrict__ zero_out,
                         uint8_t *__restrict__ q, NormArgs na = NormArgs{}) {
    static_assert(!NORM || TPR == 256, "the fused normalisation owns a whole CTA per row");
    constexpr int ROWS_PER_CTA = 256 / TPR;
    if (NORM) {   // launched with programmatic serialization: see launch_pdl
        pdl_trigger();
        pdl_wait();
    }
    const int tid = threadIdx.x;
    const int sub = tid % TPR;  // index inside the row team
    const uint32_t row = blockIdx.x * ROWS_PER_CTA + tid / TPR;
    const bool live = row < rows;
    const uint32_t nvec = cols >> 3;  // cols % 8 == 0 on this path

    __shared__ float red[2][8];

    Vec16 v[NV];
    float vmax = ASYM ? -FLT_MAX : 0.f, vmin = FLT_MAX;
    __half2 hmax2 = __floats2half2_rn(ASYM ? -65504.f : 0.f, ASYM ? -65504.f : 0.f);
    __half2 hmin2 = __floats2half2_rn(65504.f, 65504.f);
    if constexpr (NORM) {
        __shared__ float nred[8];
        const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * cols);
        const uint4 *dr = na.delta ? reinterpret_cast<const uint4 *>(na.delta + (size_t)row * cols) : nullptr;
        uint4 *sr_o = na.sum_out ? reinterpret_cast<uint4 *>(na.sum_out + (size_t)row * cols) : nullptr;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const uint32_t vi = sub + i * TPR;
            if (vi < nvec) {
                v[i].u = __ldg(xr + vi);
                if (dr) {
                    Vec16 d;
                    d.u = __ldg(dr + vi);
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[i].h2[j] = __hadd2(v[i].h2[j], d.h2[j]);
                    if (sr_o) sr_o[vi] = v[i].u;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float f = __half2float(v[i].h[j]);
                    acc += f * f;
                }
            }
        }
        acc = warp_sum(acc);
        if ((tid & 31) == 0) nred[tid >> 5] = acc;
        __syncthreads();
        acc = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) acc += nred[w];
        const float inv = rsqrtf(acc / na.mean_dim + na.eps);
        uint4 *nr_o = na.normed_out ? reinterpret_cast<uint4 *>(na.normed_out + (size_t)row * cols) : nullptr;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const uint32_t vi = sub + i * TPR;
            if (vi < nvec) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i].h[j] = __float2half(__half2float(v[i].h[j]) * inv);
                if (nr_o) nr_o[vi] = v[i].u;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (ASYM) {
                        hmax2 = __hmax2(hmax2, v[i].h2[j]);
                        hmin2 = __hmin2(hmin2, v[i].h2[j]);
                    } else {
                        hmax2 = __hmax2(hmax2, __habs2(v[i].h2[j]));
                    }
                }
            }
        }
    } else if (live) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * cols);
        const int8_t *sr_ = sign ? sign + (size_t)(expert_ids ? expert_ids[row] : 0) * cols : nullptr;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const uint32_t vi = sub + i * TPR;
            if (vi < nvec) {
                v[i].u = __ldg(xr + vi);
                if (sr_) {
                    const uint2 s8 = *reinterpret_cast<const uint2 *>(sr_ + (size_t)vi * 8);
                    // fp16 * (+-1) is exact: flip the sign bit where sign < 0
                    uint32_t sw[2] = {s8.x, s8.y};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t b0 = (sw[j >> 1] >> ((j & 1) * 16 + 7)) & 1u;
                        const uint32_t b1 = (sw[j >> 1] >> ((j & 1) * 16 + 15)) & 1u;
                        v[i].w[j] ^= (b0 << 15) | (b1 << 31);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (ASYM) {
                        hmax2 = __hmax2(hmax2, v[i].h2[j]);
                        hmin2 = __hmin2(hmin2, v[i].h2[j]);
                    } else {
                        hmax2 = __hmax2(hmax2, __habs2(v[i].h2[j]));
                    }
                }
            }
        }
    }
    // packed fp16 maxima are exact (comparisons only); widen once
    vmax = fmaxf(__low2float(hmax2), __high2float(hmax2));
    if (ASYM) vmin = fminf(__low2float(hmin2), __high2float(hmin2));
    if (!ASYM && vmax < 0.f) vmax = 0.f;
    // team reduction
    if (TPR <= 32) {
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) {
            vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
            if (ASYM) vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
        }
    } else {
        vmax = warp_max(vmax);
        if (ASYM) vmin = warp_min(vmin);
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
    }
    if (!live) return;

    float rcp;
    int zero_i = 0;
    if (!ASYM) {
        // scale = rn_h(amax / 7); clip applied afterwards with its own rounding
        __half scale = __float2half(vmax / 7.f);
        if (clip != 1.f) scale = __float2half(__half2float(scale) * clip);
        if (sub == 0) scale_out[row] = scale;
        rcp = rcp_approx_ftz(__half2float(scale));
    } else {
        __half hmin = __float2half(vmin), hmax = __float2half(vmax);
        if (clip != 1.f) {
            hmin = __float2half(__half2float(hmin) * clip);
            hmax = __float2half(__half2float(hmax) * clip);
        }
        const __half diff = __float2half(__half2float(hmax) - __half2float(hmin));
        const __half scale = __float2half(__half2float(diff) / 15.f);
        const __half ratio = __float2half(-__half2float(hmin) / __half2float(scale));
        const __half zero = __float2half(nearbyintf(__half2float(ratio)));
        if (sub == 0) {
            scale_out[row] = scale;
            zero_out[row] = zero;
        }
        zero_i = __half2int_rn(zero);
        rcp = rcp_approx_ftz(__half2float(scale));
    }

    // Codes on packed fp16 pairs, the arithmetic of sym_code / asym_code without the conversion unit:
    // quotient rn_h(x * rcp), clamp, round half to even by the fp16 addition of 1536 (the low byte of the sum is
    // then the integer; + 8 makes signed codes non-negative until the last xor), bytes gathered with permutes.
    // A zero scale gives rcp = inf and 0 * inf = NaN (code 0 in the scalar path): a huge finite factor gives the
    // same codes without the NaN.
    const float rcp_f = fminf(rcp, 3.0e38f);
    const float zf = (float)zero_i;
    const __half2 lo_c = __floats2half2_rn(ASYM ? -zf : -8.f, ASYM ? -zf : -8.f);
    const __half2 hi_c = __floats2half2_rn(ASYM ? 15.f - zf : 7.f, ASYM ? 15.f - zf : 7.f);
    const __half2 magic = __floats2half2_rn(ASYM ? 1536.f : 1544.f, ASYM ? 1536.f : 1544.f);
    const uint32_t zero_u = (uint32_t)(zero_i & 15) * 0x00010001u;
    uint32_t *qr = reinterpret_cast<uint32_t *>(q + (size_t)row * (cols >> 1));
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const uint32_t vi = sub + i * TPR;
        if (vi < nvec) {
            uint32_t bits[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(v[i].h2[j]);
                __half2 qh = __floats2half2_rn(f.x * rcp_f, f.y * rcp_f);
                qh = __hmin2(__hmax2(qh, lo_c), hi_c);
                qh = __hadd2(qh, magic);
                bits[j] = *reinterpret_cast<uint32_t *>(&qh);
                if (ASYM) bits[j] += zero_u;
            }
            // bits[j] = halves (code of element 2j, code of element 2j + 1) in their low bytes
            const uint32_t x01 = __byte_perm(bits[0], bits[1], 0x6240), x23 = __byte_perm(bits[2], bits[3], 0x6240);
            uint32_t ev = __byte_perm(x01, x23, 0x5410), od = __byte_perm(x01, x23, 0x7632);
            if (ASYM) {
                ev &= 0x0F0F0F0Fu;
                od &= 0x0F0F0F0Fu;
            }
            uint32_t packed = ev + (od << 4);
            if (!ASYM) packed ^= 0x88888888u;
            qr[vi] = packed;
        }
    }
}

// Any column count (odd, not a multiple of 8, longer than 16384): two passes
// over the row, scalar accesses, one CTA per row.
template <bool ASYM>
__global__ void __launch_bounds__(256)
act_quant_dynamic_generic_kernel(const __half *__restrict__ x, const int8_t *__restrict__ sign,
                                 const int32_t *__restrict__ expert_ids, uint32_t rows, uint32_t cols,
                                 uint32_t cols_dst, float clip, __half *__restrict__ scale_out,
                                 __half *__restrict__ zero_out, uint8_t *__restrict__ q) {
    const uint32_t row = blockIdx.x;
    const int tid = threadIdx.x;
    const __half *xr = x + (size_t)row * cols;
    const int8_t *sr_ = sign ? sign + (size_t)(expert_ids ? expert_ids[row] : 0) * cols : nullptr;
    __shared__ float red[2][8];
    auto ld = [&](uint32_t i) {
        __half h = xr[i];
        if (sr_ && sr_[i] < 0) h = __hneg(h);
        return h;
    };
    float vmax = ASYM ? -FLT_MAX : 0.f, vmin = FLT_MAX;
    for (uint32_t i = tid; i < cols; i += 256) {
        const float f = __half2float(ld(i));
        if (ASYM) {
            vmax = fmaxf(vmax, f);
            vmin = fminf(vmin, f);
        } else {
            vmax = fmaxf(vmax, fabsf(f));
        }
    }
    vmax = warp_max(vmax);
    vmin = warp_min(vmin);
    if ((tid & 31) == 0) {
        red[0][tid >> 5] = vmax;
        red[1][tid >> 5] = vmin;
    }
    __syncthreads();
    vmax = red[0][0];
    vmin = red[1][0];
    for (int w = 1; w < 8; ++w) {
        vmax = fmaxf(vmax, red[0][w]);
        vmin = fminf(vmin, red[1][w]);
    }
    float rcp;
    int zero_i = 0;
    if (!ASYM) {
        __half scale = __float2half(vmax / 7.f);
        if (clip != 1.f) scale = __float2half(__half2float(scale) * clip);
        if (tid == 0) scale_out[row] = scale;
        rcp = rcp_approx_ftz(__half2float(scale));
    } else {
        __half hmin = __float2half(vmin), hmax = __float2half(vmax);
        if (clip != 1.f) {
            hmin = __float2half(__half2float(hmin) * clip);
            hmax = __float2half(__half2float(hmax) * clip);
        }
        const __half diff = __float2half(__half2float(hmax) - __half2float(hmin));
        const __half scale = __float2half(__half2float(diff) / 15.f);
        const __half ratio = __float2half(-__half2float(hmin) / __half2float(scale));
        const __half zero = __float2half(nearbyintf(__half2float(ratio)));
        if (tid == 0) {
            scale_out[row] = scale;
            zero_out[row] = zero;
        }
        zero_i = __half2int_rn(zero);
        rcp = rcp_approx_ftz(__half2float(scale));
    }
    uint8_t *qr = q + (size_t)row * cols_dst;
    for (uint32_t c = tid; c < cols_dst; c += 256) {
        uint32_t b = 0;
        for (int j = 0; j < 2; ++j) {
            const uint32_t i = 2 * c + j;
            if (i < cols) {
                const int code = ASYM ? asym_code(ld(i), rcp, zero_i, 0, 15) : sym_code(ld(i), rcp);
                b |= (uint32_t)(code & 15) << (4 * j);
            }
        }
        qr[c] = (uint8_t)b;
    }
}

template <bool ASYM>
static int launch_act_quant(const __half *x, const int8_t *sign, const int32_t *eids, int64_t rows,
                            int64_t cols, float clip, __half *scale, __half *zero, uint8_t *q,
                            cudaStream_t st) {
    if (rows == 0 || cols == 0) return SR_OK;
    const uint32_t r = (uint32_t)rows, c = (uint32_t)cols;
    const bool vec = (cols % 8 == 0) && cols <= 16384 && aligned16(x) && aligned4(q) &&
                     (!sign || (reinterpret_cast<uintptr_t>(sign) % 8 == 0));
    if (!vec) {
        act_quant_dynamic_generic_kernel<ASYM><<<r, 256, 0, st>>>(x, sign, eids, r, c, (uint32_t)((cols + 1) / 2),
                                                              clip, scale, zero, q);
        return check_launch("act_quant_dynamic_generic");
    }
#define SR_LAUNCH_AQ(TPR, NV)                                                                        \
    act_quant_dynamic_kernel<TPR, NV, ASYM><<<cdiv<uint32_t>(r, 256 / TPR), 256, 0, st>>>(           \
        x, sign, eids, r, c, clip, scale, zero, q)
    const int64_t nvec = cols / 8;
    if (nvec <= 16) SR_LAUNCH_AQ(16, 1);          // head_dim-sized rows: 16 rows per CTA
    else if (nvec <= 32) SR_LAUNCH_AQ(32, 1);
    else if (nvec <= 64) SR_LAUNCH_AQ(32, 2);
    else if (nvec <= 128) SR_LAUNCH_AQ(32, 4);
    else if (nvec <= 256) SR_LAUNCH_AQ(256, 1);
    else if (nvec <= 512) SR_LAUNCH_AQ(256, 2);
    else if (nvec <= 1024) SR_LAUNCH_AQ(256, 4);
    else SR_LAUNCH_AQ(256, 8);
#undef SR_LAUNCH_AQ
    return check_launch("act_quant_dynamic");
}

// ------------------------------------------------------------------ given-scale quant

// mode 0: symmetric s4; 1: asymmetric s4 (clamp -8..7); 2: asymmetric u4 (clamp 0..15)
template <int MODE>
__global__ void __launch_bounds__(256)
quant_given_scale_kernel(const __half *__restrict__ x, const __half *__restrict__ scale,
                         const __half *__restrict__ zero, uint32_t rows, uint32_t cols, uint32_t cols_dst,
                         uint8_t *__restrict__ q) {
    // one thread per output byte pair group: 8 elements when possible
    const uint32_t words_per_row = cdiv<uint32_t>(cols, 8);
    const size_t gid = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (gid >= (size_t)rows * words_per_row) return;
    const uint32_t row = gid / words_per_row, w = gid % words_per_row;
    const float rcp = rcp_approx_ftz(__half2float(scale[row]));
    const int z = MODE == 0 ? 0 : __half2int_rn(zero[row]);
    const __half *xr = x + (size_t)row * cols;
    uint8_t *qr = q + (size_t)row * cols_dst;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const uint32_t c = w * 4 + b;
        if (c >= cols_dst) break;
        uint32_t byte = 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t i = 2 * c + j;
            if (i < cols) {
                int code;
                if (MODE == 0) code = sym_code(xr[i], rcp);
                else if (MODE == 1) code = asym_code(xr[i], rcp, z, -8, 7);
                else code = asym_code(xr[i], rcp, z, 0, 15);
                byte |= (uint32_t)(code & 15) << (4 * j);
            }
        }
        qr[c] = (uint8_t)byte;
    }
}

template <int MODE>
static int launch_quant_given(const __half *x, const __half *scale, const __half *zero, int64_t rows,
                              int64_t cols, uint8_t *q, cudaStream_t st) {
    if (rows == 0 || cols == 0) return SR_OK;
    const size_t n = (size_t)rows * cdiv<int64_t>(cols, 8);
    quant_given_scale_kernel<MODE><<<(unsigned)cdiv<size_t>(n, 256), 256, 0, st>>>(
        x, scale, zero, (uint32_t)rows, (uint32_t)cols, (uint32_t)((cols + 1) / 2), q);
    return check_launch("quant_given_scale");
}

// ------------------------------------------------------------------ dequant

// out = rn_h((float(q - zero*wsum) * s_row) * s_col); expert tables are indexed by
// expert_ids[row] when given (w_scales / w_sum are then [E, cols]).
template <bool VEC>
__global__ void __launch_bounds__(256)
dequant_kernel(const int32_t *__restrict__ q, const __half *__restrict__ scale_row,
               const __half *__restrict__ scale_col, const int32_t *__restrict__ expert_ids,
               const int8_t *__restrict__ zero_row, const int32_t *__restrict__ w_sum, uint32_t rows,
               uint32_t cols, __half *__restrict__ out) {
    constexpr int W = VEC ? 8 : 1;
    const uint32_t groups = cdiv<uint32_t>(cols, W);
    const size_t gid = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (gid >= (size_t)rows * groups) return;
    const uint32_t row = gid / groups, c0 = (gid % groups) * W;
    const size_t e_off = expert_ids ? (size_t)expert_ids[row] * cols : 0;
    const float sr_ = __half2float(scale_row[row]);
    const int32_t z = zero_row ? (int32_t)zero_row[row] : 0;
    if (VEC) {
        const int4 *qp = reinterpret_cast<const int4 *>(q + (size_t)row * cols + c0);
        int4 a = __ldg(qp), b = __ldg(qp + 1);
        int32_t v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        Vec16 sc, o;
        sc.u = __ldg(reinterpret_cast<const uint4 *>(scale_col + e_off + c0));
        if (zero_row) {
            const int4 *wp = reinterpret_cast<const int4 *>(w_sum + e_off + c0);
            int4 wa = __ldg(wp), wb = __ldg(wp + 1);
            int32_t ws[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] -= z * ws[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            o.h[j] = __float2half_rn(((float)v[j] * sr_) * __half2float(sc.h[j]));
        *reinterpret_cast<uint4 *>(out + (size_t)row * cols + c0) = o.u;
    } else {
        int32_t v = q[(size_t)row * cols + c0];
        if (zero_row) v -= z * w_sum[e_off + c0];
        out[(size_t)row * cols + c0] = __float2half_rn(((float)v * sr_) * __half2float(scale_col[e_off + c0]));
    }
}

static int launch_dequant(const int32_t *q, const __half *srow, const __half *scol, const int32_t *eids,
                          const int8_t *zero_row, const int32_t *wsum, int64_t rows, int64_t cols,
                          __half *out, cudaStream_t st) {
    if (rows == 0 || cols == 0) return SR_OK;
    const bool vec = cols % 8 == 0 && aligned16(q) && aligned16(scol) && aligned16(out) &&
                     (!wsum || aligned16(wsum));
    const size_t n = (size_t)rows * (vec ? cols / 8 : cols);
    const unsigned grid = (unsigned)cdiv<size_t>(n, 256);
    if (vec)
        dequant_kernel<true><<<grid, 256, 0, st>>>(q, srow, scol, eids, zero_row, wsum, (uint32_t)rows,
                                                   (uint32_t)cols, out);
    else
        dequant_kernel<false><<<grid, 256, 0, st>>>(q, srow, scol, eids, zero_row, wsum, (uint32_t)rows,
                                                    (uint32_t)cols, out);
    return check_launch("dequant");
}

// ------------------------------------------------------------------ int4 row sums, rank-1 term

template <bool SIGNED>
__global__ void __launch_bounds__(256)
sum_i4_kernel(const uint8_t *__restrict__ x, uint32_t rows, uint32_t packed_cols, int32_t *__restrict__ out) {
    // one warp per row
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint8_t *xr = x + (size_t)row * packed_cols;
    int acc = 0;
    auto add_word = [&](uint32_t w) {
        // nibble sums via SWAR: low and high nibbles of each byte
        const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
        uint32_t s = lo + hi;                    // per byte <= 30
        s = (s & 0x00FF00FFu) + ((s >> 8) & 0x00FF00FFu);
        int total = (int)((s & 0xFFFFu) + (s >> 16));
        if (SIGNED) total -= 16 * __popc(w & 0x88888888u);  // each nibble >= 8 stands for n - 16
        acc += total;
    };
    const bool al = (reinterpret_cast<uintptr_t>(xr) & 3u) == 0;
    uint32_t done = 0;
    if (al) {
        const uint32_t nw = packed_cols >> 2;
        const uint32_t *xw = reinterpret_cast<const uint32_t *>(xr);
        for (uint32_t i = lane; i < nw; i += 32) add_word(__ldg(xw + i));
        done = nw << 2;
    }
    for (uint32_t i = done + lane; i < packed_cols; i += 32) add_word((uint32_t)xr[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[row] = acc;
}

__global__ void __launch_bounds__(256)
colrow_kernel(const int8_t *__restrict__ a_col, const int32_t *__restrict__ b_row, uint32_t rows,
              uint32_t cols, int32_t *__restrict__ out) {
    const size_t gid = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (gid >= (size_t)rows * cols) return;
    const uint32_t row = gid / cols, col = gid % cols;
    out[gid] = (int32_t)a_col[row] * b_row[col];
}

}  // namespace sr

// =================================================================== C ABI

using namespace sr;

extern "C" {

int sr_sym_quant_dynamic(const void *x, int64_t rows, int64_t cols, float clip_ratio, void *q, void *scale,
                         void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "sym_quant_dynamic: negative size");
    SR_REQUIRE(rows == 0 || cols == 0 || (x && q && scale), SR_ERR_INVALID, "sym_quant_dynamic: null pointer");
    return launch_act_quant<false>((const __half *)x, nullptr, nullptr, rows, cols, clip_ratio, (__half *)scale,
                                   nullptr, (uint8_t *)q, as_stream(stream));
}

int sr_asym_quant_dynamic(const void *x, int64_t rows, int64_t cols, float clip_ratio, void *q, void *scale,
                          void *zero, void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "asym_quant_dynamic: negative size");
    SR_REQUIRE(rows == 0 || cols == 0 || (x && q && scale && zero), SR_ERR_INVALID,
               "asym_quant_dynamic: null pointer");
    return launch_act_quant<true>((const __half *)x, nullptr, nullptr, rows, cols, clip_ratio, (__half *)scale,
                                  (__half *)zero, (uint8_t *)q, as_stream(stream));
}

int sr_add_rmsnorm_quant(const void *x, const void *delta, int64_t rows, int64_t cols, float eps, int64_t mean_dim,
                         float clip_ratio, int asym, void *sum_out, void *normed_out, void *q, void *scale,
                         void *zero, void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "add_rmsnorm_quant: negative size");
    if (rows == 0 || cols == 0) return SR_OK;
    SR_REQUIRE(x && q && scale && (!asym || zero), SR_ERR_INVALID, "add_rmsnorm_quant: null pointer");
    SR_REQUIRE(!sum_out || delta, SR_ERR_INVALID, "add_rmsnorm_quant: sum_out without an addend");
    SR_REQUIRE(cols % 8 == 0 && cols <= 16384 && aligned16(x) && aligned4(q) && (!delta || aligned16(delta)) &&
                   (!sum_out || aligned16(sum_out)) && (!normed_out || aligned16(normed_out)),
               SR_ERR_UNSUPPORTED, "add_rmsnorm_quant: rows must be 16-byte aligned, cols a multiple of 8 and <= 16384");
    const uint32_t r = (uint32_t)rows, c = (uint32_t)cols;
    cudaStream_t st = (cudaStream_t)stream;
    NormArgs na{(const __half *)delta, (__half *)sum_out, (__half *)normed_out, eps, (float)mean_dim};
    const int64_t nvec = cols / 8;
#define SR_LAUNCH_NQ(NV)                                                                                         \
    do {                                                                                                         \
        if (asym)                                                                                                \
            launch_pdl(act_quant_dynamic_kernel<256, NV, true, true>, dim3(r), dim3(256), 0, st,                 \
                       (const __half *)x, nullptr, nullptr, r, c, clip_ratio, (__half *)scale, (__half *)zero, (uint8_t *)q, na); \
        else                                                                                                     \
            launch_pdl(act_quant_dynamic_kernel<256, NV, false, true>, dim3(r), dim3(256), 0, st,                \
                       (const __half *)x, nullptr, nullptr, r, c, clip_ratio, (__half *)scale, nullptr, (uint8_t *)q, na); \
    } while (0)
    if (nvec <= 256) SR_LAUNCH_NQ(1);
    else if (nvec <= 512) SR_LAUNCH_NQ(2);
    else if (nvec <= 1024) SR_LAUNCH_NQ(4);
    else SR_LAUNCH_NQ(8);
#undef SR_LAUNCH_NQ
    return check_launch("add_rmsnorm_quant");
}

int sr_sym_quant_dynamic_moe(const void *x, const void *sign, const void *expert_ids, int64_t rows, int64_t cols,
                             float clip_ratio, void *q, void *scale, void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "sym_quant_dynamic_moe: negative size");
    SR_REQUIRE(rows == 0 || cols == 0 || (x && q && scale && expert_ids), SR_ERR_INVALID,
               "sym_quant_dynamic_moe: null pointer");
    return launch_act_quant<false>((const __half *)x, (const int8_t *)sign, (const int32_t *)expert_ids, rows, cols,
                                   clip_ratio, (__half *)scale, nullptr, (uint8_t *)q, as_stream(stream));
}

int sr_asym_quant_dynamic_moe(const void *x, const void *sign, const void *expert_ids, int64_t rows, int64_t cols,
                              float clip_ratio, void *q, void *scale, void *zero, void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "asym_quant_dynamic_moe: negative size");
    SR_REQUIRE(rows == 0 || cols == 0 || (x && q && scale && zero && expert_ids), SR_ERR_INVALID,
               "asym_quant_dynamic_moe: null pointer");
    return launch_act_quant<true>((const __half *)x, (const int8_t *)sign, (const int32_t *)expert_ids, rows, cols,
                                  clip_ratio, (__half *)scale, (__half *)zero, (uint8_t *)q, as_stream(stream));
}

int sr_sym_quant(const void *x, const void *scale, int64_t rows, int64_t cols, void *q, void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "sym_quant: negative size");
    SR_REQUIRE(rows == 0 || cols == 0 || (x && scale && q), SR_ERR_INVALID, "sym_quant: null pointer");
    return launch_quant_given<0>((const __half *)x, (const __half *)scale, nullptr, rows, cols, (uint8_t *)q,
                                 as_stream(stream));
}

int sr_asym_quant_f16_si4(const void *x, const void *scale, const void *zero, int64_t rows, int64_t cols, void *q,
                          void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "asym_quant_f16_si4: negative size");
    SR_REQUIRE(rows == 0 || cols == 0 || (x && scale && zero && q), SR_ERR_INVALID,
               "asym_quant_f16_si4: null pointer");
    return launch_quant_given<1>((const __half *)x, (const __half *)scale, (const __half *)zero, rows, cols,
                                 (uint8_t *)q, as_stream(stream));
}

int sr_asym_quant_f16_ui4(const void *x, const void *scale, const void *zero, int64_t rows, int64_t cols, void *q,
                          void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "asym_quant_f16_ui4: negative size");
    SR_REQUIRE(rows == 0 || cols == 0 || (x && scale && zero && q), SR_ERR_INVALID,
               "asym_quant_f16_ui4: null pointer");
    return launch_quant_given<2>((const __half *)x, (const __half *)scale, (const __half *)zero, rows, cols,
                                 (uint8_t *)q, as_stream(stream));
}

int sr_sym_dequant(const void *q, const void *scale_row, const void *scale_col, int64_t rows, int64_t cols,
                   void *out, void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "sym_dequant: negative size");
    SR_REQUIRE(rows == 0 || cols == 0 || (q && scale_row && scale_col && out), SR_ERR_INVALID,
               "sym_dequant: null pointer");
    return launch_dequant((const int32_t *)q, (const __half *)scale_row, (const __half *)scale_col, nullptr, nullptr,
                          nullptr, rows, cols, (__half *)out, as_stream(stream));
}

int sr_sym_dequant_moe(const void *q, const void *scale_row, const void *w_scales, const void *expert_ids,
                       const void *zero_row, const void *w_sum, int64_t rows, int64_t cols, void *out,
                       void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "sym_dequant_moe: negative size");
    SR_REQUIRE((zero_row == nullptr) == (w_sum == nullptr), SR_ERR_INVALID,
               "sym_dequant_moe: zero_row and w_sum must be given together");
    SR_REQUIRE(rows == 0 || cols == 0 || (q && scale_row && w_scales && expert_ids && out), SR_ERR_INVALID,
               "sym_dequant_moe: null pointer");
    return launch_dequant((const int32_t *)q, (const __half *)scale_row, (const __half *)w_scales,
                          (const int32_t *)expert_ids, (const int8_t *)zero_row, (const int32_t *)w_sum, rows, cols,
                          (__half *)out, as_stream(stream));
}

int sr_sum_i4(const void *x, int64_t rows, int64_t packed_cols, int is_signed, void *out, void *stream) {
    SR_REQUIRE(rows >= 0 && packed_cols >= 0, SR_ERR_INVALID, "sum_i4: negative size");
    if (rows == 0) return SR_OK;
    SR_REQUIRE(x && out, SR_ERR_INVALID, "sum_i4: null pointer");
    const unsigned grid = (unsigned)cdiv<int64_t>(rows, 8);
    if (is_signed)
        sum_i4_kernel<true><<<grid, 256, 0, as_stream(stream)>>>((const uint8_t *)x, (uint32_t)rows,
                                                                  (uint32_t)packed_cols, (int32_t *)out);
    else
        sum_i4_kernel<false><<<grid, 256, 0, as_stream(stream)>>>((const uint8_t *)x, (uint32_t)rows,
                                                                   (uint32_t)packed_cols, (int32_t *)out);
    return check_launch("sum_i4");
}

int sr_matmul_colrow_i8_i32(const void *a_col, const void *b_row, int64_t rows, int64_t cols, void *out,
                            void *stream) {
    SR_REQUIRE(rows >= 0 && cols >= 0, SR_ERR_INVALID, "matmul_colrow_i8_i32: negative size");
    if (rows == 0 || cols == 0) return SR_OK;
    SR_REQUIRE(a_col && b_row && out, SR_ERR_INVALID, "matmul_colrow_i8_i32: null pointer");
    const size_t n = (size_t)rows * cols;
    colrow_kernel<<<(unsigned)cdiv<size_t>(n, 256), 256, 0, as_stream(stream)>>>(
        (const int8_t *)a_col, (const int32_t *)b_row, (uint32_t)rows, (uint32_t)cols, (int32_t *)out);
    return check_launch("matmul_colrow_i8_i32");
}

}  // extern "C"
