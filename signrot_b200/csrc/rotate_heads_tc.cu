// Fused head-wise online rotation + sign + per-token int4 quantization for the o_proj input of a
// 32-head, head_dim-128 model: y = (H32 (x) I128) x / sqrt(32), the transform runs ACROSS the heads
// for every position inside a head (fake_quant/quant_utils.py:287-291, signrot/functional/hadamard.py:78-87
// with had_dim = heads), followed by sym/asym_quant_dynamic over the whole 4096-value row.
//
// The row is the matrix X[head][d] (32 x 128) and Y = H32 X with H32 = H2 (x) H16: sixteen heads are
// contracted by one mma.m16n8k16 per 8 columns (A = H16 / 4 constant; B = the row's own f16 / bf16
// values through ldmatrix.trans, so products are exact and sums fp32), the two 16-head blocks by one
// butterfly stage between accumulator registers.  No second tensor-core step and no fp32 operand
// splitting is needed.  Two warps share a row (eight 8-column tiles each); everything after the
// transform (scale, one fp16 rounding, sign, row maximum, codes, stores) is the code of the
// full-width kernel in rotate_tc.cu.
#include "rotate.cuh"
#include <cfloat>
#include <type_traits>

namespace sr {

namespace {

constexpr int TC_PAIRS = 8;                     // rows in flight per CTA; two warps share a row
constexpr int TC_WARPS = 2 * TC_PAIRS;
constexpr int TC_PITCH = 272;                   // bytes per head (128 values) of the row image: 256 + 16, ldmatrix rows on distinct banks
constexpr int TC_ROW_BYTES = 32 * TC_PITCH;     // 8704
constexpr int TC_SIGN_WORDS = 64 * 32;          // one xor mask per lane and value pair
constexpr size_t TC_SMEM = (size_t)TC_PAIRS * 2 * TC_ROW_BYTES + TC_SIGN_WORDS * 4 + TC_WARPS * 8 + 16;

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t w) { return *reinterpret_cast<__half2 *>(&w); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ float had_sign(int r, int c) { return (__popc(r & c) & 1) ? -1.f : 1.f; }

__device__ __forceinline__ void pair_sync(int pair) {
    asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
}

// InT = __half or __nv_bfloat16 (bf16 rows are multiplied as bf16: exact for every value that is also an fp16 value).
template <typename InT, bool ASYM>
__global__ void __launch_bounds__(TC_WARPS * 32, 1)
rotate_quant_heads32_tc_kernel(const InT *__restrict__ x, const int8_t *__restrict__ sign, uint32_t rows, float scale4,
                               float clip, uint8_t *__restrict__ q, __half *__restrict__ q_scale,
                               __half *__restrict__ q_zero, __half *__restrict__ rotated) {
    constexpr bool BF16 = std::is_same<InT, __nv_bfloat16>::value;
    constexpr int N = 4096;
    extern __shared__ __align__(16) uint8_t tc_smem[];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pair = warp >> 1, half = warp & 1;
    pdl_trigger();   // launched with programmatic serialization (launch_pdl): the sign table is a weight
    const int g = lane >> 2, qd = lane & 3;
    uint32_t *sgn_all = reinterpret_cast<uint32_t *>(tc_smem + (size_t)TC_PAIRS * 2 * TC_ROW_BYTES);
    float2 *exch = reinterpret_cast<float2 *>(sgn_all + TC_SIGN_WORDS);   // [warp]: (max, min) of its half row
    const uint32_t buf_u32 = (uint32_t)__cvta_generic_to_shared(tc_smem) + (uint32_t)pair * 2 * TC_ROW_BYTES;

    const uint32_t base_cnt = rows / gridDim.x, rem = rows % gridDim.x;
    const uint32_t row_begin = blockIdx.x * base_cnt + min(blockIdx.x, rem);
    const uint32_t row_end = row_begin + base_cnt + (blockIdx.x < rem ? 1u : 0u);

    // sign masks in the final register layout: warp `hf`, pair p = (hb * 2 + s) * 8 + j of lane (g, qd) holds
    // elements 128 * head + d and + 1 with head = 16 * hb + 8 * s + g, d = 8 * (8 * hf + j) + 2 * qd
    for (int i = tid; i < TC_SIGN_WORDS; i += TC_WARPS * 32) {
        const int pp = i >> 5, ln = i & 31, hf = pp >> 5, p = pp & 31;
        const int head = 16 * (p >> 4) + 8 * ((p >> 3) & 1) + (ln >> 2), d = 8 * (8 * hf + (p & 7)) + 2 * (ln & 3);
        uint32_t m = 0;
        if (sign != nullptr) {
            if (sign[128 * head + d] < 0) m |= 0x00008000u;
            if (sign[128 * head + d + 1] < 0) m |= 0x80000000u;
        }
        sgn_all[i] = m;
    }
    const uint32_t *sgn = sgn_all + (half * 32) * 32 + lane;
    // A operand: H16 / 4, rows g and g + 8, columns 2 * qd (+1) and + 8
    uint32_t a1[4];
    {
        const uint32_t pos = BF16 ? 0x3E80u : 0x3400u, neg = pos | 0x8000u;   // 0.25
        auto entry = [&](int r, int c) { return had_sign(r, c) > 0 ? pos : neg; };
        a1[0] = entry(g, 2 * qd) | (entry(g, 2 * qd + 1) << 16);
        a1[1] = entry(g + 8, 2 * qd) | (entry(g + 8, 2 * qd + 1) << 16);
        a1[2] = entry(g, 2 * qd + 8) | (entry(g, 2 * qd + 9) << 16);
        a1[3] = entry(g + 8, 2 * qd + 8) | (entry(g + 8, 2 * qd + 9) << 16);
    }
    const u64 scale2 = pack2(scale4, scale4);   // 4 * scale: the constant operand carries the 1/4
    __syncthreads();

    // each warp copies half of the row image: chunk id = 16-byte piece of the row, head id / 16
    auto fetch = [&](uint32_t row, int which) {
        const uint8_t *src = reinterpret_cast<const uint8_t *>(x + (size_t)row * N) + half * 4096 + lane * 16;
        const uint32_t dst = buf_u32 + (uint32_t)which * TC_ROW_BYTES;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int id = (half * 8 + it) * 32 + lane;
            cp_async16(dst + (uint32_t)((id >> 4) * TC_PITCH + (id & 15) * 16), src + it * 512);
        }
    };

    pdl_wait();      // x comes from the kernel before this one
    uint32_t row = row_begin + pair;
    int which = 0;
    if (row < row_end) fetch(row, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");

    while (row < row_end) {
        const uint32_t nrow = row + TC_PAIRS;
        if (nrow < row_end) fetch(nrow, which ^ 1);   // that buffer was last read before the previous row's second barrier
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        pair_sync(pair);

        const uint32_t img = buf_u32 + (uint32_t)which * TC_ROW_BYTES;
        // ldmatrix lane address: matrix m = lane >> 3: head 16 * (m >> 1) + 8 * (m & 1) + (lane & 7); 16-byte column dt
        const uint32_t ld_base = img + (uint32_t)((16 * (lane >> 4) + 8 * ((lane >> 3) & 1) + (lane & 7)) * TC_PITCH);

        __half2 hv[32];
        __half2 hmaxv = __floats2half2_rn(ASYM ? -65504.f : 0.f, ASYM ? -65504.f : 0.f);
        __half2 hminv = __floats2half2_rn(65504.f, 65504.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int dt = 8 * half + j;
            uint32_t r0, r1, r2, r3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                         : "r"(ld_base + (uint32_t)(dt * 16)));
            float c0[4], c1[4];
            mma_16816<BF16>(c0, a1, r0, r1);   // heads 0..15
            mma_16816<BF16>(c1, a1, r2, r3);   // heads 16..31
            // the last stage of H32 between the two head blocks; scale, one rounding to fp16, sign, range
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                const u64 p0 = pack2(c0[2 * s], c0[2 * s + 1]), p1 = pack2(c1[2 * s], c1[2 * s + 1]);
                const u64 y[2] = {mul2(add2(p0, p1), scale2), mul2(sub2(p0, p1), scale2)};
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
                    float lo, hi;
                    unpack2(y[hb], lo, hi);
                    const int p = (hb * 2 + s) * 8 + j;
                    const __half2 h = bits_h2(h2_bits(__floats2half2_rn(lo, hi)) ^ sgn[p * 32]);
                    hv[p] = h;
                    if (ASYM) {
                        hmaxv = __hmax2(hmaxv, h);
                        hminv = __hmin2(hminv, h);
                    } else {
                        hmaxv = __hmax2(hmaxv, __habs2(h));
                    }
                }
            }
        }
        float vmax = warp_max(fmaxf(__low2float(hmaxv), __high2float(hmaxv)));
        float vmin = ASYM ? warp_min(fminf(__low2float(hminv), __high2float(hminv))) : 0.f;
        if (lane == 0) exch[warp] = make_float2(vmax, vmin);
        pair_sync(pair);
        {
            const float2 other = exch[warp ^ 1];
            vmax = fmaxf(vmax, other.x);
            vmin = fminf(vmin, other.y);
        }

        float rcp;
        uint32_t zero_u = 0;
        bool clamp = true;
        __half2 lo_c, hi_c, mg;
        if (!ASYM) {
            __half s = __float2half(vmax / 7.f);
            if (clip != 1.f) s = __float2half(__half2float(s) * clip);
            if (lane == 0 && half == 0) q_scale[row] = s;
            rcp = rcp_approx_ftz(__half2float(s));
            lo_c = __floats2half2_rn(-8.f, -8.f);
            hi_c = __floats2half2_rn(7.f, 7.f);
            mg = __floats2half2_rn(1544.f, 1544.f);
            // scale = rn_h(amax / 7) of a normal fp16 amax keeps every |quotient| below 7.5: nothing to clamp
            clamp = clip != 1.f || __half2float(s) < 6.2e-5f;
        } else {
            __half hmin = __float2half(vmin), hmax = __float2half(vmax);
            if (clip != 1.f) {
                hmin = __float2half(__half2float(hmin) * clip);
                hmax = __float2half(__half2float(hmax) * clip);
            }
            const __half diff = __float2half(__half2float(hmax) - __half2float(hmin));
            const __half s = __float2half(__half2float(diff) / 15.f);
            const __half ratio = __float2half(-__half2float(hmin) / __half2float(s));
            const __half zero = __float2half(nearbyintf(__half2float(ratio)));
            if (lane == 0 && half == 0) {
                q_scale[row] = s;
                q_zero[row] = zero;
            }
            // clamp(rint(v) + z, 0, 15) = rint(clamp(v, -z, 15 - z)) + z for an integer z; the code's low
            // nibble is all that is kept, so z enters modulo 16
            const float zf = __half2float(zero);
            const int zi = __half2int_rn(zero);
            lo_c = __floats2half2_rn(-zf, -zf);
            hi_c = __floats2half2_rn(15.f - zf, 15.f - zf);
            mg = __floats2half2_rn(1536.f, 1536.f);
            zero_u = (uint32_t)(zi & 15) * 0x00010001u;   // added after the rounding: ties go to the even QUOTIENT
            rcp = rcp_approx_ftz(__half2float(s));
        }
        // a zero scale gives rcp = inf and 0 * inf = NaN, which the reference turns into code 0;
        // a huge finite factor gives the same codes (x != 0 still saturates) without the NaN
        rcp = fminf(rcp, 3.0e38f);
        const u64 rcp2 = pack2(rcp, rcp);

        if (rotated != nullptr) {
            __half2 *orow = reinterpret_cast<__half2 *>(rotated + (size_t)row * N);
#pragma unroll
            for (int p = 0; p < 32; ++p) {
                const int hd = 16 * (p >> 4) + 8 * ((p >> 3) & 1) + g, d = 8 * (8 * half + (p & 7)) + 2 * qd;
                orow[(128 * hd + d) >> 1] = hv[p];
            }
        }

        // ---- codes.  After the fp16 addition of the rounding constant the low nibble of each half is the code
        // (offset by 8 for signed codes); four pairs are merged into one word by shifts and byte permutes.
        uint2 *qrow = reinterpret_cast<uint2 *>(q + (size_t)row * (N / 2));
        auto emit = [&](auto clamp_tag) {
            constexpr bool CLAMP = decltype(clamp_tag)::value;
#pragma unroll
            for (int hs = 0; hs < 4; ++hs) {   // hs = hb * 2 + s: head 8 * hs + g; this warp's 32 bytes of its 64-byte row
                uint32_t w[2];
#pragma unroll
                for (int part = 0; part < 2; ++part) {
                    uint32_t bits[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __half22float2(hv[hs * 8 + part * 4 + i]);
                        float lo, hi;
                        unpack2(mul2(pack2(f.x, f.y), rcp2), lo, hi);
                        __half2 qh = __floats2half2_rn(lo, hi);   // rn_h(x * rcp): the quotient __hdiv returns
                        if (CLAMP) qh = __hmin2(__hmax2(qh, lo_c), hi_c);
                        bits[i] = h2_bits(__hadd2(qh, mg));
                        if (ASYM) bits[i] += zero_u;
                    }
                    // the sum lies in [1536, 1552): the low BYTE of each half is the code (+ zero point), the
                    // rest is constant.  Gather the bytes: x = [l0, l1, h0, h1] of two pairs, then evens and odds.
                    const uint32_t x01 = __byte_perm(bits[0], bits[1], 0x6240), x23 = __byte_perm(bits[2], bits[3], 0x6240);
                    uint32_t ev = __byte_perm(x01, x23, 0x5410), od = __byte_perm(x01, x23, 0x7632);
                    if (ASYM) {
                        ev &= 0x0F0F0F0Fu;
                        od &= 0x0F0F0F0Fu;
                    }
                    w[part] = ev + (od << 4);
                }
                if (!ASYM) {
                    w[0] ^= 0x88888888u;
                    w[1] ^= 0x88888888u;
                }
                // lane qd holds bytes 4 * j + qd (j = 0..7) of the 32-byte run; gather bytes 8 qd .. 8 qd + 7
                // exchange 1 (partner qd ^ 2): lanes 0,1 collect the words of nt 0..3, lanes 2,3 those of nt 4..7
                const bool upper = (qd & 2) != 0;
                const uint32_t got = __shfl_xor_sync(0xffffffffu, upper ? w[0] : w[1], 2);
                const uint32_t wa = upper ? got : w[0];    // from lane (qd & 1)
                const uint32_t wb = upper ? w[1] : got;    // from lane (qd & 1) + 2
                // exchange 2 (partner qd ^ 1): even lanes need bytes 0,1 of all four source lanes, odd lanes bytes 2,3
                const bool odd = (qd & 1) != 0;
                const uint32_t keep = odd ? __byte_perm(wa, wb, 0x7632) : __byte_perm(wa, wb, 0x5410);
                const uint32_t give = odd ? __byte_perm(wa, wb, 0x5410) : __byte_perm(wa, wb, 0x7632);
                const uint32_t recv = __shfl_xor_sync(0xffffffffu, give, 1);
                // source lanes in order 0,1,2,3: even lane: keep = lanes (0,2), recv = lanes (1,3); odd lane: the reverse
                const uint32_t s02 = odd ? recv : keep, s13 = odd ? keep : recv;
                uint2 o;
                o.x = __byte_perm(s02, s13, 0x6240);   // first byte of lanes 0,1,2,3
                o.y = __byte_perm(s02, s13, 0x7351);   // second byte
                qrow[(8 * hs + g) * 8 + 4 * half + qd] = o;
            }
        };
        if (clamp) emit(std::true_type{});
        else emit(std::false_type{});

        row = nrow;
        which ^= 1;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
}

}  // namespace

int launch_rotate_heads32(const RotateArgs &a, cudaStream_t st) {
    const bool shape_ok = a.n == 4096 && a.K == 1 && a.S == 32 && a.stride == 128 && a.q != nullptr && !a.fp32_mode &&
                          (a.in_dtype == SR_F16 || (a.in_dtype == SR_BF16 && a.cast_in_to_f16)) &&
                          a.expert_ids == nullptr && aligned16(a.x) && aligned16(a.q) &&
                          (a.out == nullptr || (a.out_dtype == SR_F16 && aligned4(a.out)));
    if (!shape_ok) return SR_ERR_UNSUPPORTED;
    const int sm_count = current_sm_count();
    const uint32_t want = cdiv<uint32_t>(a.rows, TC_PAIRS);
    const uint32_t grid = want < (uint32_t)sm_count ? want : (uint32_t)sm_count;
    const float scale4 = a.scale * 4.f;
#define SR_RQ(T, ASYM)                                                                                          \
    do {                                                                                                        \
        auto kfn = rotate_quant_heads32_tc_kernel<T, ASYM>;                                                     \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);   \
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "rotate_quant: %s", cudaGetErrorString(e));              \
        launch_pdl(kfn, dim3(grid), dim3(TC_WARPS * 32), (size_t)TC_SMEM, st, (const T *)a.x, a.sign, a.rows, scale4, \
                   a.clip, a.q, a.q_scale, a.q_zero, (__half *)a.out);                                         \
    } while (0)
    if (a.in_dtype == SR_F16) {
        if (a.asym) SR_RQ(__half, true);
        else SR_RQ(__half, false);
    } else {
        if (a.asym) SR_RQ(__nv_bfloat16, true);
        else SR_RQ(__nv_bfloat16, false);
    }
#undef SR_RQ
    return check_launch("rotate_quant_heads32_tc");
}

}  // namespace sr
