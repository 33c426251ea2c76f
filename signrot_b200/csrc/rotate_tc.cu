// Fused online rotation + sign + per-token int4 quantization for rows of 4096 values, with the
// Walsh-Hadamard transform on the tensor cores.
//
// One launch replaces fast_hadamard_transform + sign multiply + sym/asym_quant_dynamic
// (signrot/functional/hadamard.py:81, signrot/nn/hadamard.py:39, signrot/kernels/fused.cu:68-112)
// and touches HBM once: 2 bytes in and 0.5 bytes out per value.
//
// A row is the 64 x 64 matrix X[h][l] (element 64*h + l) and H4096 = H64 (x) H64 is separable:
//   Y = H64 * X * H64 / 64.
// One warp owns a row.  The butterfly form of the transform costs about two issue slots per
// value and stage on the floating-point pipes; here nine of the twelve stages run as matrix
// products against constant +-1/8 fragments instead:
//   step 1  U = H64 * X.  Bits 0..3 of h: mma.m16n8k16 (f16 or bf16 operands are the row's own
//           values, so the products are exact and the sums are fp32), A = H16 / 8, B = 16 x 8
//           blocks of X read with ldmatrix.trans from the row's shared-memory image.  Bits 4..5
//           of h: two butterfly stages between accumulator registers (packed fp32 adds).
//   step 2  Y = U * H64.  Bits 0..2 of l sit across the lanes of the accumulator layout; they are
//           contracted by mma.m16n8k8 (tf32) with B = H8 / 8.  U is fp32, so it enters as the
//           sum of a 11-bit head and the remainder's 11-bit head (two MMAs): the error is about
//           2^-21 relative, the size of the fp32 rounding noise of the butterfly form.
//           Bits 3..5 of l: three butterfly stages between registers.
// The values are then rounded once to fp16 (the dtype the reference's transform returns); sign,
// row maximum and the code decision run on packed fp16 pairs, bit-compatible with the reference's
// quantizer: scale rn_h(amax / 7), quotient rn_h(x * rcp(scale)), round half to even, clamp.
//
// Rows arrive through cp.async into a per-warp double buffer (the next row is in flight while
// this one is transformed); row pitch 144 bytes keeps ldmatrix bank-conflict free.  Codes leave
// as 8-byte stores, 256 contiguous bytes per warp instruction.
#include "rotate.cuh"
#include <cfloat>
#include <type_traits>

namespace sr {

namespace {

constexpr int TC_PAIRS = 8;                     // rows in flight per CTA; two warps share a row
constexpr int TC_WARPS = 2 * TC_PAIRS;
constexpr int TC_PITCH = 144;                   // bytes per 64-value line of the row image
constexpr int TC_ROW_BYTES = 64 * TC_PITCH;     // 9216
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

// d = a * b (+ d when ACC)
template <bool ACC>
__device__ __forceinline__ void mma_1688_tf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    if (ACC)
        asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ float had_sign(int r, int c) { return (__popc(r & c) & 1) ? -1.f : 1.f; }

__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
    u64 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

__device__ __forceinline__ void pair_sync(int pair) {
    asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
}

// InT = __half or __nv_bfloat16.  bf16 rows are multiplied as bf16: every bf16 value of magnitude
// 2^-17 .. 65504 (and zero) is also an fp16 value, so the reference's x.to(float16) changes nothing
// there; smaller magnitudes differ from it by less than 2^-25 in absolute terms.
//
// Two warps share a row: both run step 1 over the whole row image (the tensor pipe has room), warp
// `half` keeps the lines h = 32 * half .. 32 * half + 31 of U and finishes them, so a lane holds 64
// results instead of 128 and fourteen warps fit on an SM.
template <typename InT, bool ASYM>
__global__ void __launch_bounds__(TC_WARPS * 32, 1)
rotate_quant_4096_tc_kernel(const InT *__restrict__ x, const int8_t *__restrict__ sign, uint32_t rows, float clip,
                            uint8_t *__restrict__ q, __half *__restrict__ q_scale, __half *__restrict__ q_zero,
                            __half *__restrict__ rotated) {
    constexpr bool BF16 = std::is_same<InT, __nv_bfloat16>::value;
    constexpr int N = 4096;
    extern __shared__ __align__(16) uint8_t tc_smem[];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_trigger();   // launched with programmatic serialization (launch_pdl): the sign table is a weight
    const int pair = warp >> 1, half = warp & 1;
    const int g = lane >> 2, qd = lane & 3;
    uint32_t *sgn_all = reinterpret_cast<uint32_t *>(tc_smem + (size_t)TC_PAIRS * 2 * TC_ROW_BYTES);
    float2 *exch = reinterpret_cast<float2 *>(sgn_all + TC_SIGN_WORDS);   // [warp]: (max, min) of its half row
    const uint32_t buf_u32 = (uint32_t)__cvta_generic_to_shared(tc_smem) + (uint32_t)pair * 2 * TC_ROW_BYTES;

    // rows of this CTA: an even split, the first (rows % grid) CTAs take one more
    const uint32_t base_cnt = rows / gridDim.x, rem = rows % gridDim.x;
    const uint32_t row_begin = blockIdx.x * base_cnt + min(blockIdx.x, rem);
    const uint32_t row_end = row_begin + base_cnt + (blockIdx.x < rem ? 1u : 0u);

    // ---- per-CTA constants: sign masks in the final register layout.  Pair p = (hh * 2 + s) * 8 + nt of lane
    // (g, qd) holds elements 64 * h + l and + 1 with h = 16 * hh + 8 * s + g, l = 8 * nt + 2 * qd.
    for (int i = tid; i < TC_SIGN_WORDS; i += TC_WARPS * 32) {
        const int p = i >> 5, ln = i & 31;
        const int h = 16 * (p >> 4) + 8 * ((p >> 3) & 1) + (ln >> 2), l = 8 * (p & 7) + 2 * (ln & 3);
        uint32_t m = 0;
        if (sign != nullptr) {
            if (sign[64 * h + l] < 0) m |= 0x00008000u;
            if (sign[64 * h + l + 1] < 0) m |= 0x80000000u;
        }
        sgn_all[i] = m;
    }
    const uint32_t *sgn = sgn_all + (half * 32) * 32 + lane;   // this warp's 32 pairs: hh = 2 * half + hl
    // A operand of step 1: H16 / 8, rows g and g + 8, columns 2 * qd (+1) and + 8
    uint32_t a1[4];
    {
        const uint32_t pos = BF16 ? 0x3E00u : 0x3000u, neg = pos | 0x8000u;
        auto entry = [&](int r, int c) { return had_sign(r, c) > 0 ? pos : neg; };
        a1[0] = entry(g, 2 * qd) | (entry(g, 2 * qd + 1) << 16);
        a1[1] = entry(g + 8, 2 * qd) | (entry(g + 8, 2 * qd + 1) << 16);
        a1[2] = entry(g, 2 * qd + 8) | (entry(g, 2 * qd + 9) << 16);
        a1[3] = entry(g + 8, 2 * qd + 8) | (entry(g + 8, 2 * qd + 9) << 16);
    }
    // B operand of step 2: H8 / 8; physical k = qd carries logical l = 2 * qd, k = qd + 4 carries 2 * qd + 1
    const uint32_t b2_0 = __float_as_uint(0.125f * had_sign(2 * qd, g));
    const uint32_t b2_1 = __float_as_uint(0.125f * had_sign(2 * qd + 1, g));
    // second butterfly stage over the 16-line blocks: this warp keeps blocks 2 * half and 2 * half + 1
    const float sg2 = half ? -1.f : 1.f;
    const u64 sigma = pack2(sg2, sg2);
    __syncthreads();

    // each warp copies its half of the row image: chunk id = 16-byte piece of the row, line id / 8
    auto fetch = [&](uint32_t row, int which) {
        const uint8_t *src = reinterpret_cast<const uint8_t *>(x + (size_t)row * N) + half * 4096 + lane * 16;
        const uint32_t dst = buf_u32 + (uint32_t)which * TC_ROW_BYTES;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int id = (half * 8 + it) * 32 + lane;
            cp_async16(dst + (uint32_t)((id >> 3) * TC_PITCH + (id & 7) * 16), src + it * 512);
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
        // ldmatrix lane address: matrix (lane >> 3): lines 8 * (m & 1) + (lane & 7), 16-byte column m >> 1
        const uint32_t ld_base = img + (uint32_t)((8 * ((lane >> 3) & 1) + (lane & 7)) * TC_PITCH + (lane >> 4) * 16);

        float c2[2][8][4];   // [hl][nt][slot] after step 2's MMA; slot 0,1: line g, l = 2 qd, 2 qd + 1; slot 2,3: line g + 8
#pragma unroll
        for (int ntp = 0; ntp < 4; ++ntp) {
            uint32_t frag[4][4];
#pragma unroll
            for (int hh = 0; hh < 4; ++hh)
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(frag[hh][0]), "=r"(frag[hh][1]), "=r"(frag[hh][2]), "=r"(frag[hh][3])
                             : "r"(ld_base + (uint32_t)(hh * 16 * TC_PITCH + ntp * 32)));
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int nt = 2 * ntp + e;
                float c1[4][4];
#pragma unroll
                for (int hh = 0; hh < 4; ++hh) mma_16816<BF16>(c1[hh], a1, frag[hh][2 * e], frag[hh][2 * e + 1]);
                // bits 4..5 of h: butterflies over hh on the packed pairs (slot 0,1) and (slot 2,3); of the
                // four results this warp needs two: (p0 +- p1) + sigma * (p2 +- p3)
                u64 u2[2][2];   // [hl][s]
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    const u64 p0 = pack2(c1[0][2 * s], c1[0][2 * s + 1]), p1 = pack2(c1[1][2 * s], c1[1][2 * s + 1]);
                    const u64 p2 = pack2(c1[2][2 * s], c1[2][2 * s + 1]), p3 = pack2(c1[3][2 * s], c1[3][2 * s + 1]);
                    u2[0][s] = fma2(add2(p2, p3), sigma, add2(p0, p1));
                    u2[1][s] = fma2(sub2(p2, p3), sigma, sub2(p0, p1));
                }
                // step 2, bits 0..2 of l: head + remainder as two tf32 operands
#pragma unroll
                for (int hl = 0; hl < 2; ++hl) {
                    float u[4];
                    unpack2(u2[hl][0], u[0], u[1]);
                    unpack2(u2[hl][1], u[2], u[3]);
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) hi[i] = __float_as_uint(u[i]) & 0xFFFFE000u;
                    float r[4];
                    unpack2(sub2(u2[hl][0], pack2(__uint_as_float(hi[0]), __uint_as_float(hi[1]))), r[0], r[1]);
                    unpack2(sub2(u2[hl][1], pack2(__uint_as_float(hi[2]), __uint_as_float(hi[3]))), r[2], r[3]);
                    // the tensor core reads the upper 19 bits of a tf32 operand: the remainder needs no mask
#pragma unroll
                    for (int i = 0; i < 4; ++i) lo[i] = __float_as_uint(r[i]);
                    // A slots: a0 = (line g, k qd) = l 2 qd; a1 = (line g + 8, k qd); a2 = (line g, k qd + 4) = l 2 qd + 1; a3
                    mma_1688_tf32<false>(c2[hl][nt], hi[0], hi[2], hi[1], hi[3], b2_0, b2_1);
                    mma_1688_tf32<true>(c2[hl][nt], lo[0], lo[2], lo[1], lo[3], b2_0, b2_1);
                }
            }
        }

        // ---- bits 3..5 of l: butterflies over nt; then one rounding to fp16, sign, range
        __half2 hv[32];
        __half2 hmaxv = __floats2half2_rn(ASYM ? -65504.f : 0.f, ASYM ? -65504.f : 0.f);
        __half2 hminv = __floats2half2_rn(65504.f, 65504.f);
#pragma unroll
        for (int hl = 0; hl < 2; ++hl) {
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                u64 v[8];
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) v[nt] = pack2(c2[hl][nt][2 * s], c2[hl][nt][2 * s + 1]);
#pragma unroll
                for (int dist = 1; dist < 8; dist <<= 1) {
#pragma unroll
                    for (int nt = 0; nt < 8; ++nt) {
                        if ((nt & dist) == 0) {
                            const u64 a = v[nt], b = v[nt + dist];
                            v[nt] = add2(a, b);
                            v[nt + dist] = sub2(a, b);
                        }
                    }
                }
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    float lo, hi;
                    unpack2(v[nt], lo, hi);
                    const int p = (hl * 2 + s) * 8 + nt;
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
                const int h = 32 * half + 16 * (p >> 4) + 8 * ((p >> 3) & 1) + g, l = 8 * (p & 7) + 2 * qd;
                orow[(64 * h + l) >> 1] = hv[p];
            }
        }

        // ---- codes.  After the fp16 addition of the rounding constant the low nibble of each half is the code
        // (offset by 8 for signed codes); four pairs are merged into one word by shifts and byte permutes.
        uint2 *qrow = reinterpret_cast<uint2 *>(q + (size_t)row * (N / 2));
        auto emit = [&](auto clamp_tag) {
            constexpr bool CLAMP = decltype(clamp_tag)::value;
#pragma unroll
            for (int hs = 0; hs < 4; ++hs) {   // hs = hl * 2 + s: line h = 32 * half + 8 * hs + g of the row
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
                // lane qd holds bytes 4 * nt + qd (nt = 0..7) of the 32-byte line; gather bytes 8 qd .. 8 qd + 7
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
                qrow[(32 * half + 8 * hs + g) * 4 + qd] = o;
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

int launch_rotate_tc4096(const RotateArgs &a, cudaStream_t st) {
    const bool shape_ok = a.n == 4096 && a.K == 1 && a.stride == 1 && a.S == 4096 && a.q != nullptr && !a.fp32_mode &&
                          (a.in_dtype == SR_F16 || (a.in_dtype == SR_BF16 && a.cast_in_to_f16)) &&
                          a.expert_ids == nullptr && a.scale == 1.f / 64.f && aligned16(a.x) && aligned16(a.q) &&
                          (a.out == nullptr || (a.out_dtype == SR_F16 && aligned4(a.out)));
    if (!shape_ok) return SR_ERR_UNSUPPORTED;
    const int sm_count = current_sm_count();
    const uint32_t want = cdiv<uint32_t>(a.rows, TC_PAIRS);
    const uint32_t grid = want < (uint32_t)sm_count ? want : (uint32_t)sm_count;
#define SR_RQ(T, ASYM)                                                                                          \
    do {                                                                                                        \
        auto kfn = rotate_quant_4096_tc_kernel<T, ASYM>;                                                        \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);   \
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "rotate_quant: %s", cudaGetErrorString(e));              \
        launch_pdl(kfn, dim3(grid), dim3(TC_WARPS * 32), (size_t)TC_SMEM, st, (const T *)a.x, a.sign, a.rows, a.clip, \
                   a.q, a.q_scale, a.q_zero, (__half *)a.out);                                                 \
    } while (0)
    if (a.in_dtype == SR_F16) {
        if (a.asym) SR_RQ(__half, true);
        else SR_RQ(__half, false);
    } else {
        if (a.asym) SR_RQ(__nv_bfloat16, true);
        else SR_RQ(__nv_bfloat16, false);
    }
#undef SR_RQ
    return check_launch("rotate_quant_4096_tc");
}

}  // namespace sr
