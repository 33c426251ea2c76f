// Fused online rotation + sign + symmetric per-token int4 quantization for rows of
// 14336 = 28 x 512 values (the down_proj input of an 8B model): y = (had28 (x) H_512) x / sqrt(n).
//
// Replaces, in one launch and one pass over HBM, fast_hadamard_transform over the 28 segments,
// the fp16 had28 matmul, the sign multiply and sym_quant_dynamic
// (signrot/functional/hadamard.py:78-87, signrot/nn/hadamard.py:39, signrot/kernels/fused.cu:68-112).
// The rounding points are the reference's: the 512-point sums are fp32, scaled and rounded to
// fp16; the 28-point stage multiplies fp16 values by +-1 and accumulates in fp32 (exactly what an
// fp16 tensor-core matmul does), rounded to fp16 again.
//
// One CTA of 448 threads (14 warps) per row, persistent over rows:
//   1. the row arrives by cp.async as 28 segment images of 16 lines x 32 values (the copy of the
//      next row is issued as soon as this stage is done with the buffer and overlaps stages 3-4).
//      Warp w transforms segments 2w and 2w + 1 on the tensor cores: with a segment as the matrix
//      X[h][l] (element 32 h + l), U = H16 X is one mma.m16n8k16 per 8 columns (f16 or bf16 operands
//      are the row's own values: exact products, fp32 sums; B fragments by ldmatrix.trans), bits
//      0..2 of l sit across the lanes of the accumulators and are contracted by mma.m16n8k8 (tf32,
//      the fp32 accumulator enters as an 11-bit head plus its remainder), bits 3..4 of l are two
//      butterfly stages between registers (packed fp32 adds);
//   2. the scaled fp16 values go to shared memory as Z[k][j] (columns skewed by 8 every 32 so that
//      the 4-byte stores and the later 8x8 matrix loads are bank-conflict free);
//   3. Y[32 x 512] = H28 (zero padded to 32 x 32) * Z on mma.sync.m16n8k16 (fp16 in, fp32
//      accumulate): 64 column tiles spread over the 14 warps, the A fragments of H28 and the sign
//      bits of a thread's outputs stay in registers for the whole (persistent) kernel;
//   4. fp16 rounding, sign, row maximum, codes; bytes are staged in shared memory and leave as
//      one 16-byte store per thread.
#include "rotate.cuh"
#include <cfloat>
#include <type_traits>

namespace sr {

namespace {

constexpr int N = 14336, SEG = 512, KH = 28;
constexpr int THREADS = 448;
constexpr int LINE = 80;       // bytes per 32-value line of a segment image (64 + 16: ldmatrix rows hit distinct banks)
constexpr int IMG_SEG = 16 * LINE;             // 1280 bytes per segment
constexpr int IMG_BYTES = KH * IMG_SEG;        // 35840
constexpr int PZ = 648;        // halves per row of Z: 512 + 8 per 32 (skew) + 8; PZ * 2 / 16 is odd
constexpr int Z_BYTES = 32 * PZ * 2;           // 41472
constexpr int OUTP = 272;      // bytes per output row in the staging buffer (256 + 16)
constexpr int SMEM_BYTES = IMG_BYTES + Z_BYTES + KH * OUTP;

__device__ __forceinline__ int zcol(int j) { return j + 8 * (j >> 5); }

__device__ __forceinline__ float had_pm(int r, int c) { return (__popc(r & c) & 1) ? -1.f : 1.f; }

// LATE: the sign is applied to the packed codes instead of the values.  For a symmetric quantizer
// code(-v) = -code(v) as long as nothing saturates, which holds for clip = 1 and a normal fp16 scale
// (|v / scale| < 7.5); such launches (no per-row sign table, no rotated output) skip the per-value
// sign work, and a row whose scale is subnormal falls back to the value path.
// ASYM (never together with LATE): unsigned codes with a per-row zero point (asym_quant_dynamic).
template <typename InT, bool LATE, bool ASYM>
__global__ void __launch_bounds__(THREADS, 2)
rotate_quant_had28_kernel(const InT *__restrict__ x, const __half *__restrict__ hadk,
                          const int8_t *__restrict__ sign, const int32_t *__restrict__ expert_ids, uint32_t rows,
                          float scale, float clip, uint8_t *__restrict__ q, __half *__restrict__ q_scale,
                          __half *__restrict__ q_zero, __half *__restrict__ rotated) {
    static_assert(!(LATE && ASYM), "the sign can only move onto symmetric codes");
    constexpr bool BF16 = std::is_same<InT, __nv_bfloat16>::value;
    extern __shared__ __align__(16) uint8_t smem[];
    __half *zbuf = reinterpret_cast<__half *>(smem + IMG_BYTES);
    uint8_t *obuf = smem + IMG_BYTES + Z_BYTES;
    const uint32_t img_u32 = (uint32_t)__cvta_generic_to_shared(smem);
    __shared__ float red[2][14];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, qd = lane & 3;  // mma fragment coordinates
    pdl_trigger();   // launched with programmatic serialization (launch_pdl): the tables below are weights

    // ---- A fragments of H (28 x 28 padded with zeros to 32 x 32), row-major fp16
    uint32_t afr[2][2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int kt = 0; kt < 2; ++kt)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int row = 16 * mt + g + 8 * (r & 1);
                const int col = 16 * kt + 2 * qd + 8 * (r >> 1);
                __half2 h2 = __floats2half2_rn(0.f, 0.f);
                if (row < KH && col < KH) h2.x = hadk[row * KH + col];
                if (row < KH && col + 1 < KH) h2.y = hadk[row * KH + col + 1];
                afr[mt][kt][r] = *reinterpret_cast<uint32_t *>(&h2);
            }
    const int n_tiles = (warp + 56 < 64) ? 5 : 4;  // column tiles warp, warp+14, ...

    // sign bits of this thread's outputs: bit (tile*8 + mt*4 + r) <-> y[16mt + g + 8(r>>1)][8nt + 2qd + (r&1)]
    const bool per_row_sign = sign != nullptr && expert_ids != nullptr;
    uint64_t neg_static = 0;
    auto load_sign = [&](const int8_t *sg) {
        uint64_t m = 0;
        for (int ti = 0; ti < n_tiles; ++ti) {
            const int nt = warp + 14 * ti;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int kp = 16 * mt + g + 8 * (r >> 1);
                    const int j = 8 * nt + 2 * qd + (r & 1);
                    if (kp < KH && sg[kp * SEG + j] < 0) m |= 1ull << (ti * 8 + mt * 4 + r);
                }
        }
        return m;
    };
    if (sign != nullptr && !per_row_sign) neg_static = load_sign(sign);
    // sign of the 32 codes this thread stores at the end (row tid / 16, values 32 * (tid % 16) ..): one 0xF per -1
    uint32_t late_mask[4] = {0, 0, 0, 0};
    auto load_late = [&](const int8_t *tab) {
        const int8_t *sg = tab + (tid >> 4) * SEG + (tid & 15) * 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            late_mask[i] = 0;
#pragma unroll
            for (int n = 0; n < 8; ++n)
                if (sg[8 * i + n] < 0) late_mask[i] |= 0xFu << (4 * n);
        }
    };
    if (LATE && sign != nullptr && !per_row_sign) load_late(sign);
    // per-row sign tables (MoE): rows arrive sorted by expert, so the table of the previous row is usually still
    // the right one; it is reloaded only when the expert changes
    int cur_expert = -1;
    uint64_t neg_row = 0;

    // step-1 A operand: H16 / 8 (rows g, g + 8; columns 2 qd (+1), + 8); step-2 B operand: H8 / 8 with
    // physical k = qd carrying logical l = 2 qd and k = qd + 4 carrying 2 qd + 1
    uint32_t a1[4];
    {
        const uint32_t pos = BF16 ? 0x3E00u : 0x3000u, ng = pos | 0x8000u;
        auto entry = [&](int r, int c) { return had_pm(r, c) > 0 ? pos : ng; };
        a1[0] = entry(g, 2 * qd) | (entry(g, 2 * qd + 1) << 16);
        a1[1] = entry(g + 8, 2 * qd) | (entry(g + 8, 2 * qd + 1) << 16);
        a1[2] = entry(g, 2 * qd + 8) | (entry(g, 2 * qd + 9) << 16);
        a1[3] = entry(g + 8, 2 * qd + 8) | (entry(g + 8, 2 * qd + 9) << 16);
    }
    const uint32_t b2_0 = __float_as_uint(0.125f * had_pm(2 * qd, g));
    const uint32_t b2_1 = __float_as_uint(0.125f * had_pm(2 * qd + 1, g));
    const float scale64 = scale * 64.f;   // the two constant operands carry 1/8 each
    const u64 scale2 = pack2(scale64, scale64);

    // 1792 16-byte chunks per row, 4 per thread: chunk id -> segment id / 64, line (id / 4) % 16, piece id % 4
    auto fetch = [&](uint32_t row) {
        const uint8_t *src = reinterpret_cast<const uint8_t *>(x + (size_t)row * N);
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int id = it * THREADS + tid;
            const uint32_t dst = img_u32 + (uint32_t)((id >> 6) * IMG_SEG + ((id >> 2) & 15) * LINE + (id & 3) * 16);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + (size_t)id * 16) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // rows 28..31 of Z are the zero padding of the k dimension (written once: nothing else touches them)
    if (tid < 4 * PZ / 8) reinterpret_cast<uint4 *>(zbuf + KH * PZ)[tid] = make_uint4(0, 0, 0, 0);
    pdl_wait();      // x and expert_ids come from the kernels before this one
    if (blockIdx.x < rows) fetch(blockIdx.x);

    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();   // the row image is complete; Z and the staging bytes of the previous row are dead

        // ---- 1 + 2. 512-point transforms of segments 2 * warp and 2 * warp + 1, Z[k][j] = rn_h(sum * scale)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int seg = 2 * warp + e;
            // ldmatrix lane address: matrix m = lane >> 3: lines 8 * (m & 1) + (lane & 7), 16-byte piece m >> 1
            const uint32_t ld = img_u32 + (uint32_t)(seg * IMG_SEG + (8 * ((lane >> 3) & 1) + (lane & 7)) * LINE +
                                                     (lane >> 4) * 16);
            uint32_t fr[2][4];
#pragma unroll
            for (int pp = 0; pp < 2; ++pp)
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(fr[pp][0]), "=r"(fr[pp][1]), "=r"(fr[pp][2]), "=r"(fr[pp][3])
                             : "r"(ld + (uint32_t)(pp * 32)));
            float c2[4][4];   // [nt][slot]: slot 0,1 = line g, l 2 qd (+1); slot 2,3 = line g + 8
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                float c1[4];
                const uint32_t f0 = fr[nt >> 1][2 * (nt & 1)], f1 = fr[nt >> 1][2 * (nt & 1) + 1];
                if (BF16)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                                 : "=f"(c1[0]), "=f"(c1[1]), "=f"(c1[2]), "=f"(c1[3])
                                 : "r"(a1[0]), "r"(a1[1]), "r"(a1[2]), "r"(a1[3]), "r"(f0), "r"(f1), "f"(0.f));
                else
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                                 : "=f"(c1[0]), "=f"(c1[1]), "=f"(c1[2]), "=f"(c1[3])
                                 : "r"(a1[0]), "r"(a1[1]), "r"(a1[2]), "r"(a1[3]), "r"(f0), "r"(f1), "f"(0.f));
                // bits 0..2 of l on tf32 MMAs: the fp32 value enters as an 11-bit head plus its remainder (of
                // which the tensor core reads the upper 11 bits): about 2^-22 relative, the size of the
                // rounding noise of fp32 sums
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) hi[i] = __float_as_uint(c1[i]) & 0xFFFFE000u;
                float r[4];
                unpack2(sub2(pack2(c1[0], c1[1]), pack2(__uint_as_float(hi[0]), __uint_as_float(hi[1]))), r[0], r[1]);
                unpack2(sub2(pack2(c1[2], c1[3]), pack2(__uint_as_float(hi[2]), __uint_as_float(hi[3]))), r[2], r[3]);
#pragma unroll
                for (int i = 0; i < 4; ++i) lo[i] = __float_as_uint(r[i]);
                asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                             : "=f"(c2[nt][0]), "=f"(c2[nt][1]), "=f"(c2[nt][2]), "=f"(c2[nt][3])
                             : "r"(lo[0]), "r"(lo[2]), "r"(lo[1]), "r"(lo[3]), "r"(b2_0), "r"(b2_1), "f"(0.f));
                asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(c2[nt][0]), "+f"(c2[nt][1]), "+f"(c2[nt][2]), "+f"(c2[nt][3])
                             : "r"(hi[0]), "r"(hi[2]), "r"(hi[1]), "r"(hi[3]), "r"(b2_0), "r"(b2_1));
            }
            // bits 3..4 of l: butterflies over nt; scale, one rounding, Z[seg][32 h + l] as fp16 pairs
            __half *zr = zbuf + seg * PZ;
#pragma unroll
            for (int sl = 0; sl < 2; ++sl) {
                u64 v[4];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) v[nt] = pack2(c2[nt][2 * sl], c2[nt][2 * sl + 1]);
                const u64 q0 = add2(v[0], v[1]), q1 = sub2(v[0], v[1]), q2 = add2(v[2], v[3]), q3 = sub2(v[2], v[3]);
                v[0] = add2(q0, q2);
                v[2] = sub2(q0, q2);
                v[1] = add2(q1, q3);
                v[3] = sub2(q1, q3);
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    float lo_, hi_;
                    unpack2(mul2(v[nt], scale2), lo_, hi_);
                    const int j = 32 * (g + 8 * sl) + 8 * nt + 2 * qd;
                    *reinterpret_cast<__half2 *>(zr + zcol(j)) = __floats2half2_rn(lo_, hi_);
                }
            }
        }
        __syncthreads();   // Z is complete and nobody reads the row image any more
        if (row + gridDim.x < rows) fetch(row + gridDim.x);

        // ---- 3. Y = H * Z on the tensor cores, fp16 rounding, (sign), row maximum
        if (per_row_sign) {
            const int e = expert_ids[row];
            if (e != cur_expert) {
                cur_expert = e;
                if (LATE) load_late(sign + (size_t)e * N);
                else neg_row = load_sign(sign + (size_t)e * N);
            }
        }
        uint64_t neg = per_row_sign ? neg_row : neg_static;
        __half2 y[5][2][2];  // [tile][mt][half: rows g / g+8] = columns (2qd, 2qd+1)
        auto flip = [&](int ti, int mt) {   // sign of the four values of slot pair (ti, mt), from the bit mask
            const uint32_t sb = (uint32_t)(neg >> (ti * 8 + mt * 4)) & 15u;
            uint32_t lw = *reinterpret_cast<uint32_t *>(&y[ti][mt][0]), hw_ = *reinterpret_cast<uint32_t *>(&y[ti][mt][1]);
            lw ^= ((sb & 1u) << 15) | ((sb & 2u) << 30);
            hw_ ^= ((sb & 4u) << 13) | ((sb & 8u) << 28);
            y[ti][mt][0] = *reinterpret_cast<__half2 *>(&lw);
            y[ti][mt][1] = *reinterpret_cast<__half2 *>(&hw_);
        };
        __half2 amax2 = __floats2half2_rn(ASYM ? -65504.f : 0.f, ASYM ? -65504.f : 0.f);
        __half2 amin2 = __floats2half2_rn(65504.f, 65504.f);
#pragma unroll
        for (int ti = 0; ti < 5; ++ti) {
            if (ti < n_tiles) {
                const int nt = warp + 14 * ti;
                uint32_t b0, b1, b2, b3;
                {
                    const int t = lane >> 3, r = lane & 7;
                    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(zbuf + (8 * t + r) * PZ + zcol(8 * nt));
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                                 : "r"(addr));
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    float c0, c1, c2, c3;
                    asm volatile(
                        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                        : "=f"(c0), "=f"(c1), "=f"(c2), "=f"(c3)
                        : "r"(afr[mt][0][0]), "r"(afr[mt][0][1]), "r"(afr[mt][0][2]), "r"(afr[mt][0][3]), "r"(b0), "r"(b1),
                          "f"(0.f));
                    asm volatile(
                        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                        : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
                        : "r"(afr[mt][1][0]), "r"(afr[mt][1][1]), "r"(afr[mt][1][2]), "r"(afr[mt][1][3]), "r"(b2), "r"(b3));
                    y[ti][mt][0] = __floats2half2_rn(c0, c1);
                    y[ti][mt][1] = __floats2half2_rn(c2, c3);
                    if (!LATE) flip(ti, mt);
                    if (ASYM) {
                        // rows 28..31 are padding: their zeros must not enter the range
                        amax2 = __hmax2(amax2, y[ti][mt][0]);
                        amin2 = __hmin2(amin2, y[ti][mt][0]);
                        if (mt == 0 || g < 4) {
                            amax2 = __hmax2(amax2, y[ti][mt][1]);
                            amin2 = __hmin2(amin2, y[ti][mt][1]);
                        }
                    } else {
                        amax2 = __hmax2(amax2, __hmax2(__habs2(y[ti][mt][0]), __habs2(y[ti][mt][1])));
                    }
                }
            }
        }
        float amax = warp_max(fmaxf(__low2float(amax2), __high2float(amax2)));
        float amin = ASYM ? warp_min(fminf(__low2float(amin2), __high2float(amin2))) : 0.f;
        if (lane == 0) {
            red[0][warp] = amax;
            red[1][warp] = amin;
        }
        __syncthreads();
        amax = red[0][0];
        amin = red[1][0];
#pragma unroll
        for (int w = 1; w < 14; ++w) {
            amax = fmaxf(amax, red[0][w]);
            amin = fminf(amin, red[1][w]);
        }
        __half s;
        __half2 lo_c, hi_c, magic;
        uint32_t zero_u = 0;
        if (!ASYM) {
            s = __float2half(amax / 7.f);
            if (clip != 1.f) s = __float2half(__half2float(s) * clip);
            if (tid == 0) q_scale[row] = s;
            lo_c = __floats2half2_rn(-8.f, -8.f);
            hi_c = __floats2half2_rn(7.f, 7.f);
            magic = __floats2half2_rn(1544.f, 1544.f);   // codes leave as code + 8 until the last step
        } else {
            __half hmin = __float2half(amin), hmax = __float2half(amax);
            if (clip != 1.f) {
                hmin = __float2half(__half2float(hmin) * clip);
                hmax = __float2half(__half2float(hmax) * clip);
            }
            const __half diff = __float2half(__half2float(hmax) - __half2float(hmin));
            s = __float2half(__half2float(diff) / 15.f);
            const __half ratio = __float2half(-__half2float(hmin) / __half2float(s));
            const __half zero = __float2half(nearbyintf(__half2float(ratio)));
            if (tid == 0) {
                q_scale[row] = s;
                q_zero[row] = zero;
            }
            // clamp(rint(v) + z, 0, 15) = rint(clamp(v, -z, 15 - z)) + z for an integer z; z enters modulo 16 after the rounding
            const float zf = __half2float(zero);
            lo_c = __floats2half2_rn(-zf, -zf);
            hi_c = __floats2half2_rn(15.f - zf, 15.f - zf);
            magic = __floats2half2_rn(1536.f, 1536.f);
            zero_u = (uint32_t)(__half2int_rn(zero) & 15) * 0x00010001u;
        }
        // a zero scale would give 0 * inf = NaN (code 0 in the reference): a huge finite factor
        // yields the same codes without the NaN
        const float rcp = fminf(rcp_approx_ftz(__half2float(s)), 3.0e38f);
        const u64 rcp2 = pack2(rcp, rcp);
        // no quotient reaches 7.5 when the scale is a normal fp16 number and nothing was clipped
        const bool safe = LATE && __half2float(s) >= 6.2e-5f;
        if (LATE && !safe) {
            if (per_row_sign) neg = load_sign(sign + (size_t)cur_expert * N);   // rare: subnormal scale
#pragma unroll
            for (int ti = 0; ti < 5; ++ti)
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
                    if (ti < n_tiles) flip(ti, mt);
        }

        // ---- 4. codes -> staging bytes -> one 16-byte store per thread
        uint8_t *ob = obuf + g * OUTP + 4 * warp + qd;
#pragma unroll
        for (int ti = 0; ti < 5; ++ti) {
            if (ti < n_tiles) {
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int kp = 16 * mt + g + 8 * hh;
                        if (mt == 0 || hh == 0 || kp < KH) {
                            const __half2 p = y[ti][mt][hh];
                            // rn_h(x * rcp), (clamp), round to nearest even by the fp16 addition of the constant
                            const float2 f = __half22float2(p);
                            float lo, hi;
                            unpack2(mul2(pack2(f.x, f.y), rcp2), lo, hi);
                            __half2 qh = __floats2half2_rn(lo, hi);
                            if (!safe) qh = __hmin2(__hmax2(qh, lo_c), hi_c);
                            qh = __hadd2(qh, magic);
                            const uint32_t r = (*reinterpret_cast<uint32_t *>(&qh) + zero_u) & 0x000F000Fu;
                            ob[(16 * mt + 8 * hh) * OUTP + 56 * ti] = (uint8_t)(r | (r >> 12));
                            if (!LATE && rotated != nullptr)
                                *reinterpret_cast<__half2 *>(rotated + (size_t)row * N + kp * SEG + 8 * (warp + 14 * ti) + 2 * qd) = p;
                        }
                    }
            }
        }
        __syncthreads();
        {
            const int kp = tid >> 4, part = tid & 15;  // 448 threads x 16 B = 28 rows x 256 B
            uint4 val = *reinterpret_cast<const uint4 *>(obuf + kp * OUTP + part * 16);
            uint32_t w[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (safe) {
                    // negate where the sign is -1: a code + 8 in 1..15 becomes 16 - it, nibble by nibble without carries
                    w[i] = (w[i] ^ late_mask[i]) + (late_mask[i] & 0x11111111u);
                }
                if (!ASYM) w[i] ^= 0x88888888u;   // code + 8 -> two's complement nibble
            }
            reinterpret_cast<uint4 *>(q + (size_t)row * (N / 2))[tid] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

}  // namespace

int launch_rotate_had28(const RotateArgs &a, cudaStream_t st) {
    const bool ok = a.n == N && a.K == KH && a.stride == 1 && a.q != nullptr && !a.fp32_mode &&
                    (!a.asym || a.q_zero != nullptr) &&
                    a.hadk != nullptr && (a.in_dtype == SR_F16 || (a.in_dtype == SR_BF16 && a.cast_in_to_f16)) &&
                    aligned16(a.x) && aligned16(a.q) && (a.out == nullptr || (a.out_dtype == SR_F16 && aligned4(a.out)));
    if (!ok) return SR_ERR_UNSUPPORTED;
    const int sm_count = current_sm_count();
    const uint32_t grid = a.rows < (uint32_t)(2 * sm_count) ? a.rows : (uint32_t)(2 * sm_count);
    const bool late = a.clip == 1.f && a.out == nullptr && !a.asym;
#define SR_H28(T, LATE, ASYM)                                                                                  \
    do {                                                                                                   \
        auto kfn = rotate_quant_had28_kernel<T, LATE, ASYM>;                                                   \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);\
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "rotate_quant: %s", cudaGetErrorString(e));         \
        launch_pdl(kfn, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, st, (const T *)a.x, (const __half *)a.hadk,   \
                   a.sign, a.expert_ids, a.rows, a.scale, a.clip, a.q, a.q_scale, a.q_zero, (__half *)a.out); \
    } while (0)
    if (a.in_dtype == SR_F16) {
        if (late) SR_H28(__half, true, false);
        else if (a.asym) SR_H28(__half, false, true);
        else SR_H28(__half, false, false);
    } else {
        if (late) SR_H28(__nv_bfloat16, true, false);
        else if (a.asym) SR_H28(__nv_bfloat16, false, true);
        else SR_H28(__nv_bfloat16, false, false);
    }
#undef SR_H28
    return check_launch("rotate_quant_had28");
}

}  // namespace sr
