// W4A4 GEMM for the decode regime (at most 64 activation rows): the int4 weights are streamed
// from HBM exactly once, straight into registers, and multiplied on the tensor cores.
//
// Same contract as the other GEMM kernels (C = A * B^T on packed 4-bit operands, exact int32
// accumulation, optional fused dequant epilogue); replaces signrot/kernels/gemm.cu:7-85, whose
// 128 x 256 CTA tiles leave most SMs idle when M is small (at most N/256 CTAs).
//
// Work split.  A CTA owns 16 weight rows (grid = N / 16) and its 8 warps take the 64-byte steps
// of K in turn (warp w: steps w, w + 8, ...), so the eight warps together read contiguous 512-byte
// runs of every row.  The weight tile is the 16-row operand of mma.sync.m16n8k32 (s8), the
// activation rows are its 8-wide operand, one MMA column block per 8 tokens.
//
// No shared-memory staging: a lane's 16-byte load is exactly the data of its own fragments.
// Nibble n becomes the byte 16*n ((w << 4) & 0xF0F0F0F0 for the even nibbles of a word, w &
// 0xF0F0F0F0 for the odd ones), which reorders k inside a word in the same way for both operands,
// so the dot product is unchanged; every product carries a factor 256 that the epilogue removes
// with an exact shift.  Loads run PF steps ahead of the math in registers.
// The eight partial accumulators meet in shared memory; the epilogue is the shared one.
#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace sr {

namespace {

constexpr int SK_WARPS = 8;
constexpr int SK_ROWS = 16;      // weight rows per CTA
constexpr int SK_STEP = 64;      // packed bytes of K per row and step (128 values)
constexpr int SK_PF = 4;         // steps in flight per warp

template <bool A_UNSIGNED>
__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (A_UNSIGNED)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t word(const uint4 &v, int j) { return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w)); }

// NT = token blocks of 8 (M <= 8 * NT).  A = activations [M, K/2], B = weights [N, K/2].
template <int NT, bool A_UNSIGNED>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ B, uint32_t M, uint32_t N, uint32_t K,
                   Epilogue ep) {
    __shared__ int red[SK_WARPS][NT][4][32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const uint32_t kp = K >> 1;                         // packed bytes per row
    const uint32_t steps = (kp + SK_STEP - 1) / SK_STEP;
    const uint32_t n0 = blockIdx.x * SK_ROWS;

    // this lane's 16 bytes of a step: offset 16*q of the two weight rows g, g + 8 and of token rows g + 8*t
    const bool row_lo = n0 + g < N, row_hi = n0 + g + 8 < N;
    const uint8_t *w_lo = B + (size_t)(n0 + g) * kp + 16 * q;
    const uint8_t *w_hi = B + (size_t)(n0 + g + 8) * kp + 16 * q;
    const uint8_t *x_row = A + (size_t)g * kp + 16 * q;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    auto in_k = [&](uint32_t step) { return step < steps && step * SK_STEP + 16 * q + 16 <= kp; };

    int acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[t][i] = 0;

    uint4 wl[SK_PF], wh[SK_PF];
#pragma unroll
    for (int p = 0; p < SK_PF; ++p) {
        const uint32_t s = warp + p * SK_WARPS;
        const bool ok = in_k(s);
        wl[p] = ok && row_lo ? __ldg(reinterpret_cast<const uint4 *>(w_lo + (size_t)s * SK_STEP)) : zero4;
        wh[p] = ok && row_hi ? __ldg(reinterpret_cast<const uint4 *>(w_hi + (size_t)s * SK_STEP)) : zero4;
    }
    for (uint32_t s0 = warp; s0 < steps; s0 += SK_PF * SK_WARPS) {
#pragma unroll
        for (int p = 0; p < SK_PF; ++p) {
            const uint32_t s = s0 + p * SK_WARPS;
            if (s >= steps) break;   // warp-uniform
            const bool ok = in_k(s);
            uint4 x[NT];
#pragma unroll
            for (int t = 0; t < NT; ++t)
                x[t] = ok && (uint32_t)(g + 8 * t) < M
                           ? __ldg(reinterpret_cast<const uint4 *>(x_row + (size_t)(8 * t) * kp + (size_t)s * SK_STEP))
                           : zero4;
            const uint4 cl = wl[p], ch = wh[p];
            {   // refill this slot for the step SK_PF rounds ahead
                const uint32_t sn = s + SK_PF * SK_WARPS;
                const bool okn = in_k(sn);
                wl[p] = okn && row_lo ? __ldg(reinterpret_cast<const uint4 *>(w_lo + (size_t)sn * SK_STEP)) : zero4;
                wh[p] = okn && row_hi ? __ldg(reinterpret_cast<const uint4 *>(w_hi + (size_t)sn * SK_STEP)) : zero4;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t pl = word(cl, j), ph = word(ch, j);
                uint32_t a[4];
                a[0] = (pl << 4) & 0xF0F0F0F0u;   // row g,     even nibbles
                a[1] = (ph << 4) & 0xF0F0F0F0u;   // row g + 8, even nibbles
                a[2] = pl & 0xF0F0F0F0u;          // row g,     odd nibbles
                a[3] = ph & 0xF0F0F0F0u;          // row g + 8, odd nibbles
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const uint32_t px = word(x[t], j);
                    mma_s8<A_UNSIGNED>(acc[t], a, (px << 4) & 0xF0F0F0F0u, px & 0xF0F0F0F0u);
                }
            }
        }
    }

#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][t][i][lane] = acc[t][i];
    __syncthreads();
    // thread (i = tid / 32 in 0..3 twice over, lane) sums the eight partials of fragment slot i:
    // slot i of lane (g, q) is weight row g + 8 * (i >> 1), token 2 * q + (i & 1) of its block
    for (int idx = tid; idx < NT * 4 * 32; idx += SK_WARPS * 32) {
        const int l = idx & 31, i = (idx >> 5) & 3, t = idx >> 7;
        int sum = 0;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) sum += red[w][t][i][l];
        const uint32_t n = n0 + (l >> 2) + 8 * (i >> 1);
        const uint32_t m = 8 * t + 2 * (l & 3) + (i & 1);
        if (n < N && m < M) ep.store(m, n, sum >> 8, N);
    }
}

}  // namespace

int launch_gemm_skinny(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                       const Epilogue &ep, cudaStream_t st) {
    SR_REQUIRE(M >= 1 && M <= 64, SR_ERR_UNSUPPORTED, "matmul: the decode kernel takes at most 64 rows");
    SR_REQUIRE(aligned16(A) && aligned16(B), SR_ERR_INVALID, "matmul: operands must be 16-byte aligned");
    SR_REQUIRE(K % 32 == 0, SR_ERR_INVALID, "matmul: K = %lld must be a multiple of 32", (long long)K);
    const unsigned grid = (unsigned)cdiv<int64_t>(N, SK_ROWS);
    const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
#define SR_SK(NT)                                                                                              \
    do {                                                                                                       \
        if (a_unsigned)                                                                                        \
            gemm_skinny_kernel<NT, true><<<grid, SK_WARPS * 32, 0, st>>>(A, B, (uint32_t)M, (uint32_t)N,       \
                                                                          (uint32_t)K, ep);                    \
        else                                                                                                   \
            gemm_skinny_kernel<NT, false><<<grid, SK_WARPS * 32, 0, st>>>(A, B, (uint32_t)M, (uint32_t)N,      \
                                                                           (uint32_t)K, ep);                   \
    } while (0)
    if (nt == 1) SR_SK(1);
    else if (nt == 2) SR_SK(2);
    else if (nt == 4) SR_SK(4);
    else SR_SK(8);
#undef SR_SK
    return check_launch("gemm_skinny");
}

}  // namespace sr
