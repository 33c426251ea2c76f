// W4A4 GEMM for the decode regime (at most 64 activation rows): the int4 weights are streamed
// from HBM exactly once and multiplied on the tensor cores.
//
// Same contract as the other GEMM kernels (C = A * B^T on packed 4-bit operands, exact int32
// accumulation, optional fused dequant epilogue); replaces signrot/kernels/gemm.cu:7-85, whose
// 128 x 256 CTA tiles leave most SMs idle when M is small (at most N/256 CTAs).
//
// Work split.  CTAs are persistent over blocks of 16 weight rows; the 8 warps of a CTA take the
// 64-byte steps of K in turn (warp w: steps w, w + 8, ...), so together they read contiguous
// 512-byte runs of every row.  The weight block is the 16-row operand of mma.sync.m16n8k32 (s8),
// the activation rows are its 8-wide operand, one MMA column block per 8 tokens.
//
// The weight stream is what must never stall: every lane copies the 16 bytes of its own MMA
// fragments with cp.async into a private shared-memory slot, SK_DEPTH steps ahead of the math, and
// the queue runs on across row blocks, so the loads of the next block are in flight while this one
// is reduced and stored.  Slots are private to a lane: no barrier guards the ring.
// Nibble n becomes the byte 16*n ((w << 4) & 0xF0F0F0F0 for the even nibbles of a word, w &
// 0xF0F0F0F0 for the odd ones), which reorders k inside a word in the same way for both operands,
// so the dot product is unchanged; every product carries a factor 256 that the epilogue removes
// with an exact shift.  The eight partial accumulators of a block meet in shared memory.
#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace sr {

namespace {

constexpr int SK_WARPS = 8;
constexpr int SK_ROWS = 16;      // weight rows per CTA
constexpr int SK_STEP = 64;      // packed bytes of K per row and step (128 values)
constexpr int SK_DEPTH = 8;      // steps in flight per warp

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

// 16-byte asynchronous copy; bytes = 0 writes zeros without touching the source
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

constexpr size_t skinny_smem(int nt) {
    return (size_t)SK_WARPS * SK_DEPTH * 2 * 32 * 16 + (size_t)2 * SK_WARPS * nt * 4 * 32 * 4;
}

// NT = token blocks of 8 (M <= 8 * NT).  A = activations [M, K/2], B = weights [N, K/2].
template <int NT, bool A_UNSIGNED>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ B, uint32_t M, uint32_t N, uint32_t K,
                   Epilogue ep) {
    extern __shared__ __align__(16) uint8_t sk_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    // ring[warp][stage][row half][lane] (16 bytes each), then red[2][warp][NT][4][32]
    uint4 *ring = reinterpret_cast<uint4 *>(sk_smem) + (size_t)warp * SK_DEPTH * 64 + lane;
    const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring);
    int *red = reinterpret_cast<int *>(sk_smem + (size_t)SK_WARPS * SK_DEPTH * 2 * 32 * 16);

    const uint32_t kp = K >> 1;                         // packed bytes per row
    const uint32_t steps = (kp + SK_STEP - 1) / SK_STEP;
    const uint32_t blocks = (N + SK_ROWS - 1) / SK_ROWS;
    const bool has_steps = (uint32_t)warp < steps;
    const uint8_t *x_row = A + (size_t)g * kp + 16 * q;

    // queue of (row block, step) items of this warp, in the order they are consumed
    uint32_t iss_blk = blockIdx.x, iss_step = warp;
    auto issue = [&](int slot) {
        if (has_steps && iss_blk < blocks) {
            const uint32_t row = iss_blk * SK_ROWS + g;
            const bool k_ok = iss_step * SK_STEP + 16 * q + 16 <= kp;
            const uint8_t *src = B + (size_t)row * kp + (size_t)iss_step * SK_STEP + 16 * q;
            const uint32_t dst = ring_u32 + (uint32_t)slot * 1024;
            const bool lo = k_ok && row < N, hi = k_ok && row + 8 < N;
            cp_async16(dst, lo ? src : B, lo ? 16u : 0u);
            cp_async16(dst + 512, hi ? src + (size_t)8 * kp : B, hi ? 16u : 0u);
            iss_step += SK_WARPS;
            if (iss_step >= steps) {
                iss_step = warp;
                iss_blk += gridDim.x;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll 1
    for (int d = 0; d < SK_DEPTH; ++d) issue(d);

    // activation fragments of the step after the current one (they come from L1/L2, one step ahead is enough)
    auto load_x = [&](uint32_t step, uint4 (&x)[NT]) {
        const bool k_ok = step * SK_STEP + 16 * q + 16 <= kp;
#pragma unroll
        for (int t = 0; t < NT; ++t)
            x[t] = k_ok && (uint32_t)(g + 8 * t) < M
                       ? __ldg(reinterpret_cast<const uint4 *>(x_row + (size_t)(8 * t) * kp + (size_t)step * SK_STEP))
                       : make_uint4(0, 0, 0, 0);
    };
    uint4 xn[NT];
    if (has_steps) load_x(warp, xn);

    int slot = 0;
    uint32_t parity = 0;
    for (uint32_t blk = blockIdx.x; blk < blocks; blk += gridDim.x, parity ^= 1) {
        int acc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[t][i] = 0;
        if (has_steps) {
#pragma unroll 1
            for (uint32_t s = warp; s < steps; s += SK_WARPS) {
                uint4 x[NT];
#pragma unroll
                for (int t = 0; t < NT; ++t) x[t] = xn[t];
                load_x(s + SK_WARPS < steps ? s + SK_WARPS : (uint32_t)warp, xn);
                asm volatile("cp.async.wait_group %0;" ::"n"(SK_DEPTH - 1) : "memory");
                const uint4 cl = ring[slot * 64], ch = ring[slot * 64 + 32];
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
                issue(slot);   // after the math that consumed the slot
                slot = slot + 1 == SK_DEPTH ? 0 : slot + 1;
            }
        }
        int *rb = red + (size_t)parity * SK_WARPS * NT * 128;
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) rb[((warp * NT + t) * 4 + i) * 32 + lane] = acc[t][i];
        __syncthreads();
        // fragment slot i of lane (g, q): weight row g + 8 * (i >> 1), token 2 * q + (i & 1) of its block.
        // The buffer written two blocks later is this one: the barrier of the block in between orders it.
        const uint32_t n0 = blk * SK_ROWS;
        for (int idx = tid; idx < NT * 128; idx += SK_WARPS * 32) {
            const int l = idx & 31, i = (idx >> 5) & 3, t = idx >> 7;
            int sum = 0;
#pragma unroll
            for (int w = 0; w < SK_WARPS; ++w) sum += rb[((w * NT + t) * 4 + i) * 32 + l];
            const uint32_t n = n0 + (l >> 2) + 8 * (i >> 1);
            const uint32_t m = 8 * t + 2 * (l & 3) + (i & 1);
            if (n < N && m < M) ep.store(m, n, sum >> 8, N);
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
}

}  // namespace

int launch_gemm_skinny(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                       const Epilogue &ep, cudaStream_t st) {
    SR_REQUIRE(M >= 1 && M <= 64, SR_ERR_UNSUPPORTED, "matmul: the decode kernel takes at most 64 rows");
    SR_REQUIRE(aligned16(A) && aligned16(B), SR_ERR_INVALID, "matmul: operands must be 16-byte aligned");
    SR_REQUIRE(K % 32 == 0, SR_ERR_INVALID, "matmul: K = %lld must be a multiple of 32", (long long)K);
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
    const int64_t blocks = cdiv<int64_t>(N, SK_ROWS);
    // two CTAs per SM; the row blocks are dealt round-robin, so shrink the grid to even the deal out
    int64_t ctas = 2 * (int64_t)sm_count;
    if (blocks < ctas) ctas = blocks;
    else ctas = cdiv<int64_t>(blocks, cdiv<int64_t>(blocks, ctas));
    const unsigned grid = (unsigned)ctas;
#define SR_SK(NT)                                                                                              \
    do {                                                                                                       \
        auto kfn = a_unsigned ? gemm_skinny_kernel<NT, true> : gemm_skinny_kernel<NT, false>;                  \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                                             (int)skinny_smem(NT));                                            \
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "matmul: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        kfn<<<grid, SK_WARPS * 32, skinny_smem(NT), st>>>(A, B, (uint32_t)M, (uint32_t)N, (uint32_t)K, ep);    \
    } while (0)
    if (nt == 1) SR_SK(1);
    else if (nt == 2) SR_SK(2);
    else if (nt == 4) SR_SK(4);
    else SR_SK(8);
#undef SR_SK
    return check_launch("gemm_skinny");
}

}  // namespace sr
