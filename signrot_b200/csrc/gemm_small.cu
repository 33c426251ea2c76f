// W4A4 GEMM for few rows on dp4a (selectable as kernel 1; the mma.sync kernel in gemm_skinny.cu is the
// default of the decode regime): C[M,N] = A[M,K] * B[N,K]^T with packed 4-bit
// operands, exact int32 accumulation, optional fused dequant epilogue.
//
// Replaces signrot/kernels/gemm.cu:7-85 (CUTLASS Sm80 s4 tensor-op GEMM, one
// 128x256 tile per CTA, at most 16 CTAs when M <= 128) for the weight-streaming
// regime, where the int4 weights (N*K/2 bytes) are the only traffic that matters:
// the grid is sized by N so that every SM streams its own slab of weights once,
// the few activation rows are unpacked to int8 once per CTA into shared memory
// and the products run on dp4a.
//
// Nibble n is expanded to the byte 16*n (its two's complement nibble moved to the
// high half of the byte), so no sign extension is needed: every product carries a
// factor 256 that the epilogue removes with an exact arithmetic shift.  Both
// operands use the same even/odd nibble order inside a 32-bit word, so the order
// of the k index inside a word is irrelevant to the dot product.
#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace sr {

template <bool A_UNSIGNED>
__device__ __forceinline__ int dp4a_mixed(uint32_t a, uint32_t b, int c) {
    int d;
    if (A_UNSIGNED)
        asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    else
        asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// MT activation rows per CTA (in shared memory as int8, K bytes each), 8 warps,
// each warp owns NR weight rows at a time and walks K in 16-byte packed chunks.
template <int MT, int NR, bool A_UNSIGNED>
__global__ void __launch_bounds__(256)
gemm_small_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ B, uint32_t M, uint32_t N, uint32_t K,
                  uint32_t rows_per_cta, Epilogue ep) {
    extern __shared__ __align__(16) uint8_t a_s8[];  // [MT][K]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t m0 = blockIdx.y * MT;
    const uint32_t kp = K >> 1;        // packed bytes per row
    const uint32_t chunks = kp >> 4;   // 16-byte packed chunks per row (K % 32 == 0)

    // unpack the activation tile: packed chunk c of row m -> 32 bytes at a_s8[m*K + 32c]
    for (uint32_t i = tid; i < MT * chunks; i += 256) {
        const uint32_t m = i / chunks, c = i % chunks;
        uint4 pk = make_uint4(0, 0, 0, 0);
        if (m0 + m < M) pk = __ldg(reinterpret_cast<const uint4 *>(A + (size_t)(m0 + m) * kp) + c);
        const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
        uint4 e, o;
        e.x = (w[0] << 4) & 0xF0F0F0F0u; o.x = w[0] & 0xF0F0F0F0u;
        e.y = (w[1] << 4) & 0xF0F0F0F0u; o.y = w[1] & 0xF0F0F0F0u;
        e.z = (w[2] << 4) & 0xF0F0F0F0u; o.z = w[2] & 0xF0F0F0F0u;
        e.w = (w[3] << 4) & 0xF0F0F0F0u; o.w = w[3] & 0xF0F0F0F0u;
        uint4 *dst = reinterpret_cast<uint4 *>(a_s8 + (size_t)m * K + (size_t)c * 32);
        dst[0] = e;
        dst[1] = o;
    }
    __syncthreads();

    const uint32_t n_begin = blockIdx.x * rows_per_cta;
    const uint32_t n_end = min(N, n_begin + rows_per_cta);
    for (uint32_t n0 = n_begin + warp * NR; n0 < n_end; n0 += 8 * NR) {
        int acc[NR][MT];
#pragma unroll
        for (int r = 0; r < NR; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0;
        for (uint32_t c = lane; c < chunks; c += 32) {
            uint4 be[NR], bo[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                uint4 pk = make_uint4(0, 0, 0, 0);
                if (n0 + r < n_end) pk = __ldg(reinterpret_cast<const uint4 *>(B + (size_t)(n0 + r) * kp) + c);
                be[r].x = (pk.x << 4) & 0xF0F0F0F0u; bo[r].x = pk.x & 0xF0F0F0F0u;
                be[r].y = (pk.y << 4) & 0xF0F0F0F0u; bo[r].y = pk.y & 0xF0F0F0F0u;
                be[r].z = (pk.z << 4) & 0xF0F0F0F0u; bo[r].z = pk.z & 0xF0F0F0F0u;
                be[r].w = (pk.w << 4) & 0xF0F0F0F0u; bo[r].w = pk.w & 0xF0F0F0F0u;
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint4 *ap = reinterpret_cast<const uint4 *>(a_s8 + (size_t)m * K + (size_t)c * 32);
                const uint4 ae = ap[0], ao = ap[1];
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    int s = acc[r][m];
                    s = dp4a_mixed<A_UNSIGNED>(ae.x, be[r].x, s);
                    s = dp4a_mixed<A_UNSIGNED>(ae.y, be[r].y, s);
                    s = dp4a_mixed<A_UNSIGNED>(ae.z, be[r].z, s);
                    s = dp4a_mixed<A_UNSIGNED>(ae.w, be[r].w, s);
                    s = dp4a_mixed<A_UNSIGNED>(ao.x, bo[r].x, s);
                    s = dp4a_mixed<A_UNSIGNED>(ao.y, bo[r].y, s);
                    s = dp4a_mixed<A_UNSIGNED>(ao.z, bo[r].z, s);
                    s = dp4a_mixed<A_UNSIGNED>(ao.w, bo[r].w, s);
                    acc[r][m] = s;
                }
            }
        }
        // reduce over lanes; lane (r*MT + m) % 32 keeps result (r, m)
#pragma unroll
        for (int r = 0; r < NR; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                int s = acc[r][m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == ((r * MT + m) & 31)) {
                    const uint32_t row = m0 + m, col = n0 + r;
                    if (row < M && col < n_end) ep.store(row, col, s >> 8, N);
                }
            }
    }
}

template <bool A_UNSIGNED>
static int launch_small_t(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, const Epilogue &ep,
                          cudaStream_t st) {
    int mt = K <= 8192 ? 16 : (K <= 16384 ? 8 : 4);
    if (M <= 4) mt = 4;
    else if (M <= 8 && mt > 8) mt = 8;
    const size_t smem = (size_t)mt * K;
    SR_REQUIRE(smem <= 200 * 1024, SR_ERR_UNSUPPORTED, "matmul (few rows): K = %lld is too large", (long long)K);
    const uint32_t rows_per_cta = 16;
    dim3 grid((unsigned)cdiv<int64_t>(N, rows_per_cta), (unsigned)cdiv<int64_t>(M, mt));
#define SR_SMALL(MT_)                                                                                           \
    do {                                                                                                        \
        auto kfn = gemm_small_kernel<MT_, 2, A_UNSIGNED>;                                                       \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);    \
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "matmul: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        kfn<<<grid, 256, smem, st>>>(A, B, (uint32_t)M, (uint32_t)N, (uint32_t)K, rows_per_cta, ep);           \
    } while (0)
    if (mt == 16) SR_SMALL(16);
    else if (mt == 8) SR_SMALL(8);
    else SR_SMALL(4);
#undef SR_SMALL
    return check_launch("gemm_small");
}

int launch_gemm_small(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                      const Epilogue &ep, cudaStream_t st) {
    return a_unsigned ? launch_small_t<true>(A, B, M, N, K, ep, st) : launch_small_t<false>(A, B, M, N, K, ep, st);
}

}  // namespace sr
