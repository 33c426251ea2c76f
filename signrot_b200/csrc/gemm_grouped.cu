// Grouped W4A4 GEMM: C_p[m_p, n_p] = A_p[m_p, k_p] * B_p[n_p, k_p]^T for P problems in
// one launch, every size, pointer and leading dimension resident in device memory.
//
// Replaces signrot/kernels/gemm_grouped.cu:19-120 (CUTLASS GemmGrouped, Sm80 s4 tensor op,
// device-side problem visitor) behind the same contract as signrot._CUDA.matmul_grouped
// (signrot/kernels/bindings.cpp:49-91): nothing is read on the host, so per-expert row
// counts that change every step do not break CUDA-graph replay.
//
// Two kernels share the work and the device decides which one has it (see sr_matmul_grouped
// below): prefill-sized calls in the MoE block's layout run on the CTA-pair tcgen05 kernel of
// gemm_tc3.cu, everything else on the CUDA-core kernel in this file.
//
// Its persistent CTAs walk a tile list that each CTA derives from the problem sizes on the
// device: problem p contributes ceil(m_p/8) x ceil(n_p/32) tiles.  A tile unpacks its
// (at most 8) activation rows to int8 in shared memory once and streams 32 weight rows
// through dp4a (nibble n stored as byte 16n, factor 256 removed by an exact shift).  MoE
// decode is the weight-streaming regime (a handful of rows per expert), which is what
// this kernel is shaped for.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include <algorithm>

namespace sr {

constexpr int G_MT = 8;    // activation rows per tile
constexpr int G_NT = 32;   // weight rows per tile
constexpr int G_SMEM = 200 * 1024;

__device__ int g_grouped_status;

template <bool A_UNSIGNED>
__device__ __forceinline__ int dp4a_g(uint32_t a, uint32_t b, int c) {
    int d;
    if (A_UNSIGNED)
        asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    else
        asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Leading dimensions are in elements (4-bit values for A and B, int32 for C), as CUTLASS
// takes them (signrot/nn/moe.py:104-111 passes k, k and n).
template <bool A_UNSIGNED>
__global__ void __launch_bounds__(256)
gemm_grouped_kernel(uint32_t smem_bytes, const int32_t *__restrict__ sizes, uint32_t P, const int64_t *__restrict__ ptr_a,
                    const int64_t *__restrict__ ptr_b, const int64_t *__restrict__ ptr_c,
                    const int64_t *__restrict__ lda, const int64_t *__restrict__ ldb,
                    const int64_t *__restrict__ ldc, const int32_t *__restrict__ done_elsewhere) {
    extern __shared__ __align__(16) uint8_t a_s8[];  // [G_MT][k]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the tensor-core kernel launched just before took the problems (its planning kernel says so)
    if (done_elsewhere != nullptr && *done_elsewhere != 0) return;

    uint32_t p = 0;
    uint64_t tile_base = 0;  // first tile id of problem p
    for (uint64_t t = blockIdx.x;; t += gridDim.x) {
        // advance to the problem that owns tile t
        uint32_t m = 0, n = 0, k = 0;
        uint64_t tiles_p = 0;
        while (p < P) {
            m = (uint32_t)sizes[3 * p];
            n = (uint32_t)sizes[3 * p + 1];
            k = (uint32_t)sizes[3 * p + 2];
            tiles_p = (uint64_t)cdiv<uint32_t>(m, G_MT) * cdiv<uint32_t>(n, G_NT);
            if (t < tile_base + tiles_p) break;
            tile_base += tiles_p;
            ++p;
        }
        if (p >= P) break;
        if ((k & 31u) != 0 || (size_t)k * G_MT > (size_t)smem_bytes) {
            if (tid == 0) atomicCAS(&g_grouped_status, 0, 21);  // unsupported k
            continue;
        }
        const uint32_t local = (uint32_t)(t - tile_base);
        const uint32_t n_tiles = cdiv<uint32_t>(n, G_NT);
        const uint32_t m0 = (local / n_tiles) * G_MT, n0 = (local % n_tiles) * G_NT;
        const uint8_t *A = reinterpret_cast<const uint8_t *>(ptr_a[p]);
        const uint8_t *B = reinterpret_cast<const uint8_t *>(ptr_b[p]);
        int32_t *C = reinterpret_cast<int32_t *>(ptr_c[p]);
        const size_t sa = (size_t)lda[p] >> 1, sb = (size_t)ldb[p] >> 1, sc = (size_t)ldc[p];
        const uint32_t chunks = k >> 5;  // 16-byte packed chunks per row

        __syncthreads();  // previous tile's readers are done with a_s8
        for (uint32_t i = tid; i < G_MT * chunks; i += 256) {
            const uint32_t r = i / chunks, c = i % chunks;
            uint4 pk = make_uint4(0, 0, 0, 0);
            if (m0 + r < m) pk = *reinterpret_cast<const uint4 *>(A + (size_t)(m0 + r) * sa + (size_t)c * 16);
            uint4 e, o;
            e.x = (pk.x << 4) & 0xF0F0F0F0u; o.x = pk.x & 0xF0F0F0F0u;
            e.y = (pk.y << 4) & 0xF0F0F0F0u; o.y = pk.y & 0xF0F0F0F0u;
            e.z = (pk.z << 4) & 0xF0F0F0F0u; o.z = pk.z & 0xF0F0F0F0u;
            e.w = (pk.w << 4) & 0xF0F0F0F0u; o.w = pk.w & 0xF0F0F0F0u;
            uint4 *dst = reinterpret_cast<uint4 *>(a_s8 + (size_t)r * k + (size_t)c * 32);
            dst[0] = e;
            dst[1] = o;
        }
        __syncthreads();

        const uint32_t n_end = min(n, n0 + G_NT);
        const int m_valid = (int)min((uint32_t)G_MT, m - m0);   // rows of the tile that exist (uniform over the CTA)
        for (uint32_t nr = n0 + warp * 2; nr < n_end; nr += 16) {
            int acc[2][G_MT];
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int mm = 0; mm < G_MT; ++mm) acc[r][mm] = 0;
            for (uint32_t c = lane; c < chunks; c += 32) {
                uint4 be[2], bo[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    uint4 pk = make_uint4(0, 0, 0, 0);
                    if (nr + r < n_end) pk = __ldg(reinterpret_cast<const uint4 *>(B + (size_t)(nr + r) * sb + (size_t)c * 16));
                    be[r].x = (pk.x << 4) & 0xF0F0F0F0u; bo[r].x = pk.x & 0xF0F0F0F0u;
                    be[r].y = (pk.y << 4) & 0xF0F0F0F0u; bo[r].y = pk.y & 0xF0F0F0F0u;
                    be[r].z = (pk.z << 4) & 0xF0F0F0F0u; bo[r].z = pk.z & 0xF0F0F0F0u;
                    be[r].w = (pk.w << 4) & 0xF0F0F0F0u; bo[r].w = pk.w & 0xF0F0F0F0u;
                }
#pragma unroll
                for (int mm = 0; mm < G_MT; ++mm) {
                    if (mm >= m_valid) break;
                    const uint4 *ap = reinterpret_cast<const uint4 *>(a_s8 + (size_t)mm * k + (size_t)c * 32);
                    const uint4 ae = ap[0], ao = ap[1];
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        int s = acc[r][mm];
                        s = dp4a_g<A_UNSIGNED>(ae.x, be[r].x, s);
                        s = dp4a_g<A_UNSIGNED>(ae.y, be[r].y, s);
                        s = dp4a_g<A_UNSIGNED>(ae.z, be[r].z, s);
                        s = dp4a_g<A_UNSIGNED>(ae.w, be[r].w, s);
                        s = dp4a_g<A_UNSIGNED>(ao.x, bo[r].x, s);
                        s = dp4a_g<A_UNSIGNED>(ao.y, bo[r].y, s);
                        s = dp4a_g<A_UNSIGNED>(ao.z, bo[r].z, s);
                        s = dp4a_g<A_UNSIGNED>(ao.w, bo[r].w, s);
                        acc[r][mm] = s;
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int mm = 0; mm < G_MT; ++mm) {
                    int s = acc[r][mm];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    if (lane == ((r * G_MT + mm) & 31) && m0 + mm < m && nr + r < n_end)
                        C[(size_t)(m0 + mm) * sc + nr + r] = s >> 8;
                }
        }
    }
}

int grouped_device_status(int *out, bool clear) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_grouped_status, sizeof(int));
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
    if (clear && v != 0) {
        const int z = 0;
        cudaMemcpyToSymbol(g_grouped_status, &z, sizeof(int));
    }
    *out = v;
    return SR_OK;
}

}  // namespace sr

using namespace sr;

extern "C" int sr_matmul_grouped(const void *problem_sizes, int64_t problem_count, const void *ptr_a,
                                 const void *ptr_b, const void *ptr_c, const void *lda, const void *ldb,
                                 const void *ldc, int signed_a, int64_t max_k, void *stream) {
    SR_REQUIRE(problem_count >= 0, SR_ERR_INVALID, "matmul_grouped: negative problem count");
    if (problem_count == 0) return SR_OK;
    SR_REQUIRE(problem_sizes && ptr_a && ptr_b && ptr_c && lda && ldb && ldc, SR_ERR_INVALID,
               "matmul_grouped: null pointer");
    const int sm_count = current_sm_count();
    // Prefill-sized calls in the layout the MoE block builds go to the tensor cores; which kernel has the
    // work is decided on the device (nothing here may read a size), so both are launched and one returns at once.
    const int32_t *on_tensor_cores = nullptr;
    if (problem_count <= 512) {
        const int rc = launch_gemm_tc3_ptr_array((const int32_t *)problem_sizes, problem_count, (const int64_t *)ptr_a,
                                                 (const int64_t *)ptr_b, (const int64_t *)ptr_c, (const int64_t *)lda,
                                                 (const int64_t *)ldb, (const int64_t *)ldc, signed_a == 0,
                                                 signed_a ? 131040 : 65536, &on_tensor_cores, as_stream(stream));
        if (rc) return rc;
    }
    auto kfn = signed_a ? gemm_grouped_kernel<false> : gemm_grouped_kernel<true>;
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "matmul_grouped: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    // max_k > 0: the caller guarantees k_p <= max_k, so the activation tile needs less shared
    // memory and more CTAs fit per SM; problems that break the promise set the status word.
    size_t smem = G_SMEM;
    int ctas_per_sm = 1;
    if (max_k > 0 && (size_t)max_k * G_MT <= (size_t)G_SMEM) {
        smem = (size_t)max_k * G_MT;
        ctas_per_sm = (int)std::min<size_t>(4, (size_t)(220 * 1024) / (smem + 1024));
        if (ctas_per_sm < 1) ctas_per_sm = 1;
    }
    kfn<<<sm_count * ctas_per_sm, 256, smem, as_stream(stream)>>>((uint32_t)smem, (const int32_t *)problem_sizes, (uint32_t)problem_count,
                                                     (const int64_t *)ptr_a, (const int64_t *)ptr_b,
                                                     (const int64_t *)ptr_c, (const int64_t *)lda,
                                                     (const int64_t *)ldb, (const int64_t *)ldc, on_tensor_cores);
    return check_launch("matmul_grouped");
}
