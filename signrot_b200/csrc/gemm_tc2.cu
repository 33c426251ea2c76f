// Persistent W4A4 GEMM on tcgen05 (kind::i8) with register-path unpack.
//
// Same contract as gemm_tc.cu (C = A * B^T on packed 4-bit operands, exact int32 accumulation in
// TMEM, optional fused dequant epilogue); replaces signrot/kernels/gemm.cu:7-85 + quant.cu:66-131.
//
// Why a second design: with packed tiles staged in shared memory, every 128-wide k-block moves
// 144 KB through the SM's shared-memory port (TMA fill 24 + unpack read 24 + unpack write 48 +
// tensor-core read 48), which caps the tensor pipe well below its peak.  Here the packed
// operands never touch shared memory: eight unpack warps load them from global memory (L2) into
// registers two k-blocks ahead, expand nibble n to byte 16*n, and write only the int8 tiles
// (128-byte swizzled, K-major) that tcgen05.mma reads: 96 KB per k-block.
//
// One CTA per SM, persistent over 128 x 256 output tiles (tile index = blockIdx.x + i*gridDim.x,
// n fastest so that concurrently running CTAs share the same activation rows in L2):
//   warp 0       allocates all 512 TMEM columns (two 256-column accumulators) and issues
//                tcgen05.mma from one lane; tcgen05.commit releases ring stages / publishes tiles
//   warps 1..4   epilogue: tcgen05.ld of the finished accumulator while the next tile's MMAs
//                run into the other one; exact shift by 8, dequant, fp16/int32 stores
//   warps 5..    unpack (512 threads by default: three 16-byte packed chunks each per k-block)
// Every mbarrier wait is bounded by a cycle limit (abort flag + device status word).
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include <cstdlib>

namespace sr {
namespace tc2 {

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int SU = 4;                    // int8 ring depth
constexpr int UN_A = BM * BK;            // 16 KB
constexpr int UN_B = BN * BK;            // 32 KB
constexpr int STAGE = UN_A + UN_B;       // 48 KB
constexpr int PF = 2;                    // k-blocks prefetched into registers
constexpr long long WAIT_BUDGET = 1500000000ll;
constexpr int SMEM_BYTES = SU * STAGE + 256 + 1024;

__device__ int g_status;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_BUDGET) {
            *abort_flag = code;
            atomicCAS(&g_status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accum)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct Cursor {
    uint32_t tile, kb;  // tile index in the global tile list, k-block inside it
};

// NUM_UNPACK = number of unpack threads (256 or 512): more warps hide more of the L2 latency and
// of the dependent-issue latency of the expand/store sequence.
template <bool A_UNSIGNED, int NUM_UNPACK>
__global__ void __launch_bounds__(160 + NUM_UNPACK, 1)
gemm_tc2_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ B, uint32_t M, uint32_t N, uint32_t K,
                Epilogue ep) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + SU * STAGE;
    auto un_full = [&](int s) { return bars + 8u * s; };
    auto un_empty = [&](int s) { return bars + 8u * (SU + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * SU + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * SU + 2 + b); };

    constexpr int CHUNKS = (BM + BN) * 4 / NUM_UNPACK;  // packed 16-byte chunks per thread per k-block
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool small = (A_UNSIGNED ? 120u : 64u) * (uint64_t)K < (1u << 22);
    const uint32_t tiles_n = (N + BN - 1) / BN, tiles_m = (M + BM - 1) / BM;
    const uint32_t num_tiles = tiles_n * tiles_m;
    const uint32_t num_kb = (K + BK - 1) / BK;
    const uint32_t kp = K >> 1;  // packed bytes per row

    if (tid == 0) {
        abort_flag = g_status;
        for (int s = 0; s < SU; ++s) {
            mbar_init(un_full(s), NUM_UNPACK);
            mbar_init(un_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = tmem_base_slot;
    volatile int *ab = &abort_flag;

    if (*ab == 0) {
        if (warp == 0) {
            // ------------------------------------------------ MMA issuer
            if (lane == 0) {
                const uint32_t idesc = (2u << 4) | ((A_UNSIGNED ? 0u : 1u) << 7) | (1u << 10) |
                                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
                uint32_t g = 0, it = 0;
                bool ok = true;
                for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                    const uint32_t buf = it & 1;
                    ok = mbar_wait(acc_empty(buf), ((it >> 1) & 1) ^ 1, ab, 31);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t d_tmem = tmem_acc + buf * BN;
                    for (uint32_t kb = 0; kb < num_kb; ++kb, ++g) {
                        const int s = g % SU;
                        ok = mbar_wait(un_full(s), (g / SU) & 1, ab, 32);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t da = make_desc(base + s * STAGE);
                        const uint64_t db = make_desc(base + s * STAGE + UN_A);
#pragma unroll
                        for (int kk = 0; kk < BK / 32; ++kk)
                            mma_i8(d_tmem, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc,
                                   (kb > 0 || kk > 0) ? 1u : 0u);
                        mma_commit(un_empty(s));
                    }
                    if (ok) mma_commit(acc_full(buf));
                }
            }
        } else if (warp <= 4) {
            // ------------------------------------------------ epilogue
            const uint32_t quarter = warp & 3;
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const uint32_t buf = it & 1;
                const uint32_t m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
                ok = mbar_wait(acc_full(buf), (it >> 1) & 1, ab, 33);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t row = m0 + quarter * 32 + lane;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    int v[32];
                    tmem_ld32(tmem_acc + ((quarter * 32u) << 16) + buf * BN + (uint32_t)(c * 32), v);
                    if (c == BN / 32 - 1) {
                        // every value of this accumulator is in registers: hand it back
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        mbar_arrive(acc_empty(buf));
                    }
                    store_acc_chunk(ep, row, n0 + c * 32, v, M, N, small);
                }
            }
        } else {
            // ------------------------------------------------ unpack (register path)
            const int t = tid - 160;  // 0..255
            const uint32_t total = ((num_tiles > blockIdx.x) ? ((num_tiles - blockIdx.x - 1) / gridDim.x + 1) : 0) * num_kb;
            uint4 pf[PF][CHUNKS];
            Cursor ld = {blockIdx.x, 0};
            uint32_t issued = 0;
            // per-tile row addresses (recomputed only when the load cursor enters a new tile)
            const uint8_t *rowp[CHUNKS];
            uint32_t colq[CHUNKS];
            auto set_tile = [&](uint32_t tile) {
                const uint32_t m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
#pragma unroll
                for (int i = 0; i < CHUNKS; ++i) {
                    const int id = i * NUM_UNPACK + t;
                    const bool is_a = id < BM * 4;
                    const int cid = is_a ? id : id - BM * 4;
                    const uint32_t r = (is_a ? m0 : n0) + (cid >> 2);
                    colq[i] = (cid & 3) * 16;
                    rowp[i] = (r < (is_a ? M : N)) ? (is_a ? A : B) + (size_t)r * kp + colq[i] : nullptr;
                }
            };
            set_tile(ld.tile);
            auto issue = [&](uint4 (&dst)[CHUNKS]) {
                const uint32_t colb = ld.kb * (BK / 2);
#pragma unroll
                for (int i = 0; i < CHUNKS; ++i) {
                    dst[i] = make_uint4(0, 0, 0, 0);
                    if (rowp[i] != nullptr && colb + colq[i] < kp) dst[i] = __ldg(reinterpret_cast<const uint4 *>(rowp[i] + colb));
                }
                if (++ld.kb == num_kb) {
                    ld.kb = 0;
                    ld.tile += gridDim.x;
                    if (ld.tile < num_tiles) set_tile(ld.tile);
                }
                ++issued;
            };
            auto unpack_to = [&](const uint4 (&src)[CHUNKS], int s) {
                uint8_t *ua = base_ptr + s * STAGE;
                uint8_t *ub = ua + UN_A;
#pragma unroll
                for (int i = 0; i < CHUNKS; ++i) {
                    const int id = i * NUM_UNPACK + t;
                    const bool is_a = id < BM * 4;
                    const int cid = is_a ? id : id - BM * 4;
                    const int r = cid >> 2, qd = cid & 3;
                    const uint4 pk = src[i];
                    uint4 e, o;
                    e.x = (pk.x << 4) & 0xF0F0F0F0u; o.x = pk.x & 0xF0F0F0F0u;
                    e.y = (pk.y << 4) & 0xF0F0F0F0u; o.y = pk.y & 0xF0F0F0F0u;
                    e.z = (pk.z << 4) & 0xF0F0F0F0u; o.z = pk.z & 0xF0F0F0F0u;
                    e.w = (pk.w << 4) & 0xF0F0F0F0u; o.w = pk.w & 0xF0F0F0F0u;
                    uint8_t *rowp = (is_a ? ua : ub) + (r >> 3) * 1024 + (r & 7) * 128;
                    *reinterpret_cast<uint4 *>(rowp + (((2 * qd) ^ (r & 7)) << 4)) = e;
                    *reinterpret_cast<uint4 *>(rowp + (((2 * qd + 1) ^ (r & 7)) << 4)) = o;
                }
            };
#pragma unroll
            for (int d = 0; d < PF; ++d)
                if (issued < total) issue(pf[d]);
            bool ok = true;
            for (uint32_t g = 0; g < total && ok; g += PF) {
#pragma unroll
                for (int d = 0; d < PF; ++d) {
                    const uint32_t gg = g + d;
                    if (gg < total && ok) {
                        const int s = gg % SU;
                        ok = mbar_wait(un_empty(s), ((gg / SU) & 1) ^ 1, ab, 34);
                        if (ok) {
                            unpack_to(pf[d], s);
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            mbar_arrive(un_full(s));
                            if (issued < total) issue(pf[d]);
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------- teardown
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*ab != 0 && tid == 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) {
        }
    }
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(512u) : "memory");
    }
}

}  // namespace tc2

int launch_gemm_tc2(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                    const Epilogue &ep, cudaStream_t st) {
    using namespace tc2;
    SR_REQUIRE(aligned16(A) && aligned16(B), SR_ERR_INVALID, "matmul: operands must be 16-byte aligned");
    SR_REQUIRE(K % 32 == 0, SR_ERR_INVALID, "matmul: K = %lld must be a multiple of 32", (long long)K);
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    const int64_t tiles = cdiv<int64_t>(N, BN) * cdiv<int64_t>(M, BM);
    const unsigned grid = (unsigned)(tiles < sm_count ? tiles : sm_count);
    static int unpack_threads = 0;
    if (unpack_threads == 0) {
        const char *env = getenv("SIGNROT_B200_TC2_UNPACK");  // tuning knob: 256 or 512 unpack threads
        unpack_threads = (env && atoi(env) == 256) ? 256 : 512;
    }
    auto kfn = unpack_threads == 256 ? (a_unsigned ? gemm_tc2_kernel<true, 256> : gemm_tc2_kernel<false, 256>)
                                     : (a_unsigned ? gemm_tc2_kernel<true, 512> : gemm_tc2_kernel<false, 512>);
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "matmul: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    kfn<<<grid, 160 + unpack_threads, SMEM_BYTES, st>>>(A, B, (uint32_t)M, (uint32_t)N, (uint32_t)K, ep);
    return check_launch("gemm_tc2");
}

int tc2_device_status(int *out, bool clear) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, tc2::g_status, sizeof(int));
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
    if (clear && v != 0) {
        const int z = 0;
        cudaMemcpyToSymbol(tc2::g_status, &z, sizeof(int));
    }
    *out = v;
    return SR_OK;
}

}  // namespace sr
