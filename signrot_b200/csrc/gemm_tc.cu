// W4A4 GEMM on the 5th-generation tensor cores (tcgen05, kind::i8) for sm_100a.
//
//   C[M,N] (int32 in TMEM) = A[M,K] (packed s4/u4) * B[N,K]^T (packed s4)
//
// Replaces signrot/kernels/gemm.cu:7-85 (CUTLASS device::Gemm<int4b_t, ..., Sm80>,
// mma.sync.m16n8k64.s4) and, with the fused epilogue, the separate dequant pass
// signrot/kernels/quant.cu:66-131 that re-reads the int32 matrix from HBM.
//
// Pipeline inside one CTA (192 threads, one 128 x 256 output tile):
//   warp 0      TMA producer: packed tiles (128 x 64 B of A, 256 x 64 B of B per
//               128-wide k-block) -> shared memory ring, mbarrier complete_tx
//   warps 2..5  unpackers: each packed nibble n becomes the int8 byte 16*n
//               (nibble moved to the high half of the byte: two ALU ops per eight
//               values, no sign extension), written in the 128-byte-swizzled
//               K-major layout tcgen05 reads; afterwards the same warps are the
//               epilogue (each owns one 32-lane quarter of TMEM)
//   warp 1      allocates TMEM and issues tcgen05.mma (one elected lane), four
//               K=32 instructions per k-block, tcgen05.commit frees the stage
// Every product carries the factor 16*16, removed exactly by an arithmetic shift in
// the epilogue (|acc| <= 64*K*256 < 2^31 for K <= 131072).  Both operands use the
// same even/odd nibble order inside a 32-bit word, so the permutation of k inside a
// word cancels in the dot product.
//
// Every mbarrier wait is bounded by a cycle limit; on expiry the CTA raises the
// abort flag, the other roles leave their loops, TMEM is released and the device
// status word records the failure (read with sr_device_status()).
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include <cuda.h>

namespace sr {
namespace tc {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;              // k elements per block = 64 packed bytes = 128 int8 bytes
constexpr int PK_ROW = BK / 2;       // 64
constexpr int SP = 4;                // packed ring depth
constexpr int SU = 2;                // unpacked ring depth
constexpr int PK_A = BM * PK_ROW;    // 8 KB
constexpr int PK_B = BN * PK_ROW;    // 16 KB
constexpr int UN_A = BM * BK;        // 16 KB
constexpr int UN_B = BN * BK;        // 32 KB
constexpr int NUM_UNPACK = 128;
constexpr int THREADS = 192;
constexpr long long WAIT_BUDGET = 1500000000ll;  // cycles (~0.8 s) before a wait gives up

struct Smem {
    // offsets from a 1024-byte aligned base
    static constexpr int un_a = 0;
    static constexpr int un_b = un_a + SU * UN_A;
    static constexpr int pk_a = un_b + SU * UN_B;
    static constexpr int pk_b = pk_a + SP * PK_A;
    static constexpr int bars = pk_b + SP * PK_B;
    static constexpr int total = bars + 256;
};
constexpr int SMEM_BYTES = Smem::total + 1024;  // slack for the manual 1024-byte alignment

__device__ int g_status;  // 0 = ok; otherwise code of the first failed wait

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Bounded wait.  Returns false when the limit was reached or another role aborted.
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

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    // K-major operand, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;             // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset
    d |= (uint64_t)1 << 46;             // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;             // SWIZZLE_128B
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

template <bool A_UNSIGNED>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, uint32_t M,
               uint32_t N, uint32_t K, Epilogue ep) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + Smem::bars;
    // barrier slots (8 bytes each)
    auto pk_full = [&](int s) { return bars + 8u * s; };
    auto pk_empty = [&](int s) { return bars + 8u * (SP + s); };
    auto un_full = [&](int s) { return bars + 8u * (2 * SP + s); };
    auto un_empty = [&](int s) { return bars + 8u * (2 * SP + SU + s); };
    const uint32_t acc_full = bars + 8u * (2 * SP + 2 * SU);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool small = (A_UNSIGNED ? 120u : 64u) * (uint64_t)K < (1u << 22);
    const uint32_t n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const uint32_t num_kb = (K + BK - 1) / BK;

    if (tid == 0) {
        abort_flag = g_status;  // a failed launch earlier in the stream short-circuits the rest
        for (int s = 0; s < SP; ++s) {
            mbar_init(pk_full(s), 1);
            mbar_init(pk_empty(s), NUM_UNPACK);
        }
        for (int s = 0; s < SU; ++s) {
            mbar_init(un_full(s), NUM_UNPACK);
            mbar_init(un_empty(s), 1);
        }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)BN)
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
            // ------------------------------------------------ TMA producer
            if (lane == 0) {
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    const int s = kb % SP;
                    const uint32_t ph = (kb / SP) & 1;
                    if (!mbar_wait(pk_empty(s), ph ^ 1, ab, 11)) break;
                    mbar_expect_tx(pk_full(s), PK_A + PK_B);
                    tma_load_2d(base + Smem::pk_a + s * PK_A, &map_a, (int)(kb * PK_ROW), (int)m0, pk_full(s));
                    tma_load_2d(base + Smem::pk_b + s * PK_B, &map_b, (int)(kb * PK_ROW), (int)n0, pk_full(s));
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------ MMA issuer
            if (lane == 0) {
                const uint32_t idesc = (2u << 4) | ((A_UNSIGNED ? 0u : 1u) << 7) | (1u << 10) |
                                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
                bool ok = true;
                for (uint32_t kb = 0; kb < num_kb && ok; ++kb) {
                    const int u = kb % SU;
                    const uint32_t ph = (kb / SU) & 1;
                    ok = mbar_wait(un_full(u), ph, ab, 12);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = make_desc(base + Smem::un_a + u * UN_A);
                    const uint64_t db = make_desc(base + Smem::un_b + u * UN_B);
#pragma unroll
                    for (int kk = 0; kk < BK / 32; ++kk)
                        mma_i8(tmem_acc, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc,
                               (kb > 0 || kk > 0) ? 1u : 0u);
                    mma_commit(un_empty(u));
                }
                if (ok) mma_commit(acc_full);
            }
        } else {
            // ------------------------------------------------ unpack, then epilogue
            const int t = tid - 64;  // 0..127
            bool ok = true;
            for (uint32_t kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % SP, u = kb % SU;
                const uint32_t php = (kb / SP) & 1, phu = (kb / SU) & 1;
                ok = mbar_wait(pk_full(s), php, ab, 13);
                if (!ok) break;
                ok = mbar_wait(un_empty(u), phu ^ 1, ab, 14);
                if (!ok) break;
                const uint8_t *pa = base_ptr + Smem::pk_a + s * PK_A;
                const uint8_t *pb = base_ptr + Smem::pk_b + s * PK_B;
                uint8_t *ua = base_ptr + Smem::un_a + u * UN_A;
                uint8_t *ub = base_ptr + Smem::un_b + u * UN_B;
#pragma unroll
                for (int i = 0; i < (BM + BN) * 4 / NUM_UNPACK; ++i) {
                    const int id = i * NUM_UNPACK + t;
                    const bool is_a = id < BM * 4;
                    const int cid = is_a ? id : id - BM * 4;
                    const uint4 pk = *reinterpret_cast<const uint4 *>((is_a ? pa : pb) + cid * 16);
                    const int r = cid >> 2, qd = cid & 3;
                    uint4 e, o;
                    e.x = (pk.x << 4) & 0xF0F0F0F0u; o.x = pk.x & 0xF0F0F0F0u;
                    e.y = (pk.y << 4) & 0xF0F0F0F0u; o.y = pk.y & 0xF0F0F0F0u;
                    e.z = (pk.z << 4) & 0xF0F0F0F0u; o.z = pk.z & 0xF0F0F0F0u;
                    e.w = (pk.w << 4) & 0xF0F0F0F0u; o.w = pk.w & 0xF0F0F0F0u;
                    uint8_t *rowp = (is_a ? ua : ub) + (r >> 3) * 1024 + (r & 7) * 128;
                    *reinterpret_cast<uint4 *>(rowp + (((2 * qd) ^ (r & 7)) << 4)) = e;
                    *reinterpret_cast<uint4 *>(rowp + (((2 * qd + 1) ^ (r & 7)) << 4)) = o;
                }
                // generic-proxy writes must be visible to the tensor core (async proxy)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(un_full(u));
                mbar_arrive(pk_empty(s));
            }
            if (ok) ok = mbar_wait(acc_full, 0, ab, 15);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t quarter = warp & 3;  // TMEM lanes this warp may read
                const uint32_t row = m0 + quarter * 32 + lane;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    int v[32];
                    tmem_ld32(tmem_acc + ((quarter * 32u) << 16) + (uint32_t)(c * 32), v);
                    store_acc_chunk(ep, row, n0 + c * 32, v, M, N, small);
                }
            }
        }
    }

    // ---------------------------------------------------- teardown
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*ab != 0 && tid == 0) {
        // give copies and MMAs that are still in flight time to land before the CTA's
        // shared memory and TMEM go away
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) {
        }
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)BN) : "memory");
    }
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D uint8 view [rows][row_bytes] of a packed operand, box = 64 bytes x box_rows rows.
static int make_map(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    SR_REQUIRE(fn != nullptr, SR_ERR_CUDA, "matmul: cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)PK_ROW, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SR_REQUIRE(r == CUDA_SUCCESS, SR_ERR_CUDA, "matmul: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return SR_OK;
}

}  // namespace tc

int launch_gemm_tc(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                   const Epilogue &ep, cudaStream_t st) {
    using namespace tc;
    SR_REQUIRE(aligned16(A) && aligned16(B), SR_ERR_INVALID, "matmul: operands must be 16-byte aligned");
    SR_REQUIRE(K % 32 == 0, SR_ERR_INVALID, "matmul: K = %lld must be a multiple of 32", (long long)K);
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, (uint64_t)M, (uint64_t)K / 2, BM);
    if (rc) return rc;
    rc = make_map(&mb, B, (uint64_t)N, (uint64_t)K / 2, BN);
    if (rc) return rc;
    dim3 grid((unsigned)cdiv<int64_t>(N, BN), (unsigned)cdiv<int64_t>(M, BM));
    auto kfn = a_unsigned ? gemm_tc_kernel<true> : gemm_tc_kernel<false>;
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "matmul: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    kfn<<<grid, THREADS, SMEM_BYTES, st>>>(ma, mb, (uint32_t)M, (uint32_t)N, (uint32_t)K, ep);
    return check_launch("gemm_tc");
}

int tc_device_status(int *out, bool clear) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, tc::g_status, sizeof(int));
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
    if (clear && v != 0) {
        const int z = 0;
        cudaMemcpyToSymbol(tc::g_status, &z, sizeof(int));
    }
    *out = v;
    return SR_OK;
}

}  // namespace sr
