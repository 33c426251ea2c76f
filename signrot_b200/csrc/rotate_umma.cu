// Fused online rotation + sign + per-token symmetric int4 quantization for rows of 4096 values, with the
// first seven of the twelve Walsh-Hadamard stages on the 5th-generation tensor cores (tcgen05) and the
// rows staged by TMA.
//
// One launch replaces fast_hadamard_transform + sign multiply + sym_quant_dynamic
// (signrot/functional/hadamard.py:81, signrot/nn/hadamard.py:39, signrot/kernels/fused.cu:68-112) and
// touches HBM once: 2 bytes in and 0.5 bytes out per value.
//
// A row is the 128 x 32 matrix X[h][l] (element 32 h + l) and H4096 = H128 (x) H32:
//   stage A  D = (H128 / 64) X on the tensor core: tcgen05.mma kind::f16, M = 128, N = 32, K = 128.
//            A = H128 / 64 is a constant K-major tile in shared memory (+-2^-6 is exact in fp16 and bf16, so
//            every product is exact and the sums are fp32); B is the row itself, exactly as TMA lays it down
//            (128 lines of 64 bytes, N-major, 64-byte swizzle); D lives in tensor memory, lane = output line.
//   stage B  tcgen05.ld hands every thread of four epilogue warps one output line: 32 consecutive values.  The
//            remaining five stages are butterflies between the thread's own registers (packed fp32 adds),
//            which is the arithmetic of the reference's fp32 transform with nothing split or re-rounded.
// The values are then rounded once to fp16 (the dtype the reference's transform returns); sign, row maximum
// and the code decision run on packed fp16 pairs, bit-compatible with the reference's quantizer: scale
// rn_h(amax / 7), quotient rn_h(x * rcp(scale)), round half to even, clamp.  A thread's 32 codes are the 16
// consecutive bytes of its line: one 16-byte store, 512 contiguous bytes per warp.
//
// Roles of the one CTA per SM (persistent over a contiguous range of rows): warp 0 issues the TMA loads into a
// ring of row slots, warp 1 issues the MMAs into a ring of eight 32-column accumulators, sixteen epilogue warps
// in four groups take rows round-robin.  Every mbarrier wait is bounded (status word, normal return).
#include "umma.cuh"
#include <type_traits>

namespace sr {

namespace um {

using namespace umma;

constexpr int N = 4096, LINES = 128, LW = 32;
constexpr int SLOT_BYTES = LINES * LW * 2;          // 8192: one row
constexpr int BATCH = 4;                             // rows per MMA set: B is four row tiles side by side, N = 128
constexpr int NBATCH = 3, SLOTS = NBATCH * BATCH;    // row batches in flight from HBM
constexpr int NACC = 2, ACC_COLS = 32, TMEM_COLS = NACC * BATCH * ACC_COLS;   // two accumulator batches of 128 columns
constexpr int GROUPS = BATCH;                        // epilogue groups of four warps: group g takes row g of every batch
constexpr int THREADS = (2 + 4 * GROUPS) * 32;       // 576
constexpr int A_BYTES = 128 * 128 * 2;               // H128 / 64, two K panels of 128 rows x 128 bytes
// shared memory: row slots first (a descriptor never reaches past the allocation), then A, barriers, exchange
constexpr int OFF_SLOTS = 0, OFF_A = SLOTS * SLOT_BYTES, OFF_BARS = OFF_A + A_BYTES;
constexpr int NUM_BARS = 2 * NBATCH + 2 * NACC + GROUPS;
constexpr int OFF_EXCH = OFF_BARS + NUM_BARS * 8;
constexpr int SMEM_BYTES = OFF_EXCH + 2 * GROUPS * 4 * 4 + 1024;   // + slack for the 1024-byte alignment
constexpr long long WAIT_BUDGET = 1500000000ll;

__device__ int g_status;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    return mbar_wait_bounded(bar, parity, abort_flag, code, WAIT_BUDGET, &g_status);
}
// shared-memory matrix descriptors (16-byte units; bit 46: descriptor version of this architecture)
// A: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_a(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// B: N-major, 64-byte swizzle: 32 values (64 bytes) of N contiguous per K line, groups of eight K lines 512 bytes
// apart (stride offset); one 64-byte block along N, so the leading offset (next block along N) is never used
__device__ __forceinline__ uint64_t desc_b(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(SLOT_BYTES >> 4) << 16) | ((uint64_t)(512 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)4 << 61);
}
template <bool BF16>
__global__ void __launch_bounds__(THREADS, 1)
rotate_quant_4096_umma_kernel(const __grid_constant__ CUtensorMap map_x, const int8_t *__restrict__ sign, uint32_t rows,
                              float clip, uint8_t *__restrict__ q, __half *__restrict__ q_scale,
                              __half *__restrict__ rotated) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + OFF_BARS;
    auto slot_full = [&](int s) { return bars + 8u * s; };                          // per row batch
    auto slot_empty = [&](int s) { return bars + 8u * (NBATCH + s); };
    auto acc_full = [&](int a) { return bars + 8u * (2 * NBATCH + a); };            // per accumulator batch
    auto acc_empty = [&](int a) { return bars + 8u * (2 * NBATCH + NACC + a); };
    auto amax_bar = [&](int g) { return bars + 8u * (2 * NBATCH + 2 * NACC + g); }; // the four warps of a group meet here
    float *exch = reinterpret_cast<float *>(base_ptr + OFF_EXCH);        // [parity][group][warp of the group]: its part of amax

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_trigger();   // launched with programmatic serialization: everything up to pdl_wait touches constants only

    // rows of this CTA: an even split, the first (rows % grid) CTAs take one more
    const uint32_t base_cnt = rows / gridDim.x, rem = rows % gridDim.x;
    const uint32_t row_begin = blockIdx.x * base_cnt + min(blockIdx.x, rem);
    const uint32_t cnt = base_cnt + (blockIdx.x < rem ? 1u : 0u);

    // ---- set-up: barriers, tensor memory, the constant A tile H128 / 64 (K-major, 128-byte swizzle, two K panels)
    if (tid == 0) {
        abort_flag = g_status;
        for (int s = 0; s < NBATCH; ++s) {
            mbar_init(slot_full(s), 1);
            mbar_init(slot_empty(s), 1);
        }
        for (int a = 0; a < NACC; ++a) {
            mbar_init(acc_full(a), 1);
            mbar_init(acc_empty(a), 4 * GROUPS);       // every epilogue warp, whether or not its group has a row in the batch
        }
        for (int g = 0; g < GROUPS; ++g) mbar_init(amax_bar(g), 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {
        const uint32_t pos = BF16 ? 0x3C80u : 0x2400u;     // 2^-6
        for (int c = tid; c < 2 * 128 * 8; c += THREADS) {
            const int panel = c >> 10, m = (c >> 3) & 127, ch = c & 7;   // 16-byte chunk `ch` of row m: k = 64 panel + 8 ch + e
            uint32_t w[4];
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
                const int k0 = 64 * panel + 8 * ch + 2 * e2;
                const uint32_t lo = pos | ((__popc(m & k0) & 1) ? 0x8000u : 0u);
                const uint32_t hi = pos | ((__popc(m & (k0 + 1)) & 1) ? 0x8000u : 0u);
                w[e2] = lo | (hi << 16);
            }
            uint8_t *dst = base_ptr + OFF_A + panel * 16384 + (m >> 3) * 1024 + (m & 7) * 128 + ((ch ^ (m & 7)) << 4);
            *reinterpret_cast<uint4 *>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads A through the async proxy
    }
    // sign masks of this thread's output line (epilogue warps): pair p holds elements 32 h + 2 p and + 1
    const int quarter = warp & 3;                 // tensor-memory lanes 32 * (warp % 4) .. + 31 belong to this warp
    const int line = quarter * 32 + lane;
    uint32_t sgn[16];
#pragma unroll
    for (int p = 0; p < 16; ++p) sgn[p] = 0;
    if (warp >= 2 && sign != nullptr) {
        const uint4 *sp = reinterpret_cast<const uint4 *>(sign + 32 * line);
        const uint4 s0 = sp[0], s1 = sp[1];
        const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int p = 0; p < 16; ++p) {
            const uint32_t two = sw[p >> 1] >> (16 * (p & 1));          // bytes of elements 2 p and 2 p + 1
            sgn[p] = ((two & 0x80u) ? 0x00008000u : 0u) | ((two & 0x8000u) ? 0x80000000u : 0u);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = tmem_base_slot;
    volatile int *ab = &abort_flag;

    const uint32_t batches = (cnt + BATCH - 1) / BATCH;
    if (*ab == 0) {
        if (warp == 0) {
            // ------------------------------------------------ TMA producer: one barrier per batch of up to four rows
            if (lane == 0) {
                pdl_wait();      // x comes from the kernel before this one
                for (uint32_t b = 0; b < batches; ++b) {
                    const int s = (int)(b % NBATCH);
                    const uint32_t n_rows = min((uint32_t)BATCH, cnt - b * BATCH);
                    if (!mbar_wait(slot_empty(s), ((b / NBATCH) & 1) ^ 1, ab, 51)) break;
                    mbar_expect_tx(slot_full(s), n_rows * SLOT_BYTES);
                    for (uint32_t r = 0; r < n_rows; ++r)
                        tma_load_2d(base + OFF_SLOTS + (s * BATCH + r) * SLOT_BYTES, &map_x, 0,
                                    (int)((row_begin + b * BATCH + r) * LINES), slot_full(s));
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------ MMA issuer: eight instructions per batch
            if (lane == 0) {
                const uint32_t fmt = BF16 ? 1u : 0u;
                const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) |
                                       ((uint32_t)((BATCH * ACC_COLS) >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
                // (D fp32, B N-major, N = 128: the four row tiles of a batch are the four 64-byte blocks along N, one
                // slot apart; M = 128.  A batch with fewer rows multiplies what is left in the unused slots into
                // accumulator columns nobody reads.)
                uint64_t da[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) da[j] = desc_a(base + OFF_A + (j >> 2) * 16384 + (j & 3) * 32);
                for (uint32_t b = 0; b < batches; ++b) {
                    const int s = (int)(b % NBATCH), a = (int)(b % NACC);
                    if (!mbar_wait(slot_full(s), (b / NBATCH) & 1, ab, 52)) break;
                    if (!mbar_wait(acc_empty(a), ((b / NACC) & 1) ^ 1, ab, 53)) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t d_tmem = tmem_acc + (uint32_t)(a * BATCH * ACC_COLS);
                    const uint64_t db = desc_b(base + OFF_SLOTS + s * BATCH * SLOT_BYTES);
#pragma unroll
                    for (int j = 0; j < 8; ++j)     // K = 16 lines (1024 bytes of every row tile) per instruction
                        mma_f16(d_tmem, da[j], db + (uint64_t)(j * (1024 >> 4)), idesc, j > 0 ? 1u : 0u);
                    mma_commit(slot_empty(s));
                    mma_commit(acc_full(a));
                }
            }
        } else {
            // ------------------------------------------------ epilogue: group g takes row g of every batch
            const int grp = (warp - 2) >> 2;
            pdl_wait();          // q / q_scale may still be read by the kernel before this one
            uint32_t it = 0;     // rows this group has taken
            for (uint32_t b = 0; b < batches; ++b) {
                const int a = (int)(b % NACC);
                const uint32_t i = b * BATCH + (uint32_t)grp;
                const uint32_t row = row_begin + i;
                // (the decision to go on is taken by the whole warp: the tensor-memory load below is warp-collective)
                if (!__all_sync(0xffffffffu, mbar_wait(acc_full(a), (b / NACC) & 1, ab, 54))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float d[32];
                if (i < cnt) tmem_ld32(tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((a * BATCH + grp) * ACC_COLS), d);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty(a));
                if (i >= cnt) continue;
                ++it;
                const uint32_t itp = (it - 1) & 1;

                // ---- the five stages over l, between this thread's registers
                u64 v[16];
#pragma unroll
                for (int p = 0; p < 16; ++p) v[p] = pack2(d[2 * p], d[2 * p + 1]);
                fwht_pairs<16, 16>(v);
                // ---- one rounding to fp16, sign, range
                __half2 hv[16], am[16];
#pragma unroll
                for (int p = 0; p < 16; ++p) {
                    float lo, hi;
                    unpack2(v[p], lo, hi);
                    hv[p] = bits_h2(h2_bits(__floats2half2_rn(lo, hi)) ^ sgn[p]);
                    am[p] = __habs2(hv[p]);
                }
#pragma unroll
                for (int w2 = 8; w2 > 0; w2 >>= 1)      // a tree: four dependent steps instead of sixteen
#pragma unroll
                    for (int p = 0; p < w2; ++p) am[p] = __hmax2(am[p], am[p + w2]);
                const __half2 hmaxv = am[0];
                float vmax = warp_max(fmaxf(__low2float(hmaxv), __high2float(hmaxv)));
                // the row's maximum over the four warps of the group: parts through shared memory (double-buffered by the
                // parity of the group's row count), met at a barrier whose wait is bounded like every other wait here
                float *part = exch + (itp * GROUPS + grp) * 4;
                if (lane == 0) {
                    part[quarter] = vmax;
                    mbar_arrive(amax_bar(grp));
                }
                if (!__all_sync(0xffffffffu, mbar_wait(amax_bar(grp), itp, ab, 55))) break;
                vmax = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));

                __half s = __float2half(vmax / 7.f);
                if (clip != 1.f) s = __float2half(__half2float(s) * clip);
                if (quarter == 0 && lane == 0) q_scale[row] = s;
                // a zero scale gives rcp = inf and 0 * inf = NaN, which the reference turns into code 0;
                // a huge finite factor gives the same codes (x != 0 still saturates) without the NaN
                const float rcp = fminf(rcp_approx_ftz(__half2float(s)), 3.0e38f);
                const u64 rcp2 = pack2(rcp, rcp);
                // scale = rn_h(amax / 7) of a normal fp16 amax keeps every |quotient| below 7.5: nothing to clamp
                const bool clamp = clip != 1.f || __half2float(s) < 6.2e-5f;
                const __half2 lo_c = __floats2half2_rn(-8.f, -8.f), hi_c = __floats2half2_rn(7.f, 7.f);
                const __half2 mg = __floats2half2_rn(1544.f, 1544.f);

                if (rotated != nullptr) {
                    uint4 *orow = reinterpret_cast<uint4 *>(rotated + (size_t)row * N + 32 * line);
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4)
                        orow[c4] = make_uint4(h2_bits(hv[4 * c4]), h2_bits(hv[4 * c4 + 1]), h2_bits(hv[4 * c4 + 2]),
                                              h2_bits(hv[4 * c4 + 3]));
                }
                // ---- codes.  After the fp16 addition of the rounding constant (sum in [1536, 1552)) the low byte of
                // each half is the code + 8; four pairs are merged into one word of four bytes by byte permutes.
                uint32_t w[4];
                auto emit = [&](auto clamp_tag) {
                    constexpr bool CLAMP = decltype(clamp_tag)::value;
#pragma unroll
                    for (int part = 0; part < 4; ++part) {
                        uint32_t bits[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float2 f = __half22float2(hv[part * 4 + k]);
                            float lo, hi;
                            unpack2(mul2(pack2(f.x, f.y), rcp2), lo, hi);
                            __half2 qh = __floats2half2_rn(lo, hi);      // rn_h(x * rcp): the quotient __hdiv returns
                            if (CLAMP) qh = __hmin2(__hmax2(qh, lo_c), hi_c);
                            bits[k] = h2_bits(__hadd2(qh, mg));
                        }
                        // x = [l0, l1, h0, h1] of two pairs, then the low values and the high values of all four
                        const uint32_t x01 = __byte_perm(bits[0], bits[1], 0x6240), x23 = __byte_perm(bits[2], bits[3], 0x6240);
                        const uint32_t ev = __byte_perm(x01, x23, 0x5410), od = __byte_perm(x01, x23, 0x7632);
                        w[part] = (ev + (od << 4)) ^ 0x88888888u;       // offset-8 codes -> two's complement nibbles
                    }
                };
                if (clamp) emit(std::true_type{});
                else emit(std::false_type{});
                *reinterpret_cast<uint4 *>(q + (size_t)row * (N / 2) + 16 * line) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }

    // ---------------------------------------------------- teardown
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*ab != 0 && tid == 0) {          // a role gave up: let copies that are still in flight land before the CTA goes
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000ll) {
        }
    }
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)TMEM_COLS) : "memory");
}

}  // namespace um

int launch_rotate_umma4096(const RotateArgs &a, cudaStream_t st) {
    using namespace um;
    const bool shape_ok = a.n == 4096 && a.K == 1 && a.stride == 1 && a.S == 4096 && a.q != nullptr && !a.fp32_mode && !a.asym &&
                          (a.in_dtype == SR_F16 || (a.in_dtype == SR_BF16 && a.cast_in_to_f16)) &&
                          a.expert_ids == nullptr && a.scale == 1.f / 64.f && aligned16(a.x) && aligned16(a.q) &&
                          (a.sign == nullptr || aligned16(a.sign)) &&
                          (a.out == nullptr || (a.out_dtype == SR_F16 && aligned16(a.out)));
    if (!shape_ok || a.rows >= (1u << 23)) return SR_ERR_UNSUPPORTED;
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return SR_ERR_UNSUPPORTED;      // the mma.sync kernel takes the call
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)LW, (cuuint64_t)a.rows * LINES};
    const cuuint64_t strides[1] = {(cuuint64_t)LW * 2};
    const cuuint32_t box[2] = {(cuuint32_t)LW, (cuuint32_t)LINES};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&map, a.in_dtype == SR_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                    const_cast<void *>(a.x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SR_REQUIRE(r == CUDA_SUCCESS, SR_ERR_CUDA, "rotate_quant: cuTensorMapEncodeTiled failed with code %d", (int)r);
    const int sm_count = current_sm_count();
    const uint32_t grid = a.rows < (uint32_t)sm_count ? a.rows : (uint32_t)sm_count;
#define SR_RU(BF)                                                                                                \
    do {                                                                                                         \
        auto kfn = rotate_quant_4096_umma_kernel<BF>;                                                            \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES); \
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "rotate_quant: %s", cudaGetErrorString(e));               \
        launch_pdl(kfn, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, st, map, a.sign, a.rows, a.clip, a.q,     \
                   a.q_scale, (__half *)a.out);                                                                  \
    } while (0)
    if (a.in_dtype == SR_BF16) SR_RU(true);
    else SR_RU(false);
#undef SR_RU
    return check_launch("rotate_quant_4096_umma");
}

int rotate_umma_device_status(int *out, bool clear) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, um::g_status, sizeof(int));
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
    if (clear && v != 0) {
        const int z = 0;
        cudaMemcpyToSymbol(um::g_status, &z, sizeof(int));
    }
    *out = v;
    return SR_OK;
}

}  // namespace sr
