// Fused online rotation + sign + per-token symmetric int4 quantization for rows of 14336 = 28 x 512 values
// (the down_proj input of an 8B model), y = (had28 (x) H_512) x / sqrt(n), with both matrix stages on the
// 5th-generation tensor cores (tcgen05) and the rows staged by TMA.
//
// One launch replaces fast_hadamard_transform over the 28 segments, the fp16 had28 matmul, the sign multiply
// and sym_quant_dynamic (signrot/functional/hadamard.py:78-87, signrot/nn/hadamard.py:39,
// signrot/kernels/fused.cu:68-112) and touches HBM once.  The rounding points are the reference's: the
// 512-point sums are fp32, scaled and rounded to fp16; the 28-point stage multiplies fp16 values by +-1 and
// accumulates in fp32 (what an fp16 tensor-core matmul does), rounded to fp16 again.
//
// A row is 448 lines of 32 values; line 16 k + h of the row is X[k][h][.] of segment k, and H_512 = H16 (x) H32.
// One tcgen05.mma instruction costs about the same time for any N up to 128-256, so every instruction is made as
// wide as tensor memory allows:
//   stage A   D1 = (I8 (x) H16 / 8) X on SUPER TILES of four tiles of 128 lines side by side (kind::f16, M = 128,
//             N = 128, K = 128: eight instructions per row).  A super tile is ONE row: the TMA map is three-
//             dimensional (row, line, value), the fourth tile's last 64 lines lie past the row's 448 and are filled with
//             zeros, so no tile ever holds lines of two rows and rows stay independent (the zeros of the block-diagonal
//             constant would otherwise turn one row's NaN or infinity into its neighbour's: 0 x inf).
//   stage B   eight warps read D1 (one line per thread), finish the 512-point transform with five butterfly stages
//             between registers, scale, round to fp16 and store Z[k][j] (j = 32 h' + l') into shared memory: K line =
//             segment, 128-byte swizzle, blocks of 64 j.  A warp's 32 lines are two whole segments of ONE row
//             (448 = 14 x 32), so a row's Z is complete after 14 warp arrivals.
//   stage C   D2[(c, k')][j] = sum_k had28[k'][k] Z[k][j] with Z as the N-major B operand (N = 128 columns j per
//             instruction, K = 32 with the zero padding of 28 -> 32) and A = had28 repeated in all four lane quarters
//             of tensor memory, so that every warp finds the 28 output lines in the quarter it may read.
//   stage D   sixteen warps per row, four per chunk of 128 columns: thread k' of a warp holds y[k'][j0 .. j0 + 31],
//             rounds to fp16, applies the sign, takes the row maximum (one bounded barrier across the sixteen warps),
//             quantizes exactly as the reference does (scale rn_h(amax / 7), quotient rn_h(x * rcp(scale)), round half
//             to even, clamp) and stores its 32 codes as 16 consecutive bytes.
// Roles of the one CTA per SM: warp 0 TMA producer, warp 1 stage-A MMAs, warp 2 stage-C MMAs, warps 4-11 stage B,
// warps 12-27 stage D.  Every mbarrier wait is bounded (status word, normal return).
#include "umma.cuh"
#include <type_traits>

namespace sr {

namespace h28u {

using namespace umma;

constexpr int N = 14336, KH = 28, LINES_PER_ROW = 448, LW = 32, PORTIONS_PER_ROW = 14;
constexpr int TILE_BYTES = 128 * LW * 2;            // 8192: 128 lines
constexpr int SUPER = 4;                            // tiles per stage-A MMA set (N = 128)
constexpr int XS = 3;                               // super tiles in flight from HBM
constexpr int D1_RING = 2, D2_RING = 2;             // accumulators of 128 columns: two super tiles, two chunks of a row
constexpr int TMEM_COLS = 512, D2_COL0 = D1_RING * 128;
constexpr int A1_BYTES = 128 * 128 * 2;             // I8 (x) H16 / 8: two K panels of 128 rows x 128 bytes
constexpr int Z_BYTES = 8 * 4096;                   // one row of Z: 8 blocks of 64 j, each 32 K lines x 128 bytes
constexpr int A2_BYTES = 128 * 64;                  // had28 padded to 32 x 32 fp16, repeated in the four lane quarters
constexpr int OFF_X = 0, OFF_A1 = XS * SUPER * TILE_BYTES, OFF_Z = OFF_A1 + A1_BYTES, OFF_A2 = OFF_Z + 2 * Z_BYTES;
constexpr int OFF_BARS = OFF_A2 + A2_BYTES;
constexpr int NUM_BARS = 2 * XS + 2 * D1_RING + 2 * 2 + 4 + D2_RING + 2;
constexpr int OFF_EXCH = OFF_BARS + ((NUM_BARS * 8 + 15) / 16) * 16;
constexpr int SMEM_BYTES = OFF_EXCH + 2 * 16 * 4 + 1024;
constexpr int THREADS = 28 * 32;
constexpr long long WAIT_BUDGET = 1500000000ll;

__device__ int g_status;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    return mbar_wait_bounded(bar, parity, abort_flag, code, WAIT_BUDGET, &g_status);
}
// shared-memory matrix descriptors (16-byte units; bit 46: descriptor version of this architecture)
__device__ __forceinline__ uint64_t desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)swizzle << 61);
}
constexpr uint32_t SW128 = 2, SW64 = 4;

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 1)
rotate_quant_had28_umma_kernel(const __grid_constant__ CUtensorMap map_x, const __half *__restrict__ hadk,
                               const int8_t *__restrict__ sign, uint32_t rows, float scale, float clip,
                               uint8_t *__restrict__ q, __half *__restrict__ q_scale, __half *__restrict__ rotated) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + OFF_BARS;
    auto x_full = [&](int s) { return bars + 8u * s; };                                   // per super tile slot
    auto x_empty = [&](int s) { return bars + 8u * (XS + s); };
    auto d1_full = [&](int a) { return bars + 8u * (2 * XS + a); };
    auto d1_empty = [&](int a) { return bars + 8u * (2 * XS + D1_RING + a); };
    auto z_full = [&](int z) { return bars + 8u * (2 * XS + 2 * D1_RING + z); };            // per row parity
    auto z_empty = [&](int z) { return bars + 8u * (2 * XS + 2 * D1_RING + 2 + z); };
    // A barrier whose waiters each consume EVERY phase can be tracked by one parity bit; so "full" is one barrier per chunk
    // position of a row (its four warps see every phase), while "empty" is one per accumulator (one waiter: the MMA thread)
    auto d2_full = [&](int c) { return bars + 8u * (2 * XS + 2 * D1_RING + 4 + c); };       // per chunk position 0..3
    auto d2_empty = [&](int b) { return bars + 8u * (2 * XS + 2 * D1_RING + 8 + b); };      // per chunk accumulator
    auto amax_bar = [&](int p) { return bars + 8u * (2 * XS + 2 * D1_RING + 8 + D2_RING + p); };
    float *exch = reinterpret_cast<float *>(base_ptr + OFF_EXCH);       // [parity][stage-D warp]: its part of amax

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_trigger();   // launched with programmatic serialization: everything up to pdl_wait touches constants only

    // rows of this CTA: an even split, the first (rows % grid) CTAs take one more
    const uint32_t base_cnt = rows / gridDim.x, rem = rows % gridDim.x;
    const uint32_t row_begin = blockIdx.x * base_cnt + min(blockIdx.x, rem);
    const uint32_t cnt = base_cnt + (blockIdx.x < rem ? 1u : 0u);
    const uint32_t supers = cnt;                                // one super tile (four tiles of 128 lines) per row: the last
                                                                // 64 lines of the fourth tile lie past the row and arrive as zeros

    // ---- set-up
    if (tid == 0) {
        abort_flag = g_status;
        for (int s = 0; s < XS; ++s) {
            mbar_init(x_full(s), 1);
            mbar_init(x_empty(s), 1);
        }
        for (int a = 0; a < D1_RING; ++a) {
            mbar_init(d1_full(a), 1);
            mbar_init(d1_empty(a), 8);                 // every stage-B warp
        }
        for (int z = 0; z < 2; ++z) {
            mbar_init(z_full(z), PORTIONS_PER_ROW);
            mbar_init(z_empty(z), 1);
            mbar_init(d2_empty(z), 4);                 // the four stage-D warps of the chunk
            mbar_init(amax_bar(z), 16);
        }
        for (int c = 0; c < 4; ++c) mbar_init(d2_full(c), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {
        // A1 = I8 (x) H16 / 8, K-major, 128-byte swizzle, two K panels: entry (m, k) is +-2^-3 when m and k lie in the
        // same block of 16, else 0
        const uint32_t pos = BF16 ? 0x3E00u : 0x3000u;
        for (int c = tid; c < 2 * 128 * 8; c += THREADS) {
            const int panel = c >> 10, m = (c >> 3) & 127, ch = c & 7;
            uint32_t w[4];
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
                const int k0 = 64 * panel + 8 * ch + 2 * e2;
                const bool same = (k0 >> 4) == (m >> 4);
                const uint32_t lo = same ? (pos | ((__popc(m & k0 & 15) & 1) ? 0x8000u : 0u)) : 0u;
                const uint32_t hi = same ? (pos | ((__popc(m & (k0 + 1) & 15) & 1) ? 0x8000u : 0u)) : 0u;
                w[e2] = lo | (hi << 16);
            }
            uint8_t *dst = base_ptr + OFF_A1 + panel * 16384 + (m >> 3) * 1024 + (m & 7) * 128 + ((ch ^ (m & 7)) << 4);
            *reinterpret_cast<uint4 *>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        // A2[m][k] = had28[m % 32][k] as fp16 (zero for m % 32 >= 28 or k >= 28): the 28 output lines once per lane
        // quarter.  K-major, 64-byte swizzle: row m is 64 bytes, its four 16-byte chunks XOR-ed with (m / 2) % 4.
        for (int c = tid; c < 128 * 4; c += THREADS) {
            const int m = c >> 2, ch = c & 3, kp = m & 31;
            __half v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int k = 8 * ch + e;
                v[e] = (kp < KH && k < KH) ? hadk[kp * KH + k] : __float2half(0.f);
            }
            uint8_t *dst = base_ptr + OFF_A2 + m * 64 + ((ch ^ ((m >> 1) & 3)) << 4);
            *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(v);
        }
        // K lines 28..31 of both Z buffers are the zero padding of the 28-point stage (written once)
        for (int c = tid; c < 2 * 8 * 4 * 8; c += THREADS) {
            const int zb = c >> 8, blk = (c >> 5) & 7, k = 28 + ((c >> 3) & 3), ch = c & 7;
            uint8_t *dst = base_ptr + OFF_Z + zb * Z_BYTES + blk * 4096 + (k >> 3) * 1024 + (k & 7) * 128 + (ch << 4);
            *reinterpret_cast<uint4 *>(dst) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads these through the async proxy
    }
    const int quarter = warp & 3;                 // tensor-memory lanes 32 * (warp % 4) .. + 31 belong to this warp
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_slot;
    volatile int *ab = &abort_flag;

    if (*ab == 0) {
        if (warp == 0) {
            // ------------------------------------------------ TMA producer: one super tile (four tiles of 128 lines) per row
            if (lane == 0) {
                pdl_wait();      // x comes from the kernel before this one
                for (uint32_t sp = 0; sp < supers; ++sp) {
                    const int s = (int)(sp % XS);
                    if (!mbar_wait(x_empty(s), ((sp / XS) & 1) ^ 1, ab, 71)) break;
                    mbar_expect_tx(x_full(s), SUPER * TILE_BYTES);     // lines past the row's end arrive as zeros and count
                    for (uint32_t i = 0; i < (uint32_t)SUPER; ++i)
                        tma_load_3d(base + OFF_X + (s * SUPER + i) * TILE_BYTES, &map_x, 0, (int)(i * 128),
                                    (int)(row_begin + sp), x_full(s));
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------ stage-A MMAs: eight instructions per super tile
            if (lane == 0) {
                const uint32_t fmt = BF16 ? 1u : 0u;
                // D fp32, B N-major, N = 128 (the four tiles are the four 64-byte blocks along N, one tile apart), M = 128
                const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(128 >> 3) << 17) |
                                       ((uint32_t)(128 >> 4) << 24);
                uint64_t da[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) da[j] = desc(base + OFF_A1 + (j >> 2) * 16384 + (j & 3) * 32, 16, 1024, SW128);
                for (uint32_t sp = 0; sp < supers; ++sp) {
                    const int s = (int)(sp % XS), a = (int)(sp % D1_RING);
                    if (!mbar_wait(x_full(s), (sp / XS) & 1, ab, 72)) break;
                    if (!mbar_wait(d1_empty(a), ((sp / D1_RING) & 1) ^ 1, ab, 73)) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t db = desc(base + OFF_X + s * SUPER * TILE_BYTES, TILE_BYTES, 512, SW64);
#pragma unroll
                    for (int j = 0; j < 8; ++j)     // K = 16 lines (1024 bytes of every tile) per instruction
                        mma_f16(tmem + (uint32_t)(a * 128), da[j], db + (uint64_t)(j * (1024 >> 4)), idesc, j > 0 ? 1u : 0u);
                    mma_commit(x_empty(s));
                    mma_commit(d1_full(a));
                }
            }
        } else if (warp == 2) {
            // ------------------------------------------------ stage-C MMAs: per row four chunks of 128 columns j, K = 32
            if (lane == 0) {
                // D fp32, A (had28) fp16 K-major, B (Z) fp16 N-major, N = 128, M = 128
                const uint32_t idesc = (1u << 4) | (1u << 16) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
                const uint64_t da0 = desc(base + OFF_A2, 16, 512, SW64), da1 = desc(base + OFF_A2 + 32, 16, 512, SW64);
                for (uint32_t r = 0; r < cnt; ++r) {
                    const int z = (int)(r & 1);
                    if (!mbar_wait(z_full(z), (r >> 1) & 1, ab, 74)) break;
                    const uint32_t zb = base + OFF_Z + z * Z_BYTES;
                    bool ok = true;
                    for (uint32_t c = 0; c < 4 && ok; ++c) {
                        const uint32_t n = 4 * r + c;            // chunk number in the CTA's stream
                        const int b = (int)(n & 1);
                        ok = mbar_wait(d2_empty(b), ((n >> 1) & 1) ^ 1, ab, 75);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        // the chunk is two blocks of 64 j, 4096 bytes apart (leading offset); groups of eight K lines are
                        // 1024 bytes apart (stride offset)
                        const uint64_t dz = desc(zb + c * 8192, 4096, 1024, SW128);
                        const uint32_t d = tmem + (uint32_t)(D2_COL0 + b * 128);
                        mma_f16(d, da0, dz, idesc, 0u);                              // K lines 0..15
                        mma_f16(d, da1, dz + (uint64_t)(2048 >> 4), idesc, 1u);      // K lines 16..31
                        if (c == 3) mma_commit(z_empty(z));
                        mma_commit(d2_full((int)c));
                    }
                    if (!ok) break;
                }
            }
        } else if (warp >= 4 && warp < 12) {
            // ------------------------------------------------ stage B: warp (g, quarter) takes tiles g and g + 2 of every super tile
            const int grp = (warp - 4) >> 2;
            const float sc8 = scale * 8.f;                    // the constant operand of stage A carries 1 / 8
            const u64 scale2 = pack2(sc8, sc8);
            bool alive = true;
            for (uint32_t sp = 0; sp < supers && alive; ++sp) {
                const int a = (int)(sp % D1_RING);
                if (!__all_sync(0xffffffffu, mbar_wait(d1_full(a), (sp / D1_RING) & 1, ab, 76))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    // portion (32 lines = two segments) of row sp that this warp holds in tile grp + 2 i: 14 exist
                    const uint32_t pr = 4u * (uint32_t)(grp + 2 * i) + (uint32_t)quarter;
                    float d[32];
                    if (pr < (uint32_t)PORTIONS_PER_ROW)
                        tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * 128 + (grp + 2 * i) * 32), d);
                    if (i == 1) {            // both of this warp's tiles are in registers (or skipped): release the accumulator
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(d1_empty(a));
                    }
                    if (pr >= (uint32_t)PORTIONS_PER_ROW) continue;  // the zero padding behind the row's 448 lines
                    const uint32_t r = sp;
                    const int z = (int)(r & 1);
                    const int k = (int)(2 * pr) + (lane >> 4), hp = lane & 15;       // segment and line h' of this thread
                    // The Z buffer of row r was last read by the stage-C MMAs of row r - 2.  Every warp has a portion in tile
                    // grp of EVERY row (4 grp + quarter < 14), so it sees every phase of this barrier in order, which is
                    // what makes the parity test valid.
                    if (!__all_sync(0xffffffffu, mbar_wait(z_empty(z), ((r >> 1) & 1) ^ 1, ab, 77))) {
                        alive = false;
                        break;
                    }
                    u64 v[16];
#pragma unroll
                    for (int p = 0; p < 16; ++p) v[p] = pack2(d[2 * p], d[2 * p + 1]);
                    fwht_pairs<16, 16>(v);
                    uint32_t zw[16];
#pragma unroll
                    for (int p = 0; p < 16; ++p) {
                        float lo, hi;
                        unpack2(mul2(v[p], scale2), lo, hi);
                        zw[p] = h2_bits(__floats2half2_rn(lo, hi));      // the reference's first rounding point
                    }
                    // Z[k][32 h' + l']: block of 64 j = h' / 2, 16-byte chunks 4 (h' % 2) + c, K line k, 128-byte swizzle
                    uint8_t *zrow = base_ptr + OFF_Z + z * Z_BYTES + (hp >> 1) * 4096 + (k >> 3) * 1024 + (k & 7) * 128;
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        *reinterpret_cast<uint4 *>(zrow + (((4 * (hp & 1) + c) ^ (k & 7)) << 4)) =
                            make_uint4(zw[4 * c], zw[4 * c + 1], zw[4 * c + 2], zw[4 * c + 3]);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(z_full(z));
                }
            }
        } else if (warp >= 12) {
            // ------------------------------------------------ stage D: warp (chunk, quarter); thread k' = lane holds y[k'][j0 .. j0 + 31]
            const int dw = warp - 12, chunk = dw >> 2;
            const int j0 = 128 * chunk + 32 * quarter;
            const bool real = lane < KH;                          // lanes 28..31 read the zero padding lines
            uint32_t sgn[16];
#pragma unroll
            for (int p = 0; p < 16; ++p) sgn[p] = 0;
            if (real && sign != nullptr) {
                const uint4 *sp4 = reinterpret_cast<const uint4 *>(sign + lane * 512 + j0);
                const uint4 s0 = sp4[0], s1 = sp4[1];
                const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int p = 0; p < 16; ++p) {
                    const uint32_t two = sw[p >> 1] >> (16 * (p & 1));          // bytes of elements 2 p and 2 p + 1
                    sgn[p] = ((two & 0x80u) ? 0x00008000u : 0u) | ((two & 0x8000u) ? 0x80000000u : 0u);
                }
            }
            pdl_wait();          // q / q_scale may still be read by the kernel before this one
            for (uint32_t r = 0; r < cnt; ++r) {
                const int z = (int)(r & 1);
                const uint32_t n = 4 * r + (uint32_t)chunk;        // this warp's chunk number in the CTA's stream
                const int b = (int)(n & 1);
                const uint32_t row = row_begin + r;
                if (!__all_sync(0xffffffffu, mbar_wait(d2_full(chunk), r & 1, ab, 78))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float d[32];
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(D2_COL0 + b * 128 + quarter * 32), d);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(d2_empty(b));
                // ---- second rounding point, sign, range
                __half2 hv[16], am[16];
#pragma unroll
                for (int p = 0; p < 16; ++p) {
                    hv[p] = bits_h2(h2_bits(__floats2half2_rn(d[2 * p], d[2 * p + 1])) ^ sgn[p]);
                    am[p] = __habs2(hv[p]);
                }
#pragma unroll
                for (int w2 = 8; w2 > 0; w2 >>= 1)
#pragma unroll
                    for (int p = 0; p < w2; ++p) am[p] = __hmax2(am[p], am[p + w2]);
                float vmax = warp_max(fmaxf(__low2float(am[0]), __high2float(am[0])));
                float *part = exch + z * 16;
                if (lane == 0) {
                    part[dw] = vmax;
                    mbar_arrive(amax_bar(z));
                }
                if (!__all_sync(0xffffffffu, mbar_wait(amax_bar(z), (r >> 1) & 1, ab, 79))) break;
                {
                    const float4 p0 = *reinterpret_cast<const float4 *>(part), p1 = *reinterpret_cast<const float4 *>(part + 4);
                    const float4 p2 = *reinterpret_cast<const float4 *>(part + 8), p3 = *reinterpret_cast<const float4 *>(part + 12);
                    vmax = fmaxf(fmaxf(fmaxf(fmaxf(p0.x, p0.y), fmaxf(p0.z, p0.w)), fmaxf(fmaxf(p1.x, p1.y), fmaxf(p1.z, p1.w))),
                                 fmaxf(fmaxf(fmaxf(p2.x, p2.y), fmaxf(p2.z, p2.w)), fmaxf(fmaxf(p3.x, p3.y), fmaxf(p3.z, p3.w))));
                }
                __half s = __float2half(vmax / 7.f);
                if (clip != 1.f) s = __float2half(__half2float(s) * clip);
                if (dw == 0 && lane == 0) q_scale[row] = s;
                // a zero scale gives rcp = inf and 0 * inf = NaN, which the reference turns into code 0;
                // a huge finite factor gives the same codes (x != 0 still saturates) without the NaN
                const float rcp = fminf(rcp_approx_ftz(__half2float(s)), 3.0e38f);
                const u64 rcp2 = pack2(rcp, rcp);
                // scale = rn_h(amax / 7) of a normal fp16 amax keeps every |quotient| below 7.5: nothing to clamp
                const bool clamp = clip != 1.f || __half2float(s) < 6.2e-5f;
                const __half2 lo_c = __floats2half2_rn(-8.f, -8.f), hi_c = __floats2half2_rn(7.f, 7.f);
                const __half2 mg = __floats2half2_rn(1544.f, 1544.f);
                if (rotated != nullptr && real) {
                    uint4 *orow = reinterpret_cast<uint4 *>(rotated + (size_t)row * N + lane * 512 + j0);
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4)
                        orow[c4] = make_uint4(h2_bits(hv[4 * c4]), h2_bits(hv[4 * c4 + 1]), h2_bits(hv[4 * c4 + 2]),
                                              h2_bits(hv[4 * c4 + 3]));
                }
                // ---- codes.  After the fp16 addition of the rounding constant (sum in [1536, 1552)) the low byte of each half
                // is the code + 8; four pairs are merged into one word of four bytes by byte permutes.
                uint32_t w[4];
                auto emit = [&](auto clamp_tag) {
                    constexpr bool CLAMP = decltype(clamp_tag)::value;
#pragma unroll
                    for (int part4 = 0; part4 < 4; ++part4) {
                        uint32_t bits[4];
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const float2 f = __half22float2(hv[part4 * 4 + kk]);
                            float lo, hi;
                            unpack2(mul2(pack2(f.x, f.y), rcp2), lo, hi);
                            __half2 qh = __floats2half2_rn(lo, hi);      // rn_h(x * rcp): the quotient __hdiv returns
                            if (CLAMP) qh = __hmin2(__hmax2(qh, lo_c), hi_c);
                            bits[kk] = h2_bits(__hadd2(qh, mg));
                        }
                        // x = [l0, l1, h0, h1] of two pairs, then the low values and the high values of all four
                        const uint32_t x01 = __byte_perm(bits[0], bits[1], 0x6240), x23 = __byte_perm(bits[2], bits[3], 0x6240);
                        const uint32_t ev = __byte_perm(x01, x23, 0x5410), od = __byte_perm(x01, x23, 0x7632);
                        w[part4] = (ev + (od << 4)) ^ 0x88888888u;       // offset-8 codes -> two's complement nibbles
                    }
                };
                if (clamp) emit(std::true_type{});
                else emit(std::false_type{});
                if (real)
                    *reinterpret_cast<uint4 *>(q + (size_t)row * (N / 2) + lane * 256 + (j0 >> 1)) = make_uint4(w[0], w[1], w[2], w[3]);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
}

}  // namespace h28u

int launch_rotate_had28_umma(const RotateArgs &a, cudaStream_t st) {
    using namespace h28u;
    const bool ok = a.n == (uint32_t)N && a.K == (uint32_t)KH && a.stride == 1 && a.q != nullptr && !a.fp32_mode && !a.asym &&
                    a.expert_ids == nullptr && a.hadk != nullptr &&
                    (a.in_dtype == SR_F16 || (a.in_dtype == SR_BF16 && a.cast_in_to_f16)) && aligned16(a.x) && aligned16(a.q) &&
                    (a.sign == nullptr || aligned16(a.sign)) && (a.out == nullptr || (a.out_dtype == SR_F16 && aligned16(a.out))) &&
                    a.rows < (1u << 22);
    if (!ok) return SR_ERR_UNSUPPORTED;
    umma::EncodeTiledFn fn = umma::encode_fn();
    if (fn == nullptr) return SR_ERR_UNSUPPORTED;      // the mma.sync kernel takes the call
    CUtensorMap map;
    // [row][448 lines][32 values]: a box of 128 lines never leaves its row; what lies past line 447 is filled with zeros
    const cuuint64_t dims[3] = {(cuuint64_t)LW, (cuuint64_t)LINES_PER_ROW, (cuuint64_t)a.rows};
    const cuuint64_t strides[2] = {(cuuint64_t)LW * 2, (cuuint64_t)N * 2};
    const cuuint32_t box[3] = {(cuuint32_t)LW, 128, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(&map, a.in_dtype == SR_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                    const_cast<void *>(a.x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SR_REQUIRE(r == CUDA_SUCCESS, SR_ERR_CUDA, "rotate_quant: cuTensorMapEncodeTiled failed with code %d", (int)r);
    const int sm_count = current_sm_count();
    const uint32_t grid = a.rows < (uint32_t)sm_count ? a.rows : (uint32_t)sm_count;
#define SR_RH(BF)                                                                                                \
    do {                                                                                                         \
        auto kfn = rotate_quant_had28_umma_kernel<BF>;                                                           \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES); \
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "rotate_quant: %s", cudaGetErrorString(e));               \
        launch_pdl(kfn, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, st, map, (const __half *)a.hadk, a.sign, a.rows, \
                   a.scale, a.clip, a.q, a.q_scale, (__half *)a.out);                                            \
    } while (0)
    if (a.in_dtype == SR_BF16) SR_RH(true);
    else SR_RH(false);
#undef SR_RH
    return check_launch("rotate_quant_had28_umma");
}

int rotate_had28_umma_device_status(int *out, bool clear) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, h28u::g_status, sizeof(int));
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
    if (clear && v != 0) {
        const int z = 0;
        cudaMemcpyToSymbol(h28u::g_status, &z, sizeof(int));
    }
    *out = v;
    return SR_OK;
}

}  // namespace sr
