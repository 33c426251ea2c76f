// W4A4 GEMM on tcgen05 with CTA pairs (cta_group::2): one 256 x 256 output tile per pair.
//
// Same contract as the other GEMM kernels (C = A * B^T on packed 4-bit operands, exact int32
// accumulation in TMEM, optional fused dequant epilogue); replaces signrot/kernels/gemm.cu:7-85
// and the dequant pass signrot/kernels/quant.cu:66-131.
//
// Why pairs: the kernel is bound by the SM's shared-memory data path (packed-tile fill, unpack
// read, int8 write, tensor-core operand read).  With two CTAs on one 256 x 256 tile each CTA
// unpacks 128 rows of A and only 128 of the 256 rows of B, and its tensor core reads half of B
// from the partner's shared memory: per k-block and SM the traffic drops from 144 KB (one CTA,
// 128 x 256 tile) to 96 KB for the same 128 x 256 x 128 MACs.
//
// Per CTA (448 threads), persistent over tiles (tile = cluster + i * clusters, n fastest):
//   warp 0      TMA producer (no multicast): its 128 rows of packed A and its 128 rows of packed B
//   warp 1      TMEM allocation (both CTAs, cta_group::2); in the leader CTA (cluster rank 0) one
//               lane issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 32) for the pair and
//               commits to both CTAs' barriers (tcgen05.commit ... multicast::cluster)
//   warps 2..5  epilogue of the CTA's own 128 accumulator rows (two TMEM buffers of 256 columns,
//               so the next tile's MMAs overlap the epilogue)
//   warps 6..13 unpack: packed nibble n -> int8 byte 16*n in the 128-byte-swizzled K-major layout
// Cross-CTA signalling uses mbarrier arrives on the leader's barriers through mapa addresses.
// Every wait is bounded by a cycle limit; on expiry the CTA aborts, both CTAs fall through to
// the cluster barrier at the end, TMEM is released and the device status word records the code.
//
// Split K (dense launches with a caller-provided workspace, problems with so few tiles that at least half of the
// CTA pairs would idle and K is long, e.g. M = 256, K = 14336, N = 4096: 16 tiles for 74 pairs): an item is (tile, k-range),
// S = 2 or 4 ranges per tile, tiles * S <= pairs, so every item of the launch is resident at the same time.  A
// pair's epilogue warps write their int32 accumulator to the workspace, count themselves in, wait (bounded) for the
// other ranges of the tile, and then each range sums and finishes 1 / S of the tile's columns: integer addition,
// so the result is the bit pattern of the unsplit product.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include <cuda.h>
#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace sr {
namespace tc3 {

constexpr int BMC = 128;             // rows of A per CTA (tile M = 256 per pair)
constexpr int BNC = 128;             // rows of B per CTA (tile N = 256 per pair)
constexpr int BN = 256;
constexpr int BK = 128;
constexpr int PK_ROW = BK / 2;       // 64 packed bytes per row and k-block
constexpr int MAX_STAGES = 8;        // ring depths are launch parameters (packed ring sp, int8 ring su)
constexpr int PK_A = BMC * PK_ROW;   // 8 KB
constexpr int PK_B = BNC * PK_ROW;   // 8 KB
constexpr int UN_A = BMC * BK;       // 16 KB
constexpr int UN_B = BNC * BK;       // 16 KB
constexpr int UNPACK_WARPS = 8;
constexpr int NUM_UNPACK = UNPACK_WARPS * 32;
constexpr int THREADS = 64 + 128 + NUM_UNPACK;  // 448
constexpr long long WAIT_BUDGET = 1500000000ll;

constexpr int BAR_BYTES = 512;
constexpr int MAX_EXPERTS = 512;                    // grouped launches: first m-tile of every expert, in shared memory
constexpr int SCHED_BYTES = (MAX_EXPERTS + 4) * 4;
constexpr int EPI_STAGE_BYTES = 4 * 2560;           // one 32 x 80-byte output staging area per epilogue warp
constexpr int SPLIT_COUNTERS = 1024;                // int32 words of the split-K counters: two banks (S = 2, 4)
constexpr int MAX_SMEM = 226 * 1024;   // dynamic part; the kernel also has a few static words
__host__ __device__ constexpr int smem_bytes(int sp, int su) {
    return su * (UN_A + UN_B) + sp * (PK_A + PK_B) + BAR_BYTES + SCHED_BYTES + EPI_STAGE_BYTES + 1024;
}

// position in a ring of `depth` stages and the parity of the current pass over it
struct Ring {
    int s = 0;
    uint32_t ph = 0;
    __device__ __forceinline__ void next(int depth) {
        if (++s == depth) {
            s = 0;
            ph ^= 1;
        }
    }
};

__device__ int g_status;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive on the barrier at the same offset in CTA `cta` of the cluster.  CTA-scope release (the default) is
// what is needed: the data this signal publishes (an unpacked stage, a drained accumulator) is consumed by this
// SM's own tensor core and TMEM, only the signal crosses to the partner.  A cluster-scope release stalls the
// arriving warp for several hundred cycles per k-block.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta) {
    asm volatile(
        "{\n\t.reg .b32 remaddr;\n\t"
        "mapa.shared::cluster.u32 remaddr, %0, %1;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [remaddr];\n\t}"
        ::"r"(bar), "r"(cta)
        : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    return mbar_wait_bounded(bar, parity, abort_flag, code, WAIT_BUDGET, &g_status);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
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
__device__ __forceinline__ void mma_i8_2cta(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accum)
        : "memory");
}
// arrives (once) on the barrier at this offset in both CTAs of the pair when the MMAs issued so far are done
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

// Tile -> coordinates.  Dense: tile = m_tile * tiles_n + n_tile over one [M, N] problem.
// Grouped (row_off != null): the rows of A are sorted by expert, expert e owns rows
// row_off[e] .. row_off[e+1]-1 and multiplies the weight rows e*N .. e*N+N-1 of B; its m-tiles start
// at its first row, and rows of a tile past the expert's last row are computed but never stored.
struct TileCoord {
    uint32_t a_row;     // first row of A of the pair's tile
    uint32_t b_row;     // first row of B (weight row, expert offset included)
    uint32_t n0;        // first output column
    uint32_t row_end;   // rows >= row_end are not stored
    uint32_t bn;        // output columns of this item: 256, or 128 for the halves of the last wave's tiles
    uint32_t kb0;       // first k-block of this item (split K; 0 otherwise)
    uint32_t ks;        // which k-range of its tile this item is
    uint32_t tile;      // tile index (split K: the counter the ranges of a tile meet at)
};

// Epilogue of one split-K item (see the header): the warp's 32 accumulator rows go to the workspace, the warp meets
// the warps of the same rows in the other k-ranges' pairs on a counter of its own (tile, CTA rank, quarter), then
// sums and finishes the chunks c = ks, ks + S, ... of the tile.  Only the SPLITK instantiation of the kernel contains it.
__device__ __forceinline__ bool splitk_epilogue(const Epilogue ep, int32_t *__restrict__ ws, int32_t *__restrict__ split_cnt,
                                             uint32_t tmem_rows, uint32_t acc_empty_bar, const TileCoord tc, uint32_t S,
                                             uint32_t m_pad, uint32_t n_pad, uint32_t row0, int lane, uint32_t rank,
                                             uint32_t quarter, uint32_t N, bool small, uint8_t *stage, volatile int *ab) {
    const int chunks = (int)(tc.bn / 32);
    // The workspace is not a matrix: the warp that reads a piece is the warp of the same (tile, CTA rank, quarter) in
    // another pair, with the same lane on the same row, so a piece is stored where the 32 lanes of one store (or load)
    // instruction touch 512 consecutive bytes: ws[k-range][tile][rank][quarter][chunk][j][lane] in units of int4.
    const size_t slab = (size_t)m_pad * n_pad;                            // int32 words per k-range
    const size_t at = ((((size_t)tc.tile * 2 + rank) * 4 + quarter) * 8) * 8 * 32 * 4 + (size_t)lane * 4;
#pragma unroll 1
    for (int c = 0; c < chunks; ++c) {
        int v[32];
        tmem_ld32(tmem_rows + (uint32_t)(c * 32), v);
        if (c == chunks - 1) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_bar, 0);
        }
        int4 *dst = reinterpret_cast<int4 *>(ws + (size_t)tc.ks * slab + at + (size_t)c * 8 * 32 * 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j * 32] = make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    __threadfence();                                                    // this lane's partial sums are visible device-wide
    __syncwarp();
    // The counter only ever grows: every launch adds S to it, so the arrivals of this launch are old .. old + S - 1 with
    // old a multiple of S, and everybody waits for the next multiple.  One bank of counters per S (a counter that has
    // served S = 4 need not hold a multiple of 8), nothing to put back at the end.
    const uint32_t bank = S == 2 ? 0u : 1u;
    int32_t *cnt = split_cnt + bank * (SPLIT_COUNTERS / 2) + ((2 * tc.tile + rank) * 4 + quarter);
    int gave_up = 0;
    if (lane == 0) {
        const uint32_t old = (uint32_t)atomicAdd(cnt, 1);
        const uint32_t target = (old / S + 1) * S;
        const long long t0 = clock64();
        while ((int32_t)((uint32_t)*reinterpret_cast<volatile int32_t *>(cnt) - target) < 0) {
            if (*ab != 0) {
                gave_up = 1;
                break;
            }
            if (clock64() - t0 > WAIT_BUDGET) {                          // a k-range never arrived: give up, keep the context
                atomicCAS(&g_status, 0, 47);
                *ab = 47;
                gave_up = 1;
                break;
            }
        }
    }
    gave_up = __shfl_sync(0xffffffffu, gave_up, 0);
    __threadfence();
    if (gave_up) return false;
#pragma unroll 1
    for (int c = (int)tc.ks; c < chunks; c += (int)S) {
        int v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0;
        // four int4 of every k-range at a time (S <= 4): sixteen loads in flight, two trips to L2 per chunk
        const int4 *src = reinterpret_cast<const int4 *>(ws + at + (size_t)c * 8 * 32 * 4);
#pragma unroll
        for (int j = 0; j < 8; j += 4) {
            int4 q[4][4];
#pragma unroll
            for (uint32_t r = 0; r < 4; ++r)
                if (r < S) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) q[r][i] = __ldcg(src + r * (slab / 4) + (j + i) * 32);
                }
#pragma unroll
            for (uint32_t r = 0; r < 4; ++r)
                if (r < S) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        v[4 * (j + i)] += q[r][i].x;
                        v[4 * (j + i) + 1] += q[r][i].y;
                        v[4 * (j + i) + 2] += q[r][i].z;
                        v[4 * (j + i) + 3] += q[r][i].w;
                    }
                }
        }
        store_acc_chunk_warp(ep, row0, lane, tc.n0 + c * 32, v, tc.row_end, N, small, stage);
    }
    return true;
}

// A grouped launch whose sizes the host never sees (the pointer-array entry matmul_grouped): everything the kernel
// takes from its arguments in the other modes (sizes, row offsets, both tensor maps, the output) is written here by
// group_plan_kernel, on the device, just before the GEMM kernel reads it.
struct GroupPlan {
    alignas(128) CUtensorMap map_a;   // [rows, k/2] bytes, row stride lda/2
    alignas(128) CUtensorMap map_b;   // [num * n, k/2] bytes, row stride ldb/2
    int32_t use_tc;                   // 1: this kernel computes the problems; 0: it returns at once (the CUDA-core kernel runs)
    int32_t num;                      // problems (experts)
    uint32_t n, k, rows;
    int32_t *c;                       // output of problem 0; row r of the sorted activations is row r of c
    int64_t ldc;
    int32_t row_off[MAX_EXPERTS + 1]; // first activation row of every problem
};
constexpr int PLAN_SLOTS = 16;        // one per stream that calls the entry (see plan_slot)
__device__ GroupPlan g_plans[PLAN_SLOTS];

// SPLITK: the instantiation that may split K (dense launches with a workspace); the others carry none of its code.
template <bool A_UNSIGNED, int G, bool PLAN, bool SPLITK = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tc3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, uint32_t M,
                uint32_t N_arg, uint32_t K_arg, int SP, int SU, const int32_t *__restrict__ row_off_arg,
                int num_experts_arg, Epilogue ep_arg, const GroupPlan *__restrict__ plan, int ksplit,
                int32_t *__restrict__ ws, int32_t *__restrict__ split_cnt) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    const int off_un_a = 0, off_un_b = SU * UN_A, off_pk_a = SU * (UN_A + UN_B), off_pk_b = off_pk_a + SP * PK_A;
    const uint32_t bars = base + off_pk_b + SP * PK_B;
    auto pk_full = [&](int s) { return bars + 8u * s; };
    auto pk_empty = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
    auto un_full = [&](int s) { return bars + 8u * (2 * MAX_STAGES + s); };             // used in the leader only
    auto un_empty = [&](int s) { return bars + 8u * (3 * MAX_STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (4 * MAX_STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (4 * MAX_STAGES + 2 + b); };       // used in the leader only

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    // Launched with programmatic serialization (launch_pdl): barrier set-up and the TMEM allocation below overlap
    // the tail of the kernel before this one; only the TMA producer and the epilogue warps touch memory that an
    // earlier kernel may have written (grouped launches also read the row offsets, or the whole plan, right here).
    const bool grouped = PLAN || row_off_arg != nullptr;
    pdl_trigger();
    if (grouped) pdl_wait();
    uint32_t N = N_arg, K = K_arg;
    const int32_t *row_off = row_off_arg;
    int num_experts = num_experts_arg;
    Epilogue ep = ep_arg;
    const CUtensorMap *pmap_a = &map_a, *pmap_b = &map_b;
    bool active = true;
    if (PLAN) {
        N = plan->n;
        K = plan->k;
        row_off = plan->row_off;
        num_experts = plan->num;
        ep.c = plan->c;
        ep.ldc = plan->ldc;
        pmap_a = &plan->map_a;
        pmap_b = &plan->map_b;
        active = plan->use_tc != 0;
        if (!active) num_experts = 0;
    }
    const bool small = (A_UNSIGNED ? 120u : 64u) * (uint64_t)K < (1u << 22);
    const uint32_t tiles_n = (N + BN - 1) / BN;
    const uint32_t num_kb = (K + BK - 1) / BK;
    const uint32_t cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    // mt_start[e] = number of m-tiles of the experts before e (grouped launches only)
    uint32_t *mt_start = reinterpret_cast<uint32_t *>(base_ptr + off_pk_b + SP * PK_B + BAR_BYTES);
    uint8_t *epi_stage = base_ptr + off_pk_b + SP * PK_B + BAR_BYTES + SCHED_BYTES;

    if (tid == 0) {
        if (grouped) {
            uint32_t acc = 0;
            for (int e = 0; e < num_experts; ++e) {
                mt_start[e] = acc;
                const int rows_e = row_off[e + 1] - row_off[e];
                acc += rows_e > 0 ? ((uint32_t)rows_e + 2 * BMC - 1) / (2 * BMC) : 0u;
            }
            mt_start[num_experts] = acc;
        }
        abort_flag = g_status;
        for (int s = 0; s < SP; ++s) {
            mbar_init(pk_full(s), 1);
            mbar_init(pk_empty(s), UNPACK_WARPS / G);
        }
        for (int s = 0; s < SU; ++s) {
            mbar_init(un_full(s), 2 * UNPACK_WARPS / G);
            mbar_init(un_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 2 * 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    // barriers of both CTAs are initialised before anyone signals across the pair
    asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = tmem_base_slot;
    volatile int *ab = &abort_flag;
    const uint32_t tiles_m = grouped ? mt_start[num_experts] : (M + 2 * BMC - 1) / (2 * BMC);
    const uint32_t num_tiles = tiles_n * tiles_m;
    // Work items.  Tiles are dealt round-robin to the clusters; when the last round would leave at least half of
    // the clusters idle, its tiles are split into two 256 x 128 halves so that the round costs half a tile.
    // (A problem with so few tiles that even the halves leave clusters idle is split entirely.)
    // Split K (S > 1; the host has checked tiles * S <= clusters and num_kb % S == 0): item = tile * S + k-range.
    const uint32_t S = (!SPLITK || PLAN || grouped || ksplit < 1) ? 1u : (uint32_t)ksplit;
    const uint32_t kbs = num_kb / S;                      // k-blocks of one item
    const uint32_t rem = num_tiles % clusters;
    const uint32_t split = S > 1 ? 0u
                                 : ((2 * num_tiles <= clusters) ? num_tiles : ((rem != 0 && 2 * rem <= clusters) ? rem : 0u));
    const uint32_t full_items = (num_tiles - split) * S, num_items = (num_tiles + split) * S;
    auto coord = [&](uint32_t item) {
        TileCoord c;
        uint32_t tile = item / S, half = 0;
        c.ks = item % S;
        c.kb0 = c.ks * kbs;
        c.bn = BN;
        if (item >= full_items) {
            tile = full_items + ((item - full_items) >> 1);
            half = (item - full_items) & 1;
            c.bn = BN / 2;
        }
        c.tile = tile;
        const uint32_t mt = tile / tiles_n, nt = tile % tiles_n;
        c.n0 = nt * BN + half * (BN / 2);
        if (!grouped) {
            c.a_row = mt * 2 * BMC;
            c.b_row = c.n0;
            c.row_end = M;
        } else {
            int lo = 0, hi = num_experts - 1;   // last expert whose first m-tile is <= mt (empty experts share a start)
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (mt_start[mid] <= mt) lo = mid;
                else hi = mid - 1;
            }
            c.a_row = (uint32_t)row_off[lo] + (mt - mt_start[lo]) * 2 * BMC;
            c.b_row = (uint32_t)lo * N + c.n0;
            c.row_end = (uint32_t)row_off[lo + 1];
        }
        return c;
    };

    if (*ab == 0 && active) {
        if (warp == 0) {
            // ------------------------------------------------ TMA producer (own rows only)
            if (lane == 0) {
                if (!grouped) pdl_wait();
                if (PLAN) {
                    // the maps were written by a kernel: drop any copy of these 128-byte lines that the
                    // tensor-map cache still holds from an earlier call
                    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(pmap_a) : "memory");
                    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(pmap_b) : "memory");
                }
                Ring pr;
                bool ok = true;
                for (uint32_t item = cluster; item < num_items && ok; item += clusters) {
                    const TileCoord tc = coord(item);
                    const int ya = (int)(tc.a_row + rank * BMC);
                    const int yb = (int)(tc.b_row + rank * (tc.bn / 2));   // a half tile uses the first 64 rows of the box
                    for (uint32_t kb = 0; kb < kbs; ++kb, pr.next(SP)) {
                        const int s = pr.s;
                        ok = mbar_wait(pk_empty(s), pr.ph ^ 1, ab, 41);
                        if (!ok) break;
                        mbar_expect_tx(pk_full(s), PK_A + PK_B);
                        tma_load_2d(base + off_pk_a + s * PK_A, pmap_a, (int)((tc.kb0 + kb) * PK_ROW), ya, pk_full(s));
                        tma_load_2d(base + off_pk_b + s * PK_B, pmap_b, (int)((tc.kb0 + kb) * PK_ROW), yb, pk_full(s));
                    }
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------ MMA issuer (leader CTA only)
            if (rank == 0 && lane == 0) {
                const uint32_t idesc_base = (2u << 4) | ((A_UNSIGNED ? 0u : 1u) << 7) | (1u << 10) |
                                            ((uint32_t)((2 * BMC) >> 4) << 24);
                uint32_t it = 0;
                Ring ur;
                bool ok = true;
                for (uint32_t item = cluster; item < num_items && ok; item += clusters, ++it) {
                    const uint32_t buf = it & 1;
                    const uint32_t idesc = idesc_base | (((item >= full_items ? BN / 2 : BN) >> 3) << 17);
                    ok = mbar_wait(acc_empty(buf), ((it >> 1) & 1) ^ 1, ab, 42);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t d_tmem = tmem_acc + buf * BN;
                    for (uint32_t kb = 0; kb < kbs; ++kb, ur.next(SU)) {
                        const int s = ur.s;
                        ok = mbar_wait(un_full(s), ur.ph, ab, 43);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t da = make_desc(base + off_un_a + s * UN_A);
                        const uint64_t db = make_desc(base + off_un_b + s * UN_B);
#pragma unroll
                        for (int kk = 0; kk < BK / 32; ++kk)
                            mma_i8_2cta(d_tmem, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc,
                                        (kb > 0 || kk > 0) ? 1u : 0u);
                        mma_commit_pair(un_empty(s));
                    }
                    if (ok) mma_commit_pair(acc_full(buf));
                }
            }
        } else if (warp <= 5) {
            // ------------------------------------------------ epilogue (own 128 rows)
            const uint32_t quarter = warp & 3;
            uint32_t it = 0;
            bool ok = true;
            if (!grouped) pdl_wait();
            for (uint32_t item = cluster; item < num_items && ok; item += clusters, ++it) {
                const uint32_t buf = it & 1;
                const TileCoord tc = coord(item);
                const uint32_t m0 = tc.a_row + rank * BMC, n0 = tc.n0;
                const int chunks = (int)(tc.bn / 32);
                ok = mbar_wait(acc_full(buf), (it >> 1) & 1, ab, 44);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t row0 = m0 + quarter * 32;
                uint8_t *stage = epi_stage + quarter * 2560;
                if (SPLITK && S > 1) {
                    ok = splitk_epilogue(ep, ws, split_cnt, tmem_acc + ((quarter * 32u) << 16) + buf * BN, acc_empty(buf), tc, S,
                                         tiles_m * 2 * BMC, tiles_n * BN, row0, lane, rank, quarter, N, small, stage, ab);
                    if (!ok) break;
                    continue;
                }
#pragma unroll 1
                for (int c = 0; c < chunks; ++c) {
                    int v[32];
                    tmem_ld32(tmem_acc + ((quarter * 32u) << 16) + buf * BN + (uint32_t)(c * 32), v);
                    if (c == chunks - 1) {
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(acc_empty(buf), 0);
                    }
                    store_acc_chunk_warp(ep, row0, lane, n0 + c * 32, v, tc.row_end, N, small, stage);
                }
            }
        } else {
            // ------------------------------------------------ unpack
            // The warps form G groups; group i converts k-blocks i, i + G, ...  The proxy fence
            // that publishes a stage to the tensor core takes several hundred cycles, so
            // consecutive k-blocks are converted by different warps and the fences overlap.
            constexpr int GT = NUM_UNPACK / G;        // threads per group
            constexpr int STEPS = 4 * G;              // 16-byte packed chunks per thread and k-block
            const int t = tid - 192;                  // 0..255
            const int grp = t / GT, tg = t % GT;
            // step i handles chunk i * GT + tg: row r0 + i * GT / 4 (r0 = tg / 4), quad tg % 4 of A
            // (first half of the steps) or B; the row's position inside its 8-row swizzle atom and
            // the quad never change, so every step is a constant offset from two per-thread bases
            const int r0 = tg >> 2, qd = tg & 3;
            const uint32_t ld_off = (uint32_t)tg * 16;
            const uint32_t st_off = (uint32_t)((r0 >> 3) * 1024 + (r0 & 7) * 128);
            const uint32_t sw_e = (uint32_t)(((2 * qd) ^ (r0 & 7)) << 4), sw_o = (uint32_t)(((2 * qd + 1) ^ (r0 & 7)) << 4);
            const uint32_t my_items = (num_items > cluster) ? ((num_items - cluster - 1) / clusters + 1) : 0;
            const uint32_t total = my_items * kbs;
            bool ok = true;
            Ring pr, ur;
            for (int i = 0; i < grp; ++i) {
                pr.next(SP);
                ur.next(SU);
            }
            // position of k-block g in the item sequence: a half tile needs only the first 64 rows of B
            uint32_t cur_item = cluster, kb_pos = (uint32_t)grp;
            for (uint32_t g = grp; g < total && ok; g += G, kb_pos += G) {
                while (kb_pos >= kbs) {
                    kb_pos -= kbs;
                    cur_item += clusters;
                }
                const int b_steps = cur_item >= full_items ? STEPS / 4 : STEPS / 2;
                const int s = pr.s, u = ur.s;
                ok = mbar_wait(pk_full(s), pr.ph, ab, 45);
                if (!ok) break;
                ok = mbar_wait(un_empty(u), ur.ph ^ 1, ab, 46);
                if (!ok) break;
                const uint8_t *pa = base_ptr + off_pk_a + s * PK_A + ld_off;
                const uint8_t *pb = base_ptr + off_pk_b + s * PK_B + ld_off;
                uint8_t *ua = base_ptr + off_un_a + u * UN_A + st_off;
                uint8_t *ub = base_ptr + off_un_b + u * UN_B + st_off;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint8_t *src = half ? pb : pa;
                    uint8_t *dst = half ? ub : ua;
                    const int n_steps = half ? b_steps : STEPS / 2;
                    uint4 pk[STEPS / 2];
#pragma unroll
                    for (int i = 0; i < STEPS / 2; ++i)
                        if (i < n_steps) pk[i] = *reinterpret_cast<const uint4 *>(src + i * GT * 16);
                    if (half == 1) {
                        // every packed byte of the stage is in registers (the masks below depend on the loads of this
                        // half, the first half was consumed before): the TMA producer may refill it while the rest of
                        // the conversion, the stores and the fence run
                        uint32_t seen = 0;
#pragma unroll
                        for (int i = 0; i < STEPS / 2; ++i)
                            if (i < n_steps) seen |= pk[i].x | pk[i].y | pk[i].z | pk[i].w;
                        asm volatile("" ::"r"(seen) : "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(pk_empty(s));
                    }
#pragma unroll
                    for (int i = 0; i < STEPS / 2; ++i) {
                        if (i >= n_steps) break;
                        uint4 e, od;
                        // the shift runs as a multiply on the FMA pipe, the masks on the ALU pipe
                        e.x = (pk[i].x * 16u) & 0xF0F0F0F0u; od.x = pk[i].x & 0xF0F0F0F0u;
                        e.y = (pk[i].y * 16u) & 0xF0F0F0F0u; od.y = pk[i].y & 0xF0F0F0F0u;
                        e.z = (pk[i].z * 16u) & 0xF0F0F0F0u; od.z = pk[i].z & 0xF0F0F0F0u;
                        e.w = (pk[i].w * 16u) & 0xF0F0F0F0u; od.w = pk[i].w & 0xF0F0F0F0u;
                        uint8_t *rowp = dst + i * (GT / 32) * 1024;
                        *reinterpret_cast<uint4 *>(rowp + sw_e) = e;
                        *reinterpret_cast<uint4 *>(rowp + sw_o) = od;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(un_full(u), 0);  // the leader's MMA warp waits for both CTAs
                for (int i = 0; i < G; ++i) {
                    pr.next(SP);
                    ur.next(SU);
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
    // neither CTA may leave (or free TMEM) while its partner can still signal it or read its tiles
    asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(512u) : "memory");
    }
}

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

static int make_map(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                    uint64_t stride_bytes = 0) {
    EncodeTiledFn fn = encode_fn();
    SR_REQUIRE(fn != nullptr, SR_ERR_CUDA, "matmul: cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {stride_bytes ? stride_bytes : row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)PK_ROW, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SR_REQUIRE(r == CUDA_SUCCESS, SR_ERR_CUDA, "matmul: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return SR_OK;
}

// ---------------------------------------------------------------- pointer-array front end
//
// matmul_grouped (signrot/kernels/bindings.cpp:49-91) hands over P problems as device arrays of sizes, pointers and
// leading dimensions.  The layout the reference's MoE block builds (signrot/nn/moe.py:96-111: activation rows sorted
// by expert, stacked weights, one output matrix) is exactly what the grouped launch above wants, so one small kernel
// recognises it on the device: equal n, k and leading dimensions, ptr_b[p] = ptr_b[0] + p * n rows, and
// ptr_a[p] / ptr_c[p] = row (m_0 + ... + m_{p-1}) of problem 0's matrices.  When that holds, and there are enough
// rows for the tensor cores to pay, it writes the row offsets and both tensor maps into the plan; otherwise it
// clears use_tc and the CUDA-core kernel, which takes any layout, does the work.
__global__ void __launch_bounds__(MAX_EXPERTS)
group_plan_kernel(const __grid_constant__ CUtensorMap tmpl_small, const __grid_constant__ CUtensorMap tmpl_large,
                  GroupPlan *__restrict__ plan,
                  const int32_t *__restrict__ sizes, int P, const int64_t *__restrict__ ptr_a,
                  const int64_t *__restrict__ ptr_b, const int64_t *__restrict__ ptr_c,
                  const int64_t *__restrict__ lda, const int64_t *__restrict__ ldb, const int64_t *__restrict__ ldc,
                  int64_t k_limit) {
    __shared__ alignas(128) CUtensorMap sm_map[2];
    __shared__ uint32_t warp_sum[MAX_EXPERTS / 32];
    const int p = threadIdx.x, lane = p & 31, w = p >> 5;
    const bool have = p < P;
    const int64_t m = have ? sizes[3 * p] : 0, n = have ? sizes[3 * p + 1] : 0, k = have ? sizes[3 * p + 2] : 0;
    // exclusive prefix sum of the row counts (they are below 2^31 in total or the problem is rejected below)
    uint32_t incl = (uint32_t)(m > 0 ? m : 0);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) warp_sum[w] = incl;
    __syncthreads();
    uint32_t before = 0;
    for (int i = 0; i < w; ++i) before += warp_sum[i];
    const uint32_t off = before + incl - (uint32_t)(m > 0 ? m : 0);

    const int64_t n0 = sizes[1], k0 = sizes[2], la = lda[0], lb = ldb[0], lc = ldc[0];
    const int64_t a0 = ptr_a[0], b0 = ptr_b[0], c0 = ptr_c[0];
    bool ok = true;
    if (have) {
        ok = m >= 0 && m < (1ll << 21) && n == n0 && k == k0 && lda[p] == la && ldb[p] == lb && ldc[p] == lc &&
             ptr_a[p] == a0 + (int64_t)off * (la >> 1) && ptr_b[p] == b0 + (int64_t)p * n0 * (lb >> 1) &&
             ptr_c[p] == c0 + (int64_t)off * lc * 4;
    }
    if (p == 0) {
        ok = ok && n0 > 0 && k0 > 0 && (k0 & 31) == 0 && k0 <= k_limit && la >= k0 && lb >= k0 && lc >= n0 &&
             (la & 31) == 0 && (lb & 31) == 0 && (la >> 1) < (1ll << 31) && (lb >> 1) < (1ll << 31) &&
             ((a0 | b0) & 15) == 0 && (c0 & 3) == 0 && n0 * (int64_t)P < (1ll << 31);
    }
    const bool regular = __syncthreads_and(ok) != 0;
    // rows in total: the last thread that has a problem knows
    __shared__ uint32_t rows_total;
    if (p == P - 1) rows_total = off + (uint32_t)m;
    __syncthreads();
    const uint32_t rows = rows_total;
    // the tensor cores take over where the grouped dequant entry switches as well: more than 16 rows per problem
    const bool use_tc = regular && rows > 16u * (uint32_t)P;
    if (have) plan->row_off[p] = (int32_t)off;
    if (p == 0) {
        plan->row_off[P] = (int32_t)rows;
        plan->use_tc = use_tc ? 1 : 0;
        plan->num = P;
        plan->n = (uint32_t)n0;
        plan->k = (uint32_t)k0;
        plan->rows = rows;
        plan->c = reinterpret_cast<int32_t *>(c0);
        plan->ldc = lc;
    }
    if (w == 0 && use_tc) {
        // both maps: a host-encoded template (element type, box of 64 bytes x 128 rows, no swizzle) with the
        // address, the two extents and the row stride replaced, then copied to the plan with the release that the
        // consumer's acquire pairs with.  The encoder sets one more bit from the sizes, for tensors that span
        // 128 KiB or more; it is taken from the template, so there is one template on either side of that limit and
        // the result is, bit for bit, what cuTensorMapEncodeTiled returns for the same matrix.
        if (lane < 2) {
            const uint64_t addr = (uint64_t)(lane == 0 ? a0 : b0);
            const uint32_t row_bytes = (uint32_t)(k0 >> 1);
            const uint32_t n_rows = lane == 0 ? rows : (uint32_t)(n0 * P);
            const uint64_t stride = (uint64_t)((lane == 0 ? la : lb) >> 1);
            const bool large = (uint64_t)(n_rows - 1) * stride + row_bytes >= (128u << 10);
            const uint4 *src = reinterpret_cast<const uint4 *>(large ? &tmpl_large : &tmpl_small);
            uint4 *dst = reinterpret_cast<uint4 *>(&sm_map[lane]);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = src[i];
            const uint32_t sm = smem_u32(&sm_map[lane]);
            asm volatile("tensormap.replace.tile.global_address.shared::cta.b1024.b64 [%0], %1;" ::"r"(sm), "l"(addr)
                         : "memory");
            asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 0, %1;" ::"r"(sm), "r"(row_bytes)
                         : "memory");
            asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 1, %1;" ::"r"(sm), "r"(n_rows)
                         : "memory");
            asm volatile("tensormap.replace.tile.global_stride.shared::cta.b1024.b64 [%0], 0, %1;" ::"r"(sm), "l"(stride)
                         : "memory");
        }
        __syncwarp();
        asm volatile(
            "tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], [%1], 128;"
            ::"l"(&plan->map_a), "r"(smem_u32(&sm_map[0]))
            : "memory");
        asm volatile(
            "tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], [%1], 128;"
            ::"l"(&plan->map_b), "r"(smem_u32(&sm_map[1]))
            : "memory");
    }
}

}  // namespace tc3

// Shared launcher.  row_off == null: one dense [M, N] problem.  Otherwise M is the total number
// of (expert-sorted) rows, B holds num_experts stacked [N, K/2] weights and row_off[num_experts + 1]
// lives on the device, so the grid is sized for the worst case (every expert adds a partial tile).
// K ranges per tile of a dense launch (1 = no split): 4 or 2, every item with its own CTA pair and at least sixteen
// k-blocks, for long-K problems whose tiles would leave half of the pairs idle.
static int tc3_ksplit(int64_t M, int64_t N, int64_t K, int sm_count) {
    using namespace tc3;
    const int64_t tiles = cdiv<int64_t>(N, BN) * cdiv<int64_t>(M, 2 * BMC), clusters = sm_count / 2;
    const int64_t num_kb = cdiv<int64_t>(K, BK);
    // measured on B200 at M = 256: meeting in the workspace costs about 10 us per launch, so the split pays for long K
    // only ((K, N) = (14336, 4096): 42 -> 27 us with four ranges; (4096, 4096): 16 -> 20 us, left alone)
    if (2 * tiles > clusters || num_kb < 64) return 1;
    for (int s = 4; s >= 2; s >>= 1)
        if (tiles * s <= clusters && num_kb % s == 0 && num_kb / s >= 16) return s;
    return 1;
}

int64_t gemm_tc3_splitk_bytes(int64_t M, int64_t N, int64_t K) {
    using namespace tc3;
    const int s = tc3_ksplit(M, N, K, current_sm_count());
    if (s == 1) return 0;
    return (int64_t)s * cdiv<int64_t>(M, 2 * BMC) * 2 * BMC * cdiv<int64_t>(N, BN) * BN * 4;
}

static int launch_tc3(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                      const Epilogue &ep, const int32_t *row_off, int num_experts, cudaStream_t st,
                      int32_t *ws = nullptr, int64_t ws_bytes = 0, int32_t *split_cnt = nullptr) {
    using namespace tc3;
    SR_REQUIRE(aligned16(A) && aligned16(B), SR_ERR_INVALID, "matmul: operands must be 16-byte aligned");
    SR_REQUIRE(K % 32 == 0, SR_ERR_INVALID, "matmul: K = %lld must be a multiple of 32", (long long)K);
    const int64_t b_rows = row_off ? N * (int64_t)num_experts : N;
    SR_REQUIRE(M < (1ll << 31) && b_rows < (1ll << 31), SR_ERR_UNSUPPORTED, "matmul: size out of range");
    CUtensorMap ma, mb;
    SR_REQUIRE(ep.lda % 16 == 0, SR_ERR_INVALID, "matmul: the row stride of A must be a multiple of 16 bytes");
    int rc = make_map(&ma, A, (uint64_t)M, (uint64_t)K / 2, BMC, ep.lda);
    if (rc) return rc;
    rc = make_map(&mb, B, (uint64_t)b_rows, (uint64_t)K / 2, BNC);
    if (rc) return rc;
    const int sm_count = current_sm_count();
    const int64_t m_tiles = row_off ? cdiv<int64_t>(M, 2 * BMC) + num_experts : cdiv<int64_t>(M, 2 * BMC);
    const int64_t tiles = cdiv<int64_t>(N, BN) * m_tiles;
    int64_t clusters = sm_count / 2;
    int ksplit = 1;
    if (!row_off && ws != nullptr && split_cnt != nullptr) {
        ksplit = tc3_ksplit(M, N, K, sm_count);
        if (ksplit > 1 && (ws_bytes < gemm_tc3_splitk_bytes(M, N, K) || !aligned16(ws) || 2 * tiles * 4 > SPLIT_COUNTERS / 2))
            ksplit = 1;
    }
    if (ksplit > 1) clusters = tiles * ksplit;         // every k-range of every tile has its own pair
    else if (2 * tiles <= clusters) clusters = 2 * tiles;   // every tile is split into two halves (see the kernel)
    else if (tiles < clusters) clusters = tiles;
    // ring depths: packed (TMA) stages, unpacked int8 stages, unpack warp groups (a group may run at most one
    // pass ahead of a ring's barriers, so groups <= both depths)
    constexpr int sp = 5, su = 4, groups = 4;
    static_assert(groups <= sp && groups <= su, "unpack groups exceed a ring depth");
    void (*kfn)(const CUtensorMap, const CUtensorMap, uint32_t, uint32_t, uint32_t, int, int, const int32_t *, int,
                Epilogue, const GroupPlan *, int, int32_t *, int32_t *);
    if (ksplit > 1) kfn = a_unsigned ? gemm_tc3_kernel<true, groups, false, true> : gemm_tc3_kernel<false, groups, false, true>;
    else kfn = a_unsigned ? gemm_tc3_kernel<true, groups, false> : gemm_tc3_kernel<false, groups, false>;
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "matmul: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    launch_pdl(kfn, dim3((unsigned)(2 * clusters)), dim3(THREADS), smem_bytes(sp, su), st, ma, mb, (uint32_t)M, (uint32_t)N,
               (uint32_t)K, sp, su, row_off, num_experts, ep, (const GroupPlan *)nullptr, ksplit, ws, split_cnt);
    return check_launch("gemm_tc3");
}

// The plan a stream's calls use.  Calls on one stream run one after the other, so they can share a plan; every
// stream seen gets its own, up to PLAN_SLOTS (further streams share by hash, and two graphs captured on the same
// stream must not be replayed at the same time).
static int plan_slot(cudaStream_t st) {
    static std::mutex mu;
    static cudaStream_t owner[tc3::PLAN_SLOTS];
    static int used = 0;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
        if (owner[i] == st) return i;
    if (used < tc3::PLAN_SLOTS) {
        owner[used] = st;
        return used++;
    }
    return (int)((reinterpret_cast<uintptr_t>(st) >> 4) % tc3::PLAN_SLOTS);
}

// Tensor-core side of matmul_grouped: the planning kernel, then the CTA-pair kernel on the full grid (the host knows
// no size).  *use_tc_flag receives the device address of the word that says which kernel has the work.
int launch_gemm_tc3_ptr_array(const int32_t *sizes, int64_t P, const int64_t *ptr_a, const int64_t *ptr_b,
                              const int64_t *ptr_c, const int64_t *lda, const int64_t *ldb, const int64_t *ldc,
                              bool a_unsigned, int64_t k_limit, const int32_t **use_tc_flag, cudaStream_t st) {
    using namespace tc3;
    SR_REQUIRE(P >= 1 && P <= MAX_EXPERTS, SR_ERR_UNSUPPORTED, "matmul_grouped: at most %d problems on the tensor cores",
               MAX_EXPERTS);
    GroupPlan *plans = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void **)&plans, g_plans);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "matmul_grouped: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    GroupPlan *plan = plans + plan_slot(st);
    // templates of the maps: what make_map encodes for a matrix of 128 (8 KiB) and of 4096 (256 KiB) rows of
    // 64 bytes; the planning kernel replaces address, extents and stride
    CUtensorMap tmpl, tmpl_large;
    int rc = make_map(&tmpl, plans, 128, PK_ROW, BMC);
    if (rc) return rc;
    rc = make_map(&tmpl_large, plans, 4096, PK_ROW, BMC);
    if (rc) return rc;
    group_plan_kernel<<<1, MAX_EXPERTS, 0, st>>>(tmpl, tmpl_large, plan, sizes, (int)P, ptr_a, ptr_b, ptr_c, lda, ldb, ldc,
                                                 k_limit);
    rc = check_launch("matmul_grouped plan");
    if (rc) return rc;
    constexpr int sp = 5, su = 4, groups = 4;
    void (*kfn)(const CUtensorMap, const CUtensorMap, uint32_t, uint32_t, uint32_t, int, int, const int32_t *, int,
                Epilogue, const GroupPlan *, int, int32_t *, int32_t *);
    kfn = a_unsigned ? gemm_tc3_kernel<true, groups, true> : gemm_tc3_kernel<false, groups, true>;
    e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "matmul_grouped: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    Epilogue ep = {};
    ep.mode = 0;
    const int clusters = current_sm_count() / 2;
    launch_pdl(kfn, dim3((unsigned)(2 * clusters)), dim3(THREADS), smem_bytes(sp, su), st, tmpl, tmpl, 0u, 0u, 0u, sp, su,
               (const int32_t *)nullptr, 0, ep, (const GroupPlan *)plan, 1, (int32_t *)nullptr, (int32_t *)nullptr);
    *use_tc_flag = &plan->use_tc;
    return check_launch("gemm_tc3 (pointer array)");
}

int launch_gemm_tc3(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                    const Epilogue &ep, cudaStream_t st, int32_t *ws, int64_t ws_bytes, int32_t *split_cnt) {
    return launch_tc3(A, B, M, N, K, a_unsigned, ep, nullptr, 0, st, ws, ws_bytes, split_cnt);
}

int launch_gemm_tc3_grouped(const uint8_t *A, const uint8_t *B, int64_t rows, int64_t N, int64_t K, bool a_unsigned,
                            const Epilogue &ep, const int32_t *row_off, int num_experts, cudaStream_t st) {
    SR_REQUIRE(num_experts >= 1 && num_experts <= tc3::MAX_EXPERTS, SR_ERR_UNSUPPORTED,
               "grouped_linear: at most %d experts", tc3::MAX_EXPERTS);
    return launch_tc3(A, B, rows, N, K, a_unsigned, ep, row_off, num_experts, st);
}

// One thread waits, with the given cycle budget, on a barrier nobody arrives on: the give-up path of every
// bounded wait in this file (abort flag, status word, normal return), exercised without any other machinery.
__global__ void bounded_wait_probe_kernel(long long budget_cycles, int code) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        tc3::mbar_init(tc3::smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait_bounded(tc3::smem_u32(&bar), 0, &abort_flag, code, budget_cycles, &tc3::g_status);
    __syncthreads();
}

int launch_bounded_wait_probe(long long budget_cycles, cudaStream_t st) {
    bounded_wait_probe_kernel<<<1, 32, 0, st>>>(budget_cycles, 99);
    return check_launch("selftest_bounded_wait");
}

int tc3_device_status(int *out, bool clear) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, tc3::g_status, sizeof(int));
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
    if (clear && v != 0) {
        const int z = 0;
        cudaMemcpyToSymbol(tc3::g_status, &z, sizeof(int));
    }
    *out = v;
    return SR_OK;
}

}  // namespace sr
