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
// fragments with cp.async into a private shared-memory slot, 8 KB per warp ahead of the math, and
// the queue runs on across row blocks, so the loads of the next block are in flight while this one
// is reduced and stored.  Slots are private to a lane: no barrier guards the ring.
// Nibble n becomes the byte 16*n ((w << 4) & 0xF0F0F0F0 for the even nibbles of a word, w &
// 0xF0F0F0F0 for the odd ones), which reorders k inside a word in the same way for both operands,
// so the dot product is unchanged; every product carries a factor 256 that the epilogue removes
// with an exact shift.  The eight partial accumulators of a block meet in shared memory.
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace sr {

namespace {

constexpr int SK_WARPS = 8;
constexpr int SK_ROWS = 16;      // weight rows per CTA
constexpr int SK_STEP = 64;      // packed bytes of K per row and step (128 values)

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

// ring: SK_RING_BYTES per warp (steps of 1 KB per m-tile); red: one or two buffers of [warp][MT][NT][4][32] ints
constexpr int SK_RING_BYTES = 8192;
constexpr int SK_MAX_EXPERTS = 512;
constexpr size_t skinny_smem(int nt, int mt) {
    return (size_t)SK_WARPS * SK_RING_BYTES + (size_t)(nt <= 2 ? 2 : 1) * SK_WARPS * mt * nt * 4 * 32 * 4;
}

// One unit of work: a block of ROWS weight rows of one problem against up to 8 * NT activation rows.
// Dense launches have one problem; grouped (MoE) launches one per expert and, for an expert with more
// than 8 * NT rows, one pass per 8 * NT rows (its weights are then streamed once per pass).
struct SkItem {
    uint32_t w_row;     // first weight row (expert offset included)
    uint32_t n0;        // first output column
    uint32_t x_row0;    // first activation row of the pass
    uint32_t x_end;     // activation rows >= x_end do not exist
};

// NT = token blocks of 8 (at most 8 * NT activation rows per pass), MT = blocks of 16 weight rows a warp
// multiplies per step (the activation fragments of a step are unpacked once for all of them).
// A = activations [M, K/2], B = weights [N, K/2] (grouped: [E * N, K/2], row_off[E + 1] on the device).
// SWIGLU (dense, MT = 2): B holds the gate rows [0, N) followed by the up rows [N, 2N) (w_scale likewise);
// a block is 16 gate rows plus the 16 up rows of the same columns, and the epilogue writes
// rn_h(silu(gate) * up) as [M, N] (the arithmetic of swiglu_kernel on the two dequantized fp16 values), so
// the two projections and the activation of a SwiGLU MLP are one launch.
// KW = warps that split the K steps of one row block (8: the whole CTA works on one block; 2: four groups
// of two warps work on four blocks, so the per-block reduction and epilogue are paid once per 16 steps
// of a K = 4096 row instead of once per 4).
template <int NT, int MT, bool A_UNSIGNED, bool GROUPED, bool SWIGLU = false, int KW = SK_WARPS>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ B, uint32_t M, uint32_t N, uint32_t K,
                   const int32_t *__restrict__ row_off, int num_experts, Epilogue ep) {
    static_assert(!SWIGLU || (MT == 2 && !GROUPED), "the SwiGLU epilogue pairs the two m-tiles of a dense block");
    constexpr int ROWS = SWIGLU ? SK_ROWS : SK_ROWS * MT;   // output columns per block
    constexpr int STAGE = 1024 * MT;                    // bytes per warp and step
    constexpr int DEPTH = SK_RING_BYTES / STAGE;        // steps in flight per warp
    constexpr int RED_BUFS = NT <= 2 ? 2 : 1;
    extern __shared__ __align__(16) uint8_t sk_smem[];
    __shared__ uint32_t item_start[GROUPED ? SK_MAX_EXPERTS + 1 : 1];   // first item of every expert
    // Launched with programmatic serialization (launch_pdl): the weight stream below does not depend on
    // the kernel before this one, so the first ring of copies is in flight while that kernel finishes;
    // activations, scales and (grouped) the row offsets are read only after pdl_wait().
    pdl_trigger();
    if (GROUPED) pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    constexpr int GROUPS = SK_WARPS / KW;
    const int grp = warp / KW, kw = warp % KW, gtid = tid - grp * KW * 32;
    auto group_sync = [&]() {
        if (KW == SK_WARPS) __syncthreads();
        else asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "n"(KW * 32) : "memory");
    };
    // ring[warp][stage][row slot 0 .. 2 MT - 1][lane] (16 bytes each)
    const uint4 *ring = reinterpret_cast<const uint4 *>(sk_smem + (size_t)warp * SK_RING_BYTES) + lane;
    const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring);
    int *red = reinterpret_cast<int *>(sk_smem + (size_t)SK_WARPS * SK_RING_BYTES) +
               (size_t)grp * RED_BUFS * KW * MT * NT * 128;

    const uint32_t kp = K >> 1;                         // packed bytes per row
    const uint32_t steps = (kp + SK_STEP - 1) / SK_STEP;
    const uint32_t blocks = (N + ROWS - 1) / ROWS;
    const bool has_steps = (uint32_t)kw < steps;

    uint32_t total_items = blocks;
    if (GROUPED) {
        if (tid == 0) {
            uint32_t acc = 0;
            for (int e = 0; e < num_experts; ++e) {
                item_start[e] = acc;
                const int rows_e = row_off[e + 1] - row_off[e];
                acc += rows_e > 0 ? (((uint32_t)rows_e + 8 * NT - 1) / (8 * NT)) * blocks : 0u;
            }
            item_start[num_experts] = acc;
        }
        __syncthreads();
        total_items = item_start[num_experts];
    }
    auto decode = [&](uint32_t item) {
        SkItem it;
        if (!GROUPED) {
            it.w_row = item * ROWS;
            it.n0 = it.w_row;
            it.x_row0 = 0;
            it.x_end = M;
        } else {
            int lo = 0, hi = num_experts - 1;   // last expert whose first item is <= item (empty experts share a start)
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (item_start[mid] <= item) lo = mid;
                else hi = mid - 1;
            }
            const uint32_t local = item - item_start[lo];
            it.n0 = (local % blocks) * ROWS;
            it.w_row = (uint32_t)lo * N + it.n0;
            it.x_row0 = (uint32_t)row_off[lo] + (local / blocks) * 8 * NT;
            it.x_end = (uint32_t)row_off[lo + 1];
        }
        return it;
    };

    // queue of (item, step) of this warp, in the order they are consumed
    const uint32_t first_item = blockIdx.x * GROUPS + grp, item_stride = gridDim.x * GROUPS;
    uint32_t iss_item = first_item, iss_step = kw;
    uint32_t iss_n0 = 0;
    const uint8_t *iss_ptr = B;
    auto iss_open = [&]() {
        if (iss_item < total_items) {
            const SkItem it = decode(iss_item);
            iss_n0 = it.n0;
            iss_ptr = B + ((size_t)it.w_row + g) * kp + (size_t)kw * SK_STEP + 16 * q;
        }
    };
    iss_open();
    auto issue = [&](int slot) {
        if (has_steps && iss_item < total_items) {
            const bool k_ok = iss_step * SK_STEP + 16 * q + 16 <= kp;
            const uint32_t dst = ring_u32 + (uint32_t)slot * STAGE;
#pragma unroll
            for (int r = 0; r < 2 * MT; ++r) {
                // SWIGLU: slots 0, 1 are gate rows n0 + g (+ 8), slots 2, 3 the up rows N further down
                const uint32_t rr = SWIGLU ? (uint32_t)(8 * (r & 1)) : (uint32_t)(8 * r);
                const size_t jump = SWIGLU && r >= 2 ? (size_t)N : 0;
                const bool ok = k_ok && iss_n0 + g + rr < N;
                cp_async16(dst + r * 512, ok ? iss_ptr + ((size_t)rr + jump) * kp : B, ok ? 16u : 0u);
            }
            iss_step += KW;
            iss_ptr += KW * SK_STEP;
            if (iss_step >= steps) {
                iss_step = kw;
                iss_item += item_stride;
                iss_open();
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll 1
    for (int d = 0; d < DEPTH; ++d) issue(d);
    if (!GROUPED) pdl_wait();

    // activation fragments of the step after the current one (they come from L1/L2, one step ahead is enough)
    auto load_x = [&](const SkItem &it, uint32_t step, uint4 (&x)[NT]) {
        const bool k_ok = step * SK_STEP + 16 * q + 16 <= kp;
        const uint32_t lda = ep.lda ? ep.lda : kp;
        const uint8_t *xs = A + ((size_t)it.x_row0 + g) * lda + 16 * q + (size_t)step * SK_STEP;
#pragma unroll
        for (int t = 0; t < NT; ++t)
            x[t] = k_ok && it.x_row0 + g + 8 * t < it.x_end ? __ldg(reinterpret_cast<const uint4 *>(xs + (size_t)(8 * t) * lda))
                                                           : make_uint4(0, 0, 0, 0);
    };
    uint32_t item = first_item;
    SkItem cur = decode(item < total_items ? item : 0u);
    uint4 xn[NT];
    if (has_steps && item < total_items) load_x(cur, kw, xn);

    int slot = 0;
    uint32_t parity = 0;
    for (; item < total_items; item += item_stride, parity ^= (RED_BUFS - 1)) {
        const bool more = item + item_stride < total_items;
        const SkItem nxt = decode(more ? item + item_stride : item);
        int acc[MT][NT][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[m][t][i] = 0;
        // token blocks of 8 that exist in this pass (uniform over the CTA): the step loop is instantiated for every count,
        // so the missing ones cost no nibble expansion and no MMA (a grouped launch sizes its passes for 8 * NT rows,
        // most experts of a decode batch have fewer)
        const int tb = (int)min((uint32_t)NT, (cur.x_end - cur.x_row0 + 7u) >> 3);
        auto run_steps = [&](auto tb_tag) {
            constexpr int TB = decltype(tb_tag)::value;
#pragma unroll 1
            for (uint32_t s = kw; s < steps; s += KW) {
                uint4 x[NT];
#pragma unroll
                for (int t = 0; t < NT; ++t) x[t] = xn[t];
                if (s + KW < steps) load_x(cur, s + KW, xn);
                else if (more) load_x(nxt, kw, xn);
                asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
                uint4 w[2 * MT];
#pragma unroll
                for (int r = 0; r < 2 * MT; ++r) w[r] = ring[slot * (STAGE / 16) + r * 32];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t be[TB], bo[TB];
#pragma unroll
                    for (int t = 0; t < TB; ++t) {
                        const uint32_t px = word(x[t], j);
                        be[t] = (px << 4) & 0xF0F0F0F0u;
                        bo[t] = px & 0xF0F0F0F0u;
                    }
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const uint32_t pl = word(w[2 * m], j), ph = word(w[2 * m + 1], j);
                        uint32_t a[4];
                        a[0] = (pl << 4) & 0xF0F0F0F0u;   // row g,     even nibbles
                        a[1] = (ph << 4) & 0xF0F0F0F0u;   // row g + 8, even nibbles
                        a[2] = pl & 0xF0F0F0F0u;          // row g,     odd nibbles
                        a[3] = ph & 0xF0F0F0F0u;          // row g + 8, odd nibbles
#pragma unroll
                        for (int t = 0; t < TB; ++t) mma_s8<A_UNSIGNED>(acc[m][t], a, be[t], bo[t]);
                    }
                }
                issue(slot);   // after the math that consumed the slot
                slot = slot + 1 == DEPTH ? 0 : slot + 1;
            }
        };
        if (has_steps) {
            if (NT == 1 || NT > 4 || tb >= NT) run_steps(std::integral_constant<int, NT>{});
            else if (tb <= 1) run_steps(std::integral_constant<int, 1>{});
            else if (tb == 2) run_steps(std::integral_constant<int, (NT >= 2 ? 2 : NT)>{});
            else run_steps(std::integral_constant<int, (NT >= 3 ? 3 : NT)>{});
        }
        if (RED_BUFS == 1) group_sync();   // the previous block's sums have been read
        int *rb = red + (size_t)parity * KW * MT * NT * 128;
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) rb[(((kw * MT + m) * NT + t) * 4 + i) * 32 + lane] = acc[m][t][i];
        group_sync();
        // fragment slot i of lane (g, q) in m-tile m: weight row 16 m + g + 8 * (i >> 1), token 2 * q + (i & 1) of its
        // block.  With two buffers the one written two blocks later is this one: the barrier in between orders it.
        if (SWIGLU) {
            for (int idx = gtid; idx < NT * 128; idx += KW * 32) {
                const int l = idx & 31, i = (idx >> 5) & 3, t = idx >> 7;
                if (t >= tb) continue;
                int sg = 0, su = 0;
#pragma unroll
                for (int w = 0; w < KW; ++w) {
                    sg += rb[(((w * MT + 0) * NT + t) * 4 + i) * 32 + l];
                    su += rb[(((w * MT + 1) * NT + t) * 4 + i) * 32 + l];
                }
                const uint32_t n = cur.n0 + (l >> 2) + 8 * (i >> 1);
                const uint32_t mm = cur.x_row0 + 8 * t + 2 * (l & 3) + (i & 1);
                if (n < N && mm < cur.x_end) {
                    const __half gv = ep.dequant(mm, n, sg >> 8, 2 * N), uv = ep.dequant(mm, n + N, su >> 8, 2 * N);
                    const float gf = __half2float(gv);
                    const __half sv = __float2half(gf / (1.f + expf(-gf)));
                    ep.out[(size_t)mm * N + n] = __float2half(__half2float(sv) * __half2float(uv));
                }
            }
        } else
        for (int idx = gtid; idx < MT * NT * 128; idx += KW * 32) {
            const int l = idx & 31, i = (idx >> 5) & 3, t = (idx >> 7) % NT, m = idx / (NT * 128);
            if (t >= tb) continue;
            int sum = 0;
#pragma unroll
            for (int w = 0; w < KW; ++w) sum += rb[(((w * MT + m) * NT + t) * 4 + i) * 32 + l];
            const uint32_t n = cur.n0 + 16 * m + (l >> 2) + 8 * (i >> 1);
            const uint32_t mm = cur.x_row0 + 8 * t + 2 * (l & 3) + (i & 1);
            if (n < N && mm < cur.x_end) ep.store(mm, n, sum >> 8, N);
        }
        cur = nxt;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
}

}  // namespace

// Warps that share one row block.  Two (four blocks in flight per CTA) pays when there are enough blocks to
// occupy every warp group of the grid and K is short, so that the per-block reduction and epilogue
// would otherwise weigh as much as the block's own steps; eight otherwise.
static int skinny_kw(int64_t blocks, int64_t K, int sm_count, bool grouped = false) {
    // measured: dense launches lose with two (too few blocks for four groups per CTA); the MoE gate/up shape
    // (8 experts x 14336 rows, K = 4096) gains 5 %
    return grouped && K <= 8192 && blocks >= 8ll * sm_count ? 2 : 8;
}

static int launch_skinny(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                         const Epilogue &ep, const int32_t *row_off, int num_experts, cudaStream_t st) {
    SR_REQUIRE(aligned16(A) && aligned16(B), SR_ERR_INVALID, "matmul: operands must be 16-byte aligned");
    SR_REQUIRE(K % 32 == 0, SR_ERR_INVALID, "matmul: K = %lld must be a multiple of 32", (long long)K);
    const int sm_count = current_sm_count();
    const bool grouped = row_off != nullptr;
    // grouped launches: 32 rows per pass (an expert with more rows streams its weights again for the rest)
    const int nt = grouped ? 4 : (M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8)));
    // two m-tiles per warp step when there are enough row blocks to keep every SM busy and the sums fit
    const int mt = (nt <= 4 && (N >= 8192 || (N >= 4096 && nt >= 2))) ? 2 : 1;   // measured crossover
    const int64_t blocks = cdiv<int64_t>(N, SK_ROWS * mt) * (grouped ? num_experts : 1);
    // warps per row block: see skinny_kw()
    const int kw = skinny_kw(blocks, K, sm_count, grouped);
    const int groups = SK_WARPS / kw;
    // two CTAs per SM, three when shared memory allows (one token block, one m-tile: 73 KB per CTA): a few more slots
    // turn "two blocks one after the other" into "one block each" for the 300 .. 440 block shapes (a fused q/k/v).
    // The row blocks are dealt round-robin to the warp groups, so shrink the grid to even the deal out.
    const int per_sm = !grouped && skinny_smem(nt, mt) * 3 + 3 * 1024 <= 227 * 1024 ? 3 : 2;
    int64_t ctas = per_sm * (int64_t)sm_count;
    if (blocks < ctas * groups) ctas = cdiv<int64_t>(blocks, groups);
    // (grouped launches keep every CTA slot: measured 6 % faster on the MoE decode stack than the even deal)
    else if (!grouped) ctas = cdiv<int64_t>(blocks, cdiv<int64_t>(blocks, ctas * groups) * groups);
    const unsigned grid = (unsigned)ctas;
#define SR_SK_KW(NT, MT, GR, KWV)                                                                              \
    do {                                                                                                       \
        auto kfn = a_unsigned ? gemm_skinny_kernel<NT, MT, true, GR, false, KWV>                               \
                              : gemm_skinny_kernel<NT, MT, false, GR, false, KWV>;                             \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                                             (int)skinny_smem(NT, MT));                                        \
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "matmul: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        launch_pdl(kfn, dim3(grid), dim3(SK_WARPS * 32), skinny_smem(NT, MT), st, A, B, (uint32_t)M, (uint32_t)N,   \
                   (uint32_t)K, row_off, num_experts, ep);                                                     \
    } while (0)
#define SR_SK(NT, MT, GR)                                                                                      \
    do {                                                                                                       \
        if (kw == 2) SR_SK_KW(NT, MT, GR, 2);                                                                  \
        else SR_SK_KW(NT, MT, GR, 8);                                                                          \
    } while (0)
    if (grouped) {
        if (mt == 2) SR_SK(4, 2, true);
        else SR_SK(4, 1, true);
    } else if (mt == 2) {
        if (nt == 1) SR_SK(1, 2, false);
        else if (nt == 2) SR_SK(2, 2, false);
        else SR_SK(4, 2, false);
    } else {
        if (nt == 1) SR_SK(1, 1, false);
        else if (nt == 2) SR_SK(2, 1, false);
        else if (nt == 4) SR_SK(4, 1, false);
        else SR_SK_KW(8, 1, false, 8);
    }
#undef SR_SK_KW
#undef SR_SK
    return check_launch("gemm_skinny");
}

// gate/up pair + SwiGLU: B = [2N, K/2] (gate rows then up rows), ep.w_scale = [2N], ep.out = [M, N]
int launch_gemm_skinny_swiglu(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                              const Epilogue &ep, cudaStream_t st) {
    SR_REQUIRE(M >= 1 && M <= 32, SR_ERR_UNSUPPORTED, "w4a4_swiglu: the fused kernel takes at most 32 rows");
    SR_REQUIRE(aligned16(A) && aligned16(B), SR_ERR_INVALID, "w4a4_swiglu: operands must be 16-byte aligned");
    SR_REQUIRE(K % 32 == 0, SR_ERR_INVALID, "w4a4_swiglu: K = %lld must be a multiple of 32", (long long)K);
    SR_REQUIRE(ep.mode == 1 && !ep.expert_ids, SR_ERR_INVALID, "w4a4_swiglu: dense dequant epilogue only");
    const int sm_count = current_sm_count();
    const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
    const int64_t blocks = cdiv<int64_t>(N, SK_ROWS);
    const int kw = skinny_kw(blocks, K, sm_count);
    const int groups = SK_WARPS / kw;
    int64_t ctas = 2 * (int64_t)sm_count;
    if (blocks < ctas * groups) ctas = cdiv<int64_t>(blocks, groups);
    else ctas = cdiv<int64_t>(blocks, cdiv<int64_t>(blocks, ctas * groups) * groups);
    const unsigned grid = (unsigned)ctas;
#define SR_SKS_KW(NT, KWV)                                                                                     \
    do {                                                                                                       \
        auto kfn = a_unsigned ? gemm_skinny_kernel<NT, 2, true, false, true, KWV>                              \
                              : gemm_skinny_kernel<NT, 2, false, false, true, KWV>;                            \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                                             (int)skinny_smem(NT, 2));                                         \
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "w4a4_swiglu: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        launch_pdl(kfn, dim3(grid), dim3(SK_WARPS * 32), skinny_smem(NT, 2), st, A, B, (uint32_t)M, (uint32_t)N,    \
                   (uint32_t)K, (const int32_t *)nullptr, 0, ep);                                              \
    } while (0)
#define SR_SKS(NT)                                                                                             \
    do {                                                                                                       \
        if (kw == 2) SR_SKS_KW(NT, 2);                                                                         \
        else SR_SKS_KW(NT, 8);                                                                                 \
    } while (0)
    if (nt == 1) SR_SKS(1);
    else if (nt == 2) SR_SKS(2);
    else SR_SKS(4);
#undef SR_SKS
#undef SR_SKS_KW
    return check_launch("gemm_skinny_swiglu");
}

int launch_gemm_skinny(const uint8_t *A, const uint8_t *B, int64_t M, int64_t N, int64_t K, bool a_unsigned,
                       const Epilogue &ep, cudaStream_t st) {
    SR_REQUIRE(M >= 1 && M <= 64, SR_ERR_UNSUPPORTED, "matmul: the decode kernel takes at most 64 rows");
    return launch_skinny(A, B, M, N, K, a_unsigned, ep, nullptr, 0, st);
}

int launch_gemm_skinny_grouped(const uint8_t *A, const uint8_t *B, int64_t rows, int64_t N, int64_t K, bool a_unsigned,
                               const Epilogue &ep, const int32_t *row_off, int num_experts, cudaStream_t st) {
    SR_REQUIRE(num_experts >= 1 && num_experts <= SK_MAX_EXPERTS, SR_ERR_UNSUPPORTED,
               "grouped_linear: at most %d experts", SK_MAX_EXPERTS);
    SR_REQUIRE((int64_t)num_experts * N < (1ll << 31) && rows < (1ll << 31), SR_ERR_UNSUPPORTED,
               "grouped_linear: size out of range");
    return launch_skinny(A, B, rows, N, K, a_unsigned, ep, row_off, num_experts, st);
}

}  // namespace sr
