// Split-KV GQA decode attention over the int4 paged cache, with both products on the tensor cores.
//
// Replaces kernels/flashinfer.cu:11-106 + include/flashinfer/decode.cuh:481-751 (one query token per
// request against a quantized paged cache) with the same workspace format as the CUDA-core kernel in
// kv_cache.cu: per (request, q head, chunk) 128 unnormalised outputs, the running maximum and the sum.
//
// grid (batch, kv heads, chunks), 8 or 4 warps; a warp takes blocks of 16 cached tokens (block index
// = warp, warp + warps, ... inside the chunk's range) and keeps the flash-decoding state of all q heads
// of the group (rows of an m16 tile; rows >= G stay zero).
//
// The 4-bit codes never become numbers on the CUDA cores.  A code n masked into the low bits of an
// fp16 lane IS the subnormal n * 2^-24, which mma.sync.m16n8k16 multiplies exactly; the affine
// dequantisation is applied around the products:
//   scores  x_t = (s_t 2^24) (q' . c_t 2^-24) - z_t sum(q')            (q' = q * log2(e) / sqrt(d))
//   output  O_d = 2^24 sum_t (p_t vs_t) (c_td 2^-24) - sum_t p_t vz_t
// K operand: lane (g, qd) loads bytes 16 qd .. 16 qd + 15 of token g's row, (w >> 4i) & 0x000F000F
// are the fp16 pairs (dims i, i + 4 of a word); the permutation of the head dimension is baked into
// the q fragments.  V operand: pairs run over tokens, so the rows of tokens 2 qd and 2 qd + 1 are
// merged byte-wise, (A & 0x0F..) | ((B << 4) & 0xF0..), and a byte broadcast + mask 0x00F0000F gives
// the pair (n_A 2^-24, n_B 2^-20); the factor 16 is taken off p for the odd token.  That product
// runs transposed (dims x heads, 8 MMAs per 16 tokens): the probabilities of the score tile are
// already in the layout of its second operand, and the accumulator has no padded rows.
#include "kv_cache.cuh"
#include <cfloat>

namespace sr {

namespace {

// Warps per CTA: 8 (two CTAs per SM: the step is a chain of dependent instructions and the schedulers need warps to
// switch between) unless the grid has more CTAs than fit the GPU at two per SM: then 4 warps and four CTAs per SM, so
// that large batches still run as one wave.
constexpr int DT_BLOCK = 16;   // cached tokens per warp iteration
constexpr int DT_STAGE_BYTES = 3072;   // per warp and block: 2 KB of codes + 1 KB of parameter pairs (tokens repeat across lanes)
__host__ __device__ constexpr int dt_depth(int) { return 3; }   // blocks in flight per warp: two 8-warp or four 4-warp CTAs and their rings fit one SM
__host__ __device__ constexpr int dt_ring_bytes(int warps) { return warps * dt_depth(warps) * DT_STAGE_BYTES; }

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// logical head dimension of physical operand slot (k-step ks, quad lane qd, register reg, half h) of the K product
__device__ __forceinline__ int k_dim(int ks, int qd, int reg, int h) {
    const int w = ks >> 1, i = 2 * (ks & 1) + reg;
    return 32 * qd + 8 * w + i + 4 * h;
}

template <int G, int DT_WARPS>
__global__ void __launch_bounds__(DT_WARPS * 32, DT_WARPS == 8 ? 2 : 4)
decode_tc_kernel(const __half *__restrict__ q, PagedKV kv, __half *__restrict__ o, float *__restrict__ tmp,
                 uint32_t num_chunks, int had_q, float had_scale, int32_t *__restrict__ counters, int cluster_merge,
                 RopeIn rope) {
    pdl_trigger();   // the next kernel of the stream may be scheduled early; this one is launched without the attribute
    pdl_wait();
    constexpr int DT_DEPTH = dt_depth(DT_WARPS);
    const uint32_t b = blockIdx.x, hk = blockIdx.y, chunk = blockIdx.z;
    const uint32_t hq_total = gridDim.y * G;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, qd = lane & 3;

    extern __shared__ __align__(16) uint8_t dt_smem[];
    // padded so that the gathers below are bank-conflict free: q row pitch 132 with one extra word per 32 dims
    // (lane (g, qd) reads row g, dims 32 qd + c); output rows hold dim d at d + 2 (d / 16), pitch 148
    __shared__ float sh_q[G][132];
    __shared__ float sh_o[DT_WARPS][G][148];
    __shared__ float sh_md[DT_WARPS][G][2];
    __shared__ float cl_part[G][HD + 4];      // cluster merge: this chunk's state per head (o[128], m, d), read by the other CTAs

    const bool fused = rope.k != nullptr;     // this launch also applies the rotary embedding and appends the new K / V
    // ---- q (optionally Hadamard-rotated, kv_cache.py:157-158), one warp per q head
    const float sm_scale = 1.44269504088896340736f * 0.08838834764831845f;  // log2(e) / sqrt(128)
    for (int gg = warp; gg < G; gg += DT_WARPS) {
        const uint32_t hq = hk * G + gg;
        // fused form: the projection's own q (possibly a column range), rotary embedding here, rounded to fp16 as the
        // separate launch would store it
        const __half *qp = fused ? rope.q + (size_t)b * rope.q_stride + (size_t)hq * HD + lane * 4
                                 : q + ((size_t)b * hq_total + hq) * HD + lane * 4;
        const uint2 raw = *reinterpret_cast<const uint2 *>(qp);
        __half hq4[4];
        *reinterpret_cast<uint2 *>(hq4) = raw;
        if (fused) rope_vec(hq4, raw, rope.cosv, rope.sinv, (size_t)(rope.cos_seqs == 1 ? 0 : b) * HD + lane * 4, lane);
        float a[4] = {__half2float(hq4[0]), __half2float(hq4[1]), __half2float(hq4[2]), __half2float(hq4[3])};
        if (had_q) {
            float t0 = a[0] + a[1], t1 = a[0] - a[1], t2 = a[2] + a[3], t3 = a[2] - a[3];
            a[0] = t0 + t2; a[1] = t1 + t3; a[2] = t0 - t2; a[3] = t1 - t3;
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float ot = __shfl_xor_sync(0xffffffffu, a[j], m);
                    a[j] = (lane & m) ? (ot - a[j]) : (a[j] + ot);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) a[j] = __half2float(__float2half_rn(a[j] * had_scale));
        }
        // the products take q' as fp16: round once here so that sum(q') below is the sum of what is multiplied
#pragma unroll
        for (int j = 0; j < 4; ++j) sh_q[gg][lane * 4 + j + (lane >> 3)] = __half2float(__float2half_rn(a[j] * sm_scale));
    }
    __syncthreads();

    // A fragments of q' (rows g < G; rows g + 8 are zero) in the K product's dimension order, and sum(q') per head
    uint32_t qa[8][2];
    float qsum = 0.f;
    {
        const int gq = g < G ? g : 0;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int reg = 0; reg < 2; ++reg) {
                const float lo = sh_q[gq][k_dim(ks, qd, reg, 0) + qd], hi = sh_q[gq][k_dim(ks, qd, reg, 1) + qd];
                qa[ks][reg] = g < G ? pack_h2(lo, hi) : 0u;
            }
        float s = 0.f;
        for (int j = 0; j < 32; ++j) s += sh_q[gq][qd * 33 + j];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        qsum = s;
    }

    // ---- this chunk's token range: an equal share of the request's 16-token blocks (pages are too coarse a unit: nine
    // pages over four chunks would leave one chunk empty), so every chunk count balances
    const uint32_t page_begin = (uint32_t)kv.indptr[b], page_end = (uint32_t)kv.indptr[b + 1];
    const uint32_t pages_total = page_end - page_begin;
    const uint32_t last_valid = (uint32_t)kv.last_page_offset[b];
    const uint32_t blocks_per_page = kv.page_size / DT_BLOCK;
    const uint32_t total_blocks =
        pages_total > 0 ? (pages_total - 1) * blocks_per_page + (last_valid + DT_BLOCK - 1) / DT_BLOCK : 0u;
    const uint32_t per_chunk = (total_blocks + num_chunks - 1) / num_chunks;
    const uint32_t cb_begin = min(chunk * per_chunk, total_blocks), cb_end = min(cb_begin + per_chunk, total_blocks);
    const uint32_t num_blocks = cb_end - cb_begin;
    if (fused) {
        // The new token's K and V go into their slot (the last one of the request) before anybody reads it: only the
        // chunk that owns the last block does, and it is this CTA that writes it.  Warp 0: K (rotary embedding, head_dim
        // rotation, quantizer), warp 1: V (quantizer): the arithmetic of rope_kv_append_kernel.
        const bool owner = total_blocks > 0 && cb_begin <= total_blocks - 1 && total_blocks - 1 < cb_end;
        if (owner && warp < 2) {
            const __half *src = warp == 0 ? rope.k + (size_t)b * rope.k_stride : rope.v + (size_t)b * rope.v_stride;
            const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(src + (size_t)hk * HD + lane * 4));
            __half h[4];
            *reinterpret_cast<uint2 *>(h) = raw;
            if (warp == 0) rope_vec(h, raw, rope.cosv, rope.sinv, (size_t)(rope.cos_seqs == 1 ? 0 : b) * HD + lane * 4, lane);
            kv_quant_store(kv, h, (uint32_t)warp, warp == 0 && rope.had_k, had_scale, b, hk, kv.seq_len(b) - 1, lane);
        }
        __syncthreads();      // the stores above are visible to this CTA's copies below
    }

    float m_run = -5e4f, d_run = 0.f, z_run = 0.f;   // head g: running max (quad-uniform), this lane's part of sum p and sum p vz
    // O^T accumulators: m-tile j = byte j of the lane's eight V bytes; slot 0,1: dim 16 g + 2 j, heads 2 qd, 2 qd + 1;
    // slot 2,3: dim 16 g + 2 j + 1
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

    struct Stage {
        uint4 k[2];      // K rows of tokens g and 8 + g, bytes 16 qd ..
        uint2 v[4];      // V rows of tokens 2 qd, 2 qd + 1, 8 + 2 qd, 9 + 2 qd, bytes 8 g ..
        uint2 kp[2];     // (scale, zero) fp16 pairs of K for tokens (2 qd, 2 qd + 1) and (8 + 2 qd, 9 + 2 qd)
        uint2 vp[2];
        uint32_t valid;  // tokens of the block that exist
    };
    // The rows travel through a cp.async ring in shared memory, DT_DEPTH blocks ahead of the math.  Every lane
    // copies exactly the bytes its own fragments need into slots nobody else touches: no barrier guards the ring.
    // ring[warp][stage]: 64 x 16 B (K), then 128 x 8 B (V), then 128 x 8 B (parameters), lane-interleaved.
    uint8_t *ring = dt_smem + (size_t)warp * DT_DEPTH * DT_STAGE_BYTES;
    const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring);
    // The copies run DT_DEPTH blocks ahead of the math along the warp's blocks (every DT_WARPS-th of the chunk).  A cursor
    // (block, page, offset in the page, base of the page's K and V rows) moves with them, so that a step costs neither a
    // division nor a look-up in the page table unless the page changes.
    const uint32_t seq_tokens = total_blocks > 0 ? (pages_total - 1) * kv.page_size + last_valid : 0u;
    uint32_t i_gb = cb_begin + warp, i_pi = i_gb / blocks_per_page, i_e0 = (i_gb % blocks_per_page) * DT_BLOCK;
    size_t i_kb = 0, i_vb = 0;
    auto page_bases = [&]() {
        if (i_gb < cb_end) {
            const uint32_t page = (uint32_t)kv.indices[page_begin + i_pi];
            i_kb = kv.vec_index(page, 0, hk, 0);
            i_vb = kv.vec_index(page, 1, hk, 0);
        }
    };
    page_bases();
    auto issue = [&](int slot) {
        if (i_gb < cb_end) {
            const size_t kbase = i_kb + i_e0, vbase = i_vb + i_e0;
            // rows past the end of a partially filled page belong to the same allocation: they are read and masked
            const uint8_t *krow = kv.data + (kbase + g) * 64 + qd * 16;
            const uint8_t *vrow = kv.data + (vbase + 2 * qd) * 64 + g * 8;
            const uint32_t dst = ring_u32 + (uint32_t)slot * DT_STAGE_BYTES;
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (t * 32 + lane) * 16), "l"(krow + t * 512) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + 1024 + (2 * t * 32 + lane) * 8), "l"(vrow + t * 512) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + 1024 + ((2 * t + 1) * 32 + lane) * 8), "l"(vrow + t * 512 + 64) : "memory");
                // block bases are multiples of 16 vectors: the pair of 4-byte parameters is 8-byte aligned
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + 2048 + (t * 32 + lane) * 8), "l"(kv.param + kbase + 8 * t + 2 * qd) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + 2048 + ((2 + t) * 32 + lane) * 8), "l"(kv.param + vbase + 8 * t + 2 * qd) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        i_gb += DT_WARPS;
        i_e0 += DT_WARPS * DT_BLOCK;
        if (i_e0 >= kv.page_size) {
            do {
                i_e0 -= kv.page_size;
                ++i_pi;
            } while (i_e0 >= kv.page_size);
            page_bases();
        }
    };
    auto fetch = [&](uint32_t blk, int slot, Stage &s) {
        const uint32_t t0 = (cb_begin + blk) * DT_BLOCK;      // first token of the block, counted along the request
        s.valid = seq_tokens > t0 ? min(seq_tokens - t0, (uint32_t)DT_BLOCK) : 0u;
        const uint8_t *src = ring + (size_t)slot * DT_STAGE_BYTES;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            s.k[t] = *reinterpret_cast<const uint4 *>(src + (t * 32 + lane) * 16);
            s.v[2 * t] = *reinterpret_cast<const uint2 *>(src + 1024 + (2 * t * 32 + lane) * 8);
            s.v[2 * t + 1] = *reinterpret_cast<const uint2 *>(src + 1024 + ((2 * t + 1) * 32 + lane) * 8);
            s.kp[t] = *reinterpret_cast<const uint2 *>(src + 2048 + (t * 32 + lane) * 8);
            s.vp[t] = *reinterpret_cast<const uint2 *>(src + 2048 + ((2 + t) * 32 + lane) * 8);
        }
    };

    auto process = [&](const Stage &cur) {
        // ---- scores of 16 tokens: two n-tiles of 8 tokens, 8 k-steps over the head dimension
        float sc[2][4];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            // two accumulators per tile (even and odd k-steps) halve the chain of dependent MMAs
            float s2[4] = {0.f, 0.f, 0.f, 0.f};
            sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.f;
            const uint32_t w[4] = {cur.k[t].x, cur.k[t].y, cur.k[t].z, cur.k[t].w};
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t word = w[ks >> 1];
                const int i = 2 * (ks & 1);
                const uint32_t b0 = (word >> (4 * i)) & 0x000F000Fu, b1 = (word >> (4 * i + 4)) & 0x000F000Fu;
                if (ks & 1) mma_f16(s2, qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
                else mma_f16(sc[t], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
            }
            sc[t][0] += s2[0];
            sc[t][1] += s2[1];
        }
        // lane holds head g, tokens 2 qd, 2 qd + 1 (tile 0) and 8 + 2 qd, 9 + 2 qd (tile 1)
        float x[4], kz[4], vs[4], vz[4];
        float bmax = -5e4f;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const float2 k0 = __half22float2(*reinterpret_cast<const __half2 *>(&cur.kp[t].x));
            const float2 k1 = __half22float2(*reinterpret_cast<const __half2 *>(&cur.kp[t].y));
            const float2 v0 = __half22float2(*reinterpret_cast<const __half2 *>(&cur.vp[t].x));
            const float2 v1 = __half22float2(*reinterpret_cast<const __half2 *>(&cur.vp[t].y));
            x[2 * t] = sc[t][0] * (k0.x * 16777216.f);
            x[2 * t + 1] = sc[t][1] * (k1.x * 16777216.f);
            kz[2 * t] = k0.y;
            kz[2 * t + 1] = k1.y;
            vs[2 * t] = v0.x;
            vs[2 * t + 1] = v1.x * 0.0625f;   // odd tokens carry their codes 16 times too large (see the V operand)
            vz[2 * t] = v0.y;
            vz[2 * t + 1] = v1.y;
        }
        bool live[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            live[t] = (uint32_t)(8 * (t >> 1) + 2 * qd + (t & 1)) < cur.valid;
            x[t] = live[t] ? x[t] - kz[t] * qsum : -5e4f;
            bmax = fmaxf(bmax, x[t]);
        }
        bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
        bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 2));
        const float m_new = fmaxf(m_run, bmax);
        // the running maximum moves in few blocks: the rescale of the accumulators is skipped when no lane needs it
        if (__any_sync(0xffffffffu, m_new > m_run)) {
            const float alpha = ex2(m_run - m_new);
            d_run *= alpha;
            z_run *= alpha;
            // the accumulator columns of this lane are heads 2 qd and 2 qd + 1: their factors live in lanes g = head
            const float a_lo = __shfl_sync(0xffffffffu, alpha, (2 * qd) << 2);
            const float a_hi = __shfl_sync(0xffffffffu, alpha, (2 * qd + 1) << 2);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc[j][0] *= a_lo;
                acc[j][1] *= a_hi;
                acc[j][2] *= a_lo;
                acc[j][3] *= a_hi;
            }
            m_run = m_new;
        }
        uint32_t pb[2];
        {
            float pv[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                // slots past the end of a page hold whatever was there before: their parameters are not numbers to trust
                const float p = live[t] ? ex2(x[t] - m_run) : 0.f;
                d_run += p;
                z_run = fmaf(p, live[t] ? vz[t] : 0.f, z_run);
                pv[t] = live[t] ? p * vs[t] : 0.f;
            }
            pb[0] = pack_h2(pv[0], pv[1]);
            pb[1] = pack_h2(pv[2], pv[3]);
        }
        // ---- output, transposed: O^T[dims x heads] += V^T[dims x tokens] P^T[tokens x heads]; 8 m-tiles of 16 dims.
        // bytes of the merged words = (code of the even token, code of the odd token << 4)
        uint32_t even[2][2], odd[2][2];   // [token pair][word]
#pragma unroll
        for (int tp = 0; tp < 2; ++tp) {
            const uint32_t ax = cur.v[2 * tp].x, ay = cur.v[2 * tp].y, bx = cur.v[2 * tp + 1].x, by = cur.v[2 * tp + 1].y;
            even[tp][0] = (ax & 0x0F0F0F0Fu) | ((bx << 4) & 0xF0F0F0F0u);
            even[tp][1] = (ay & 0x0F0F0F0Fu) | ((by << 4) & 0xF0F0F0F0u);
            odd[tp][0] = ((ax >> 4) & 0x0F0F0F0Fu) | (bx & 0xF0F0F0F0u);
            odd[tp][1] = ((ay >> 4) & 0x0F0F0F0Fu) | (by & 0xF0F0F0F0u);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int byte = j & 3, word = j >> 2;
            const uint32_t sel = (uint32_t)(byte | (byte << 8));
            const uint32_t a0 = __byte_perm(even[0][word], even[0][word], sel) & 0x00F0000Fu;   // dim 16 g + 2 j,     tokens 2 qd, 2 qd + 1
            const uint32_t a1 = __byte_perm(odd[0][word], odd[0][word], sel) & 0x00F0000Fu;     // dim 16 g + 2 j + 1
            const uint32_t a2 = __byte_perm(even[1][word], even[1][word], sel) & 0x00F0000Fu;   // tokens 8 + 2 qd, 9 + 2 qd
            const uint32_t a3 = __byte_perm(odd[1][word], odd[1][word], sel) & 0x00F0000Fu;
            mma_f16(acc[j], a0, a1, a2, a3, pb[0], pb[1]);
        }
    };

#pragma unroll 1
    for (int d = 0; d < DT_DEPTH; ++d) issue(d);
    int slot = 0;
#pragma unroll 1
    for (uint32_t blk = warp; blk < num_blocks; blk += DT_WARPS) {
        asm volatile("cp.async.wait_group %0;" ::"n"(DT_DEPTH - 1) : "memory");
        Stage st;
        fetch(blk, slot, st);
        process(st);
        issue(slot);   // after the math that consumed the slot
        slot = slot + 1 == DT_DEPTH ? 0 : slot + 1;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");

    // ---- fold the warp's state: sums across the quad, the 2^24 of the subnormal codes, the zero points
    d_run += __shfl_xor_sync(0xffffffffu, d_run, 1);
    d_run += __shfl_xor_sync(0xffffffffu, d_run, 2);
    z_run += __shfl_xor_sync(0xffffffffu, z_run, 1);
    z_run += __shfl_xor_sync(0xffffffffu, z_run, 2);
    {
        const float z_lo = __shfl_sync(0xffffffffu, z_run, (2 * qd) << 2);
        const float z_hi = __shfl_sync(0xffffffffu, z_run, (2 * qd + 1) << 2);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int at = 18 * g + 2 * j;   // dims 16 g + 2 j and + 1, skewed
            if (2 * qd < G)
                *reinterpret_cast<float2 *>(&sh_o[warp][2 * qd][at]) =
                    make_float2(acc[j][0] * 16777216.f - z_lo, acc[j][2] * 16777216.f - z_lo);
            if (2 * qd + 1 < G)
                *reinterpret_cast<float2 *>(&sh_o[warp][2 * qd + 1][at]) =
                    make_float2(acc[j][1] * 16777216.f - z_hi, acc[j][3] * 16777216.f - z_hi);
        }
        if (g < G && qd == 0) {
            sh_md[warp][g][0] = m_run;
            sh_md[warp][g][1] = d_run;
        }
    }
    __syncthreads();
    // thread t < HD finalises dim t for every head of the group
    for (int gg = 0; gg < G && tid < HD; ++gg) {
        float mm = sh_md[0][gg][0];
#pragma unroll
        for (int w = 1; w < DT_WARPS; ++w) mm = fmaxf(mm, sh_md[w][gg][0]);
        float dd = 0.f, oo = 0.f;
#pragma unroll
        for (int w = 0; w < DT_WARPS; ++w) {
            const float scl = ex2(sh_md[w][gg][0] - mm);
            dd += sh_md[w][gg][1] * scl;
            oo += sh_o[w][gg][tid + 2 * (tid >> 4)] * scl;
        }
        const uint32_t hq = hk * G + gg;
        if (num_chunks == 1) {
            o[((size_t)b * hq_total + hq) * HD + tid] = __float2half_rn(__fdividef(oo, dd));
        } else if (cluster_merge) {
            cl_part[gg][tid] = oo;
            if (tid == 0) {
                cl_part[gg][HD] = mm;
                cl_part[gg][HD + 1] = dd;
            }
        } else {
            float *dst = tmp + (((size_t)b * hq_total + hq) * num_chunks + chunk) * (HD + 4);
            dst[tid] = oo;
            if (tid == 0) {
                dst[HD] = mm;
                dst[HD + 1] = dd;
            }
        }
    }
    // ---- merge across chunks inside the cluster: the CTAs of one (request, KV head) are one cluster along z, every chunk's
    // state stays in its CTA's shared memory and head gg is finalised by the CTA of rank gg % chunks, which reads the
    // chunks' states in chunk order through distributed shared memory: the arithmetic and the order of
    // decode_merge_kernel, without its launch and without the round trip of the partial states through memory.
    if (cluster_merge && num_chunks > 1) {
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        const uint32_t mine = (uint32_t)__cvta_generic_to_shared(&cl_part[0][0]);
        auto peer_ld = [&](uint32_t c, uint32_t idx) {
            float v;
            asm volatile(
                "{\n\t.reg .b32 remaddr;\n\t"
                "mapa.shared::cluster.u32 remaddr, %1, %2;\n\t"
                "ld.shared::cluster.f32 %0, [remaddr];\n\t}"
                : "=f"(v)
                : "r"(mine + idx * 4u), "r"(c)
                : "memory");
            return v;
        };
        for (int gg = 0; gg < G && tid < HD; ++gg) {
            if ((uint32_t)gg % num_chunks != chunk) continue;
            const uint32_t hq = hk * G + gg, at = (uint32_t)gg * (HD + 4);
            // all remote loads first (at most eight chunks in a cluster), so that they are in flight together
            float mc[8], dc[8], oc[8];
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c) {
                const bool have = c < num_chunks;
                mc[c] = have ? peer_ld(c, at + HD) : -5e4f;
                dc[c] = have ? peer_ld(c, at + HD + 1) : 0.f;
                oc[c] = have ? peer_ld(c, at + tid) : 0.f;
            }
            float mm = -5e4f;
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c)
                if (c < num_chunks) mm = fmaxf(mm, mc[c]);
            float dd = 0.f, oo = 0.f;
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c)
                if (c < num_chunks) {
                    const float sc = ex2(mc[c] - mm);
                    dd += dc[c] * sc;
                    oo += oc[c] * sc;
                }
            o[((size_t)b * hq_total + hq) * HD + tid] = __float2half_rn(__fdividef(oo, dd));
        }
        // no CTA leaves while another one may still read its state
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        return;
    }
    // ---- merge across chunks by whichever CTA of this (request, KV head) finishes last: the arithmetic and the
    // chunk order of decode_merge_kernel, without its launch.  counters[b * kv_heads + hk] starts at zero and is
    // put back to zero by the CTA that merges, so the buffer needs no reset between calls (or graph replays).
    if (counters != nullptr && num_chunks > 1) {
        __shared__ int is_last;
        __threadfence();      // this CTA's partial state is visible device-wide before its arrival is counted
        __syncthreads();
        if (tid == 0) {
            int32_t *cnt = counters + (size_t)b * gridDim.y + hk;
            const int prev = atomicAdd(cnt, 1);
            is_last = prev == (int)num_chunks - 1;
            if (is_last) *cnt = 0;
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            for (int gg = 0; gg < G && tid < HD; ++gg) {
                const uint32_t hq = hk * G + gg;
                const float *src = tmp + ((size_t)b * hq_total + hq) * num_chunks * (HD + 4);
                float mm = -5e4f;
                for (uint32_t c = 0; c < num_chunks; ++c) mm = fmaxf(mm, __ldcg(src + c * (HD + 4) + HD));
                float dd = 0.f, oo = 0.f;
                for (uint32_t c = 0; c < num_chunks; ++c) {
                    const float sc = ex2(__ldcg(src + c * (HD + 4) + HD) - mm);
                    dd += __ldcg(src + c * (HD + 4) + HD + 1) * sc;
                    oo += __ldcg(src + c * (HD + 4) + tid) * sc;
                }
                o[((size_t)b * hq_total + hq) * HD + tid] = __float2half_rn(__fdividef(oo, dd));
            }
        }
    }
}

}  // namespace

// Returns 0 when the kernel does not take the geometry, 1 when it ran and the split-KV states still have to be merged
// (decode_merge_kernel), 2 when nothing is left to do (one chunk, or merged inside the kernel).
int launch_decode_tc(int G, dim3 grid, const __half *q, const PagedKV &kv, __half *o, float *tmp, uint32_t num_chunks,
                     int had_q, float had_scale, cudaStream_t st, int32_t *counters, const RopeIn *rope_in) {
    if (kv.page_size % DT_BLOCK != 0) return 0;
    RopeIn rope = {};
    if (rope_in != nullptr) rope = *rope_in;
    // two or four chunks: the chunks of a (request, KV head) form a cluster and merge in it.  Measured on B200 (batch 8,
    // 8 KV heads, context 2048, launches back to back): clusters of 2 and 4 cost nothing to place and the merge inside
    // them 1.0 us (the separate merge launch: 2.2 us); clusters of 5 and 8 take 3.4 us and more just to be placed.
    bool cluster = counters == nullptr && (num_chunks == 2 || num_chunks == 4);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    // 8 warps per CTA while the whole grid fits the GPU at two CTAs per SM, 4 warps (four CTAs per SM) beyond that
    // (measured, context 1024-2048: batch 128 50.3 against 56.0 us, batch 64 54.2 against 55.6 us)
    const int warps = (size_t)grid.x * grid.y * grid.z > 2 * (size_t)current_sm_count() ? 4 : 8;
    cfg.blockDim = dim3(warps * 32);
    cfg.dynamicSmemBytes = warps == 8 ? dt_ring_bytes(8) : dt_ring_bytes(4);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    // Not launched with programmatic serialization, although the kernel before it is: CTAs that become resident while
    // the projection GEMM still fills every SM are placed wherever one of its CTAs happens to retire first, up to
    // three on one SM and none on others, and the attention then runs at the pace of the crowded SMs.  Measured on
    // B200 (Llama-3-8B, batch 8, context 2100): 2.20 ms per decode step with the attribute, 2.03 ms without.
    if (cluster) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = num_chunks;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
#define SR_DT(GG)                                                                                              \
    do {                                                                                                       \
        auto kfn = warps == 8 ? decode_tc_kernel<GG, 8> : decode_tc_kernel<GG, 4>;                             \
        if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cfg.dynamicSmemBytes) != cudaSuccess) \
            return 0;                                                                                          \
        if (cudaLaunchKernelEx(&cfg, kfn, q, kv, o, tmp, num_chunks, had_q, had_scale, counters, cluster ? 1 : 0, rope) != cudaSuccess) { \
            if (!cluster) return 0;                                                                            \
            (void)cudaGetLastError();        /* a cluster of this size does not fit: plain launch, separate merge */ \
            cluster = false;                                                                                   \
            cfg.numAttrs = na - 1;                                                                             \
            if (cudaLaunchKernelEx(&cfg, kfn, q, kv, o, tmp, num_chunks, had_q, had_scale, counters, 0, rope) != cudaSuccess) \
                return 0;                                                                                      \
        }                                                                                                      \
    } while (0)
    switch (G) {
        case 1: SR_DT(1); break;
        case 2: SR_DT(2); break;
        case 4: SR_DT(4); break;
        case 8: SR_DT(8); break;
        default: return 0;
    }
#undef SR_DT
    return (num_chunks == 1 || cluster || counters != nullptr) ? 2 : 1;
}

}  // namespace sr
