// Fused online rotation + sign + symmetric per-token int4 quantization for rows of
// 14336 = 28 x 512 values (the down_proj input of an 8B model): y = (had28 (x) H_512) x / sqrt(n).
//
// Replaces, in one launch and one pass over HBM, fast_hadamard_transform over the 28 segments,
// the fp16 had28 matmul, the sign multiply and sym_quant_dynamic
// (signrot/functional/hadamard.py:78-87, signrot/nn/hadamard.py:39, signrot/kernels/fused.cu:68-112).
// The rounding points are the reference's: the 512-point sums are fp32, scaled and rounded to
// fp16; the 28-point stage multiplies fp16 values by +-1 and accumulates in fp32 (exactly what an
// fp16 tensor-core matmul does), rounded to fp16 again.
//
// One CTA of 448 threads (14 warps) per row:
//   1. segment k is owned by a half warp (16 threads x 32 values): 32-point transform in
//      registers over index bits {0,1,2,7,8}, a 32 x 16 fp32 transpose through shared memory that
//      only the half warp touches, 16-point transforms over bits {3..6};
//   2. the scaled fp16 values go to shared memory as Z[k][j] (rows padded so that the 2-byte
//      stores and the later 8x8 matrix loads are bank-conflict free);
//   3. Y[32 x 512] = H28 (zero padded to 32 x 32) * Z on mma.sync.m16n8k16 (fp16 in, fp32
//      accumulate): 64 column tiles spread over the 14 warps, the A fragments of H28 and the sign
//      bits of a thread's outputs stay in registers for the whole (persistent) kernel;
//   4. fp16 rounding, sign, row maximum, codes; bytes are staged in shared memory and leave as
//      one 16-byte store per thread.
#include "rotate.cuh"
#include <cfloat>
#include <type_traits>

namespace sr {

namespace {

constexpr int N = 14336, SEG = 512, KH = 28;
constexpr int THREADS = 448;
constexpr int XSEG = 560;      // words per segment in the fp32 exchange buffer (32 rows x pitch 17, padded)
constexpr int PZ = 584;        // halves per row of Z (512 + 4 * 16 skew + pad; PZ/2 = 4 mod 32 words)
constexpr int OUTP = 272;      // bytes per output row in the staging buffer (256 + 16)
constexpr int SMEM_BYTES = KH * XSEG * 4;  // 62720; Z (37376 B) and the staging buffer alias it
constexpr int Z_BYTES = 32 * PZ * 2;

__device__ __forceinline__ int zcol(int j) { return j + 16 * (j >> 7); }

template <typename InT>
__global__ void __launch_bounds__(THREADS, 2)
rotate_quant_had28_kernel(const InT *__restrict__ x, const __half *__restrict__ hadk,
                          const int8_t *__restrict__ sign, const int32_t *__restrict__ expert_ids, uint32_t rows,
                          float scale, float clip, uint8_t *__restrict__ q, __half *__restrict__ q_scale,
                          __half *__restrict__ rotated) {
    extern __shared__ __align__(16) uint8_t smem[];
    float *xbuf = reinterpret_cast<float *>(smem);
    __half *zbuf = reinterpret_cast<__half *>(smem);
    uint8_t *obuf = smem + Z_BYTES;
    __shared__ float red[14];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hw = lane >> 4, u = lane & 15;
    const int seg = 2 * warp + hw;
    const int g = lane >> 2, qd = lane & 3;  // mma fragment coordinates

    // ---- A fragments of H (28 x 28 padded with zeros to 32 x 32), row-major fp16
    uint32_t afr[2][2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int kt = 0; kt < 2; ++kt)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int row = 16 * mt + g + 8 * (r & 1);
                const int col = 16 * kt + 2 * qd + 8 * (r >> 1);
                __half2 h2 = __floats2half2_rn(0.f, 0.f);
                if (row < KH && col < KH) h2.x = hadk[row * KH + col];
                if (row < KH && col + 1 < KH) h2.y = hadk[row * KH + col + 1];
                afr[mt][kt][r] = *reinterpret_cast<uint32_t *>(&h2);
            }
    const int n_tiles = (warp + 56 < 64) ? 5 : 4;  // column tiles warp, warp+14, ...

    // sign bits of this thread's outputs: bit (tile*8 + mt*4 + r) <-> y[16mt + g + 8(r>>1)][8nt + 2qd + (r&1)]
    const bool per_row_sign = sign != nullptr && expert_ids != nullptr;
    uint64_t neg_static = 0;
    auto load_sign = [&](const int8_t *sg) {
        uint64_t m = 0;
        for (int ti = 0; ti < n_tiles; ++ti) {
            const int nt = warp + 14 * ti;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int kp = 16 * mt + g + 8 * (r >> 1);
                    const int j = 8 * nt + 2 * qd + (r & 1);
                    if (kp < KH && sg[kp * SEG + j] < 0) m |= 1ull << (ti * 8 + mt * 4 + r);
                }
        }
        return m;
    };
    if (sign != nullptr && !per_row_sign) neg_static = load_sign(sign);

    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        // ---- 1. 512-point transform of segment `seg`
        u64 vp[16];
        {
            const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * N) + seg * 64 + u;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                Vec16 ld;
                ld.u = __ldg(xr + c * 16);
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    float2 f;
                    if (std::is_same<InT, __half>::value) {
                        f = __half22float2(ld.h2[p]);
                    } else {
                        // bf16 -> fp32 is a shift; x.to(float16) is one packed rounding; widening is exact
                        const float lo = __uint_as_float(ld.w[p] << 16), hi = __uint_as_float(ld.w[p] & 0xFFFF0000u);
                        f = __half22float2(__floats2half2_rn(lo, hi));
                    }
                    vp[c * 4 + p] = pack2(f.x, f.y);
                }
            }
        }
        fwht_pairs<16, 16>(vp);  // bits {0,1,2} (inside a vector) and {7,8} (vector number)
        float *xs = xbuf + seg * XSEG;
#pragma unroll
        for (int a = 0; a < 16; ++a) {
            float lo, hi;
            unpack2(vp[a], lo, hi);
            xs[(2 * a) * 17 + u] = lo;
            xs[(2 * a + 1) * 17 + u] = hi;
        }
        __syncwarp();
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int uu = 0; uu < 16; uu += 2)
                vp[r * 8 + uu / 2] = pack2(xs[(u + 16 * r) * 17 + uu], xs[(u + 16 * r) * 17 + uu + 1]);
        fwht_pairs<16, 8>(vp);  // bits {3..6}: two independent 16-point transforms
        float v[32];
#pragma unroll
        for (int a = 0; a < 16; ++a) unpack2(vp[a], v[2 * a], v[2 * a + 1]);
        __syncthreads();  // every half warp is done with the exchange buffer: Z may overwrite it

        // ---- 2. Z[k][j] = rn_h(sum * scale); element of (r, uu): c = (u >> 3) + 2r, b = u & 7
        {
            __half *zr = zbuf + seg * PZ;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int c = (u >> 3) + 2 * r, b = u & 7;
#pragma unroll
                for (int uu = 0; uu < 16; uu += 2) {
                    // packed rounding (keeps the conversion unit out of the loop)
                    const __half2 h = __floats2half2_rn(v[r * 16 + uu] * scale, v[r * 16 + uu + 1] * scale);
                    zr[zcol(c * 128 + uu * 8 + b)] = __low2half(h);
                    zr[zcol(c * 128 + (uu + 1) * 8 + b)] = __high2half(h);
                }
            }
            // rows 28..31 are the zero padding of the k dimension
            if (tid < 4 * PZ / 8) reinterpret_cast<uint4 *>(zbuf + KH * PZ)[tid] = make_uint4(0, 0, 0, 0);
        }
        __syncthreads();

        // ---- 3. Y = H * Z on the tensor cores, fp16 rounding, sign, row maximum
        uint64_t neg = neg_static;
        if (per_row_sign) neg = load_sign(sign + (size_t)expert_ids[row] * N);
        __half2 y[5][2][2];  // [tile][mt][half: rows g / g+8] = columns (2qd, 2qd+1)
        __half2 amax2 = __floats2half2_rn(0.f, 0.f);
#pragma unroll
        for (int ti = 0; ti < 5; ++ti) {
            if (ti < n_tiles) {
                const int nt = warp + 14 * ti;
                uint32_t b0, b1, b2, b3;
                {
                    const int t = lane >> 3, r = lane & 7;
                    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(zbuf + (8 * t + r) * PZ + zcol(8 * nt));
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                                 : "r"(addr));
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
                    asm volatile(
                        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                        : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
                        : "r"(afr[mt][0][0]), "r"(afr[mt][0][1]), "r"(afr[mt][0][2]), "r"(afr[mt][0][3]), "r"(b0), "r"(b1));
                    asm volatile(
                        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                        : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
                        : "r"(afr[mt][1][0]), "r"(afr[mt][1][1]), "r"(afr[mt][1][2]), "r"(afr[mt][1][3]), "r"(b2), "r"(b3));
                    const uint32_t sb = (uint32_t)(neg >> (ti * 8 + mt * 4)) & 15u;
                    __half2 lo = __floats2half2_rn(c0, c1), hi = __floats2half2_rn(c2, c3);
                    uint32_t lw = *reinterpret_cast<uint32_t *>(&lo), hw_ = *reinterpret_cast<uint32_t *>(&hi);
                    lw ^= ((sb & 1u) << 15) | ((sb & 2u) << 30);
                    hw_ ^= ((sb & 4u) << 13) | ((sb & 8u) << 28);
                    lo = *reinterpret_cast<__half2 *>(&lw);
                    hi = *reinterpret_cast<__half2 *>(&hw_);
                    y[ti][mt][0] = lo;
                    y[ti][mt][1] = hi;
                    amax2 = __hmax2(amax2, __hmax2(__habs2(lo), __habs2(hi)));
                }
            }
        }
        float amax = warp_max(fmaxf(__low2float(amax2), __high2float(amax2)));
        if (lane == 0) red[warp] = amax;
        __syncthreads();
        amax = red[0];
#pragma unroll
        for (int w = 1; w < 14; ++w) amax = fmaxf(amax, red[w]);
        __half s = __float2half(amax / 7.f);
        if (clip != 1.f) s = __float2half(__half2float(s) * clip);
        if (tid == 0) q_scale[row] = s;
        // a zero scale would give 0 * inf = NaN (code 0 in the reference): a huge finite factor
        // yields the same codes without the NaN
        const float rcp = fminf(rcp_approx_ftz(__half2float(s)), 3.0e38f);
        const __half2 lo_c = __floats2half2_rn(-8.f, -8.f), hi_c = __floats2half2_rn(7.f, 7.f);
        const __half2 magic = __floats2half2_rn(1536.f, 1536.f);

        // ---- 4. codes -> staging bytes -> one 16-byte store per thread
#pragma unroll
        for (int ti = 0; ti < 5; ++ti) {
            if (ti < n_tiles) {
                const int nt = warp + 14 * ti;
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int kp = 16 * mt + g + 8 * hh;
                        if (kp < KH) {
                            const __half2 p = y[ti][mt][hh];
                            // rn_h(x * rcp), clamp, round to nearest even by the fp16 addition of 1536
                            const float2 f = __half22float2(p);
                            __half2 qh = __floats2half2_rn(f.x * rcp, f.y * rcp);
                            qh = __hmin2(__hmax2(qh, lo_c), hi_c);
                            qh = __hadd2(qh, magic);
                            const uint32_t r = *reinterpret_cast<uint32_t *>(&qh) & 0x000F000Fu;
                            obuf[kp * OUTP + 4 * nt + qd] = (uint8_t)(r | (r >> 12));
                            if (rotated != nullptr)
                                *reinterpret_cast<__half2 *>(rotated + (size_t)row * N + kp * SEG + 8 * nt + 2 * qd) = p;
                        }
                    }
            }
        }
        __syncthreads();
        {
            const int kp = tid >> 4, part = tid & 15;  // 448 threads x 16 B = 28 rows x 256 B
            const uint4 val = *reinterpret_cast<const uint4 *>(obuf + kp * OUTP + part * 16);
            reinterpret_cast<uint4 *>(q + (size_t)row * (N / 2))[tid] = val;
        }
        __syncthreads();  // staging and Z are dead: the next row may reuse the buffer
    }
}

}  // namespace

int launch_rotate_had28(const RotateArgs &a, cudaStream_t st) {
    const bool ok = a.n == N && a.K == KH && a.stride == 1 && a.q != nullptr && !a.asym && !a.fp32_mode &&
                    a.hadk != nullptr && (a.in_dtype == SR_F16 || (a.in_dtype == SR_BF16 && a.cast_in_to_f16)) &&
                    aligned16(a.x) && aligned16(a.q) && (a.out == nullptr || (a.out_dtype == SR_F16 && aligned4(a.out)));
    if (!ok) return SR_ERR_UNSUPPORTED;
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    const uint32_t grid = a.rows < (uint32_t)(2 * sm_count) ? a.rows : (uint32_t)(2 * sm_count);
#define SR_H28(T)                                                                                          \
    do {                                                                                                   \
        auto kfn = rotate_quant_had28_kernel<T>;                                                           \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);\
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "rotate_quant: %s", cudaGetErrorString(e));         \
        kfn<<<grid, THREADS, SMEM_BYTES, st>>>((const T *)a.x, (const __half *)a.hadk, a.sign, a.expert_ids, \
                                               a.rows, a.scale, a.clip, a.q, a.q_scale, (__half *)a.out);  \
    } while (0)
    if (a.in_dtype == SR_F16) SR_H28(__half);
    else SR_H28(__nv_bfloat16);
#undef SR_H28
    return check_launch("rotate_quant_had28");
}

}  // namespace sr
