// Fused online rotation + sign + per-token int4 quantization for the model shapes that carry
// the traffic: rows of 4096 values (hidden size of an 8B model, q/k/v/o/gate/up inputs).
//
// One launch replaces fast_hadamard_transform + sign multiply + sym_quant_dynamic
// (signrot/functional/hadamard.py:81, signrot/nn/hadamard.py:39, signrot/kernels/fused.cu:68-112)
// and touches HBM once: 2 bytes in and 0.5 bytes out per value.
//
// Layout.  A row is owned by 64 threads (two warps); a thread keeps 64 fp32 values as 32
// register pairs and transforms them with packed fp32 adds (add.f32x2 / sub.f32x2).
//   phase 1: thread t loads eight 16-byte vectors, vector c at element 512*c + 8*t, so each
//            warp-wide load covers 512 contiguous bytes.  Its 64 values span index bits
//            {0,1,2} (inside a vector) and {9,10,11} (the vector number): one 64-point
//            Walsh-Hadamard transform in registers.
//   exchange: a 64 x 64 fp32 transpose through shared memory; scalar stores (row pitch 68
//            words), 128-bit loads, both bank-conflict free.  Inside a group of eight the
//            values are stored in the order 0,4,1,5,2,6,3,7 so that a register pair holds
//            values i and i+4: their 4-bit codes then drop into an output word with one
//            shift-add each.
//   phase 2: thread t' = (c, b) holds element 512*c + b + 8*j, j = 0..63 (index bits {3..8}):
//            second 64-point transform.
// Sums are fp32 throughout, scaled by 1/sqrt(n) and rounded to fp16 once (the dtype the
// reference's transform returns); sign, row maximum and the code decision run on packed fp16
// pairs.  No instruction of the inner loops uses the conversion unit: roundings are packed
// cvt.rn.f16x2.f32, fp16->fp32 is an exact widening, and round-to-nearest-even of the quotient is
// the fp16 addition of 1536 (whose low mantissa bits then hold the integer).
//   output: thread (c, b) owns every 8th value of the 512-value block c, so the eight lanes
//            b = 0..7 together hold whole output words: an 8 x 8 nibble transpose across those
//            lanes (three shuffle rounds per register), then every store instruction writes 32
//            contiguous bytes per block.
// CTAs are persistent over rows; a thread's sign masks live in its own shared-memory row.
#include "rotate.cuh"
#include <cfloat>
#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace sr {

namespace {

constexpr int ROWS_PER_CTA = 4;      // 256 threads
constexpr int PITCH = 68;            // words per transposed row (16-byte aligned, bank-conflict free)
constexpr int SPITCH = 33;           // words per thread in the sign-mask table
constexpr int XCH_WORDS = 64 * PITCH;
constexpr int SGN_WORDS = 64 * SPITCH;
constexpr size_t SMEM_BYTES = (size_t)ROWS_PER_CTA * (XCH_WORDS + SGN_WORDS) * 4;

__device__ __forceinline__ void team_sync(int team) {
    asm volatile("bar.sync %0, 64;" ::"r"(team + 1) : "memory");
}

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t w) { return *reinterpret_cast<__half2 *>(&w); }

template <typename InT, bool ASYM>
__global__ void __launch_bounds__(ROWS_PER_CTA * 64, 2)
rotate_quant_4096_kernel(const InT *__restrict__ x, const int8_t *__restrict__ sign,
                         const int32_t *__restrict__ expert_ids, uint32_t rows, float scale, float clip,
                         uint8_t *__restrict__ q, __half *__restrict__ q_scale, __half *__restrict__ q_zero,
                         __half *__restrict__ rotated) {
    constexpr int N = 4096;
    extern __shared__ __align__(16) float smem_f[];
    __shared__ float red[ROWS_PER_CTA][2][2];

    const int tid = threadIdx.x;
    const int team = tid >> 6;        // row slot inside the CTA
    const int t = tid & 63;           // thread inside the team
    const int lane = tid & 31;
    float *buf = smem_f + team * XCH_WORDS;
    uint32_t *sgn = reinterpret_cast<uint32_t *>(smem_f + ROWS_PER_CTA * XCH_WORDS) + team * SGN_WORDS + t * SPITCH;
    // phase-2 identity: block c2, offset b2; slot a = 4g + m holds j = 8g + m (low) and 8g + m + 4 (high)
    const int c2 = t >> 3, b2 = t & 7;
    // where this thread's phase-1 values go inside a transposed row: position of j' = t
    const int wpos = (t & ~7) | (((t & 3) << 1) | ((t >> 2) & 1));

    const bool per_row_sign = sign != nullptr && expert_ids != nullptr;
    auto fill_sign = [&](const int8_t *sg) {
#pragma unroll 4
        for (int a = 0; a < 32; ++a) {
            const int j = 8 * (a >> 2) + (a & 3);
            uint32_t m = 0;
            if (sg != nullptr) {
                if (sg[512 * c2 + b2 + 8 * j] < 0) m |= 0x00008000u;
                if (sg[512 * c2 + b2 + 8 * (j + 4)] < 0) m |= 0x80000000u;
            }
            sgn[a] = m;
        }
    };
    if (!per_row_sign) fill_sign(sign);  // thread-private rows: no synchronisation needed

    const __half2 magic = __floats2half2_rn(1536.f, 1536.f);
    const u64 scale2 = pack2(scale, scale);

    const uint32_t row_step = gridDim.x * ROWS_PER_CTA;
    uint4 nx[8];  // the row after the current one, in flight while the current one is transformed
    {
        const uint32_t row0 = blockIdx.x * ROWS_PER_CTA + team;
        if (row0 < rows) {
            const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row0 * N);
#pragma unroll
            for (int c = 0; c < 8; ++c) nx[c] = __ldg(xr + c * 64 + t);
        }
    }
    for (uint32_t row = blockIdx.x * ROWS_PER_CTA + team; row < rows; row += row_step) {
        // ---- phase 1: 64-point transform over bits {0,1,2,9,10,11}
        u64 v[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            Vec16 ld;
            ld.u = nx[c];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                float2 f;
                if (std::is_same<InT, __half>::value) {
                    f = __half22float2(ld.h2[p]);
                } else {
                    // bf16 -> fp32 is a shift; x.to(float16) is one packed rounding; widening is exact
                    const float a = __uint_as_float(ld.w[p] << 16), b = __uint_as_float(ld.w[p] & 0xFFFF0000u);
                    f = __half22float2(__floats2half2_rn(a, b));
                }
                v[c * 4 + p] = pack2(f.x, f.y);
            }
        }
        if (row + row_step < rows) {
            const uint4 *xn = reinterpret_cast<const uint4 *>(x + (size_t)(row + row_step) * N);
#pragma unroll
            for (int c = 0; c < 8; ++c) nx[c] = __ldg(xn + c * 64 + t);
        }
        fwht_pairs<32, 32>(v);
        // ---- exchange: value j of thread t goes to row j, position wpos
#pragma unroll
        for (int a = 0; a < 32; ++a) {
            float lo, hi;
            unpack2(v[a], lo, hi);
            buf[(2 * a) * PITCH + wpos] = lo;
            buf[(2 * a + 1) * PITCH + wpos] = hi;
        }
        team_sync(team);
        {
            const uint4 *rowp = reinterpret_cast<const uint4 *>(buf + t * PITCH);
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                const uint4 w = rowp[m];  // positions 4m..4m+3 hold (j, j+4), (j+1, j+5) of group m/2
                v[2 * m] = ((u64)w.y << 32) | w.x;
                v[2 * m + 1] = ((u64)w.w << 32) | w.z;
            }
        }
        // ---- phase 2: bits {3..8}
        fwht_pairs<32, 32>(v);

        if (per_row_sign) fill_sign(sign + (size_t)expert_ids[row] * N);

        // scale, one rounding to fp16, sign, range
        __half2 hv[32];
        __half2 hmaxv = __floats2half2_rn(ASYM ? -65504.f : 0.f, ASYM ? -65504.f : 0.f);
        __half2 hminv = __floats2half2_rn(65504.f, 65504.f);
#pragma unroll
        for (int a = 0; a < 32; ++a) {
            float lo, hi;
            unpack2(mul2(v[a], scale2), lo, hi);
            const __half2 h = bits_h2(h2_bits(__floats2half2_rn(lo, hi)) ^ sgn[a]);
            hv[a] = h;
            if (ASYM) {
                hmaxv = __hmax2(hmaxv, h);
                hminv = __hmin2(hminv, h);
            } else {
                hmaxv = __hmax2(hmaxv, __habs2(h));
            }
        }
        float vmax = fmaxf(__low2float(hmaxv), __high2float(hmaxv));
        float vmin = fminf(__low2float(hminv), __high2float(hminv));
        vmax = warp_max(vmax);
        if (ASYM) vmin = warp_min(vmin);
        if (lane == 0) {
            red[team][(t >> 5)][0] = vmax;
            red[team][(t >> 5)][1] = vmin;
        }
        team_sync(team);
        vmax = fmaxf(red[team][0][0], red[team][1][0]);
        vmin = fminf(red[team][0][1], red[team][1][1]);

        float rcp;
        uint32_t zero_u = 0;
        __half2 lo_c, hi_c;
        if (!ASYM) {
            __half s = __float2half(vmax / 7.f);
            if (clip != 1.f) s = __float2half(__half2float(s) * clip);
            if (t == 0) q_scale[row] = s;
            rcp = rcp_approx_ftz(__half2float(s));
            lo_c = __floats2half2_rn(-8.f, -8.f);
            hi_c = __floats2half2_rn(7.f, 7.f);
        } else {
            __half hmin = __float2half(vmin), hmax = __float2half(vmax);
            if (clip != 1.f) {
                hmin = __float2half(__half2float(hmin) * clip);
                hmax = __float2half(__half2float(hmax) * clip);
            }
            const __half diff = __float2half(__half2float(hmax) - __half2float(hmin));
            const __half s = __float2half(__half2float(diff) / 15.f);
            const __half ratio = __float2half(-__half2float(hmin) / __half2float(s));
            const __half zero = __float2half(nearbyintf(__half2float(ratio)));
            if (t == 0) {
                q_scale[row] = s;
                q_zero[row] = zero;
            }
            const int zi = __half2int_rn(zero);
            zero_u = (uint32_t)(zi & 15) * 0x00010001u;  // only the code's low nibble matters
            // clamp(rint(v) + z, 0, 15) = rint(clamp(v, -z, 15 - z)) + z for an integer z
            lo_c = __floats2half2_rn(-(float)zi, -(float)zi);
            hi_c = __floats2half2_rn(15.f - (float)zi, 15.f - (float)zi);
            rcp = rcp_approx_ftz(__half2float(s));
        }
        // a zero scale gives rcp = inf and 0 * inf = NaN, which the reference turns into code 0;
        // a huge finite factor gives the same codes (x != 0 still saturates) without the NaN
        rcp = fminf(rcp, 3.0e38f);
        const u64 rcp2 = pack2(rcp, rcp);

        if (rotated != nullptr) {
            __half *orow = rotated + (size_t)row * N + 512 * c2 + b2;
#pragma unroll
            for (int a = 0; a < 32; ++a) {
                const int j = 8 * (a >> 2) + (a & 3);
                orow[8 * j] = __low2half(hv[a]);
                orow[8 * (j + 4)] = __high2half(hv[a]);
            }
        }

        // ---- codes: P[g] nibble i = code of j = 8g + i; slot 4g + m carries nibbles m and m + 4
        uint32_t P[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            uint32_t w = 0;
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const float2 f = __half22float2(hv[4 * g + m]);
                float lo, hi;
                unpack2(mul2(pack2(f.x, f.y), rcp2), lo, hi);
                __half2 qh = __floats2half2_rn(lo, hi);  // rn_h(x * rcp): the quotient __hdiv returns
                qh = __hmin2(__hmax2(qh, lo_c), hi_c);
                // fp16 addition of 1536 rounds to the nearest even integer; its low mantissa bits are the code
                const uint32_t r = ((h2_bits(__hadd2(qh, magic)) & 0x000F000Fu) + zero_u) & 0x000F000Fu;
                w += r << (4 * m);
            }
            P[g] = w;
        }
        // ---- 8 x 8 nibble transpose across lanes b = 0..7: afterwards lane i holds, in
        // nibble b, the code lane b had at position i (i.e. output word j = 8g + i)
#pragma unroll
        for (int k = 4; k >= 1; k >>= 1) {
            const uint32_t msk = k == 4 ? 0xFFFF0000u : (k == 2 ? 0xFF00FF00u : 0xF0F0F0F0u);
            const bool upper = (b2 & k) != 0;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const uint32_t r = __shfl_xor_sync(0xffffffffu, P[g], k);
                P[g] = upper ? ((P[g] & msk) | ((r >> (4 * k)) & ~msk)) : ((P[g] & ~msk) | ((r << (4 * k)) & msk));
            }
        }
        uint32_t *qr = reinterpret_cast<uint32_t *>(q + (size_t)row * (N / 2)) + c2 * 64 + b2;
#pragma unroll
        for (int g = 0; g < 8; ++g) qr[8 * g] = P[g];
    }
}

}  // namespace

int launch_rotate_fast(const RotateArgs &a, cudaStream_t st) {
    // tensor-core transforms first; the butterfly kernel below takes what they do not: per-row sign tables
    // (expert ids) at n = 4096
    {
        int rc = launch_rotate_umma4096(a, st);
        if (rc != SR_ERR_UNSUPPORTED) return rc;
        rc = launch_rotate_tc4096(a, st);
        if (rc != SR_ERR_UNSUPPORTED) return rc;
        rc = launch_rotate_heads32(a, st);
        if (rc != SR_ERR_UNSUPPORTED) return rc;
    }
    const bool shape_ok = a.n == 4096 && a.K == 1 && a.stride == 1 && a.S == 4096 && a.q != nullptr &&
                          !a.fp32_mode && (a.in_dtype == SR_F16 || (a.in_dtype == SR_BF16 && a.cast_in_to_f16)) &&
                          aligned16(a.x) && aligned4(a.q) && (a.out == nullptr || a.out_dtype == SR_F16);
    if (!shape_ok) {   // the other dedicated shape, or SR_ERR_UNSUPPORTED
        const int rc = launch_rotate_had28_umma(a, st);
        return rc != SR_ERR_UNSUPPORTED ? rc : launch_rotate_had28(a, st);
    }
    const int sm_count = current_sm_count();
    const uint32_t ctas_needed = cdiv<uint32_t>(a.rows, ROWS_PER_CTA);
    const uint32_t grid = ctas_needed < (uint32_t)(sm_count * 2) ? ctas_needed : (uint32_t)(sm_count * 2);
#define SR_RQ(T, ASYM)                                                                                     \
    do {                                                                                                   \
        auto kfn = rotate_quant_4096_kernel<T, ASYM>;                                                      \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES); \
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "rotate_quant: %s", cudaGetErrorString(e));         \
        kfn<<<grid, ROWS_PER_CTA * 64, SMEM_BYTES, st>>>((const T *)a.x, a.sign, a.expert_ids, a.rows,      \
                                                         a.scale, a.clip, a.q, a.q_scale, a.q_zero,        \
                                                         (__half *)a.out);                                 \
    } while (0)
    if (a.in_dtype == SR_F16) {
        if (a.asym) SR_RQ(__half, true);
        else SR_RQ(__half, false);
    } else {
        if (a.asym) SR_RQ(__nv_bfloat16, true);
        else SR_RQ(__nv_bfloat16, false);
    }
#undef SR_RQ
    return check_launch("rotate_quant_4096");
}

}  // namespace sr
