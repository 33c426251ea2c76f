// Fused online rotation + sign + per-token int4 quantization for the model shapes that carry
// the traffic: rows of 4096 values (hidden size of an 8B model, q/k/v/o/gate/up inputs).
//
// One launch replaces fast_hadamard_transform + sign multiply + sym_quant_dynamic
// (signrot/functional/hadamard.py:81, signrot/nn/hadamard.py:39, signrot/kernels/fused.cu:68-112)
// and touches HBM once: 2 bytes in and 0.5 bytes out per value.
//
// Layout.  A row is owned by 64 threads (two warps); a thread keeps 64 fp32 values.
//   phase 1: thread t loads eight 16-byte vectors, vector c at element 512*c + 8*t, so each
//            warp-wide load covers 512 contiguous bytes.  Its 64 values span index bits
//            {0,1,2} (inside a vector) and {9,10,11} (the vector number): a 64-point
//            Walsh-Hadamard transform in registers takes care of those six bits.
//   exchange: a 64 x 64 fp32 transpose through shared memory (row pitch 65 words: both the
//            write and the read touch 32 distinct banks).
//   phase 2: thread t' = (c, b) now holds the 64 values with index bits {3..8} varying:
//            element 512*c + b + 8*j, j = 0..63.  Second 64-point transform in registers.
// The sums are fp32 throughout (the butterfly order differs from any other implementation
// only by fp32 rounding), scaled by 1/sqrt(n), rounded to fp16 once, then the sign is applied
// and the row maximum reduced over the 64 threads.
//   output: thread (c, b) owns every 8th value of the 512-value block c, so the eight lanes
//            b = 0..7 together hold whole output words.  Each lane packs its codes eight per
//            register, an 8 x 8 nibble transpose across the eight lanes (three shuffle rounds
//            per register) turns them into output words, and each store instruction writes
//            32 contiguous bytes per block.
// CTAs are persistent over rows, so the 64 sign bits a thread needs stay in two registers.
#include "rotate.cuh"
#include <cfloat>
#include <type_traits>

namespace sr {

namespace {

constexpr int ROWS_PER_CTA = 4;      // 256 threads
constexpr int PITCH = 65;            // words per transposed row

__device__ __forceinline__ void fwht64(float (&v)[64]) {
#pragma unroll
    for (int h = 1; h < 64; h <<= 1) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            if ((i & h) == 0) {
                const float a = v[i], b = v[i + h];
                v[i] = a + b;
                v[i + h] = a - b;
            }
        }
    }
}

__device__ __forceinline__ void team_sync(int team) {
    asm volatile("bar.sync %0, 64;" ::"r"(team + 1) : "memory");
}

template <typename InT, bool ASYM>
__global__ void __launch_bounds__(ROWS_PER_CTA * 64, 2)
rotate_quant_4096_kernel(const InT *__restrict__ x, const int8_t *__restrict__ sign,
                         const int32_t *__restrict__ expert_ids, uint32_t rows, float scale, float clip,
                         uint8_t *__restrict__ q, __half *__restrict__ q_scale, __half *__restrict__ q_zero,
                         __half *__restrict__ rotated) {
    constexpr int N = 4096;
    extern __shared__ float xch[];   // [ROWS_PER_CTA][64 * PITCH]
    __shared__ float red[ROWS_PER_CTA][2][2];

    const int tid = threadIdx.x;
    const int team = tid >> 6;        // row slot inside the CTA
    const int t = tid & 63;           // thread inside the team
    const int lane = tid & 31;
    float *buf = xch + team * (64 * PITCH);
    // phase-2 identity: block c, offset b
    const int c2 = t >> 3, b2 = t & 7;

    // sign bits of this thread's phase-2 elements (bit j <-> element 512*c2 + b2 + 8*j)
    uint64_t neg_static = 0;
    const bool per_row_sign = sign != nullptr && expert_ids != nullptr;
    if (sign != nullptr && !per_row_sign) {
#pragma unroll 8
        for (int j = 0; j < 64; ++j)
            if (sign[512 * c2 + b2 + 8 * j] < 0) neg_static |= (1ull << j);
    }

    for (uint32_t row = blockIdx.x * ROWS_PER_CTA + team; row < rows; row += gridDim.x * ROWS_PER_CTA) {
        // ---- phase 1: load + 64-point transform over bits {0,1,2,9,10,11}
        float v[64];
        const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * N);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            Vec16 ld;
            ld.u = __ldg(xr + c * 64 + t);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (sizeof(InT) == 2 && std::is_same<InT, __half>::value)
                    v[c * 8 + j] = __half2float(ld.h[j]);
                else
                    v[c * 8 + j] = __half2float(__float2half_rn(__bfloat162float(ld.b[j])));  // x.to(float16)
            }
        }
        fwht64(v);
        // ---- exchange: buf[t][j] -> buf[j'][t']
#pragma unroll
        for (int j = 0; j < 64; ++j) buf[t * PITCH + j] = v[j];
        team_sync(team);
#pragma unroll
        for (int j = 0; j < 64; ++j) v[j] = buf[j * PITCH + t];
        // ---- phase 2: bits {3..8}
        fwht64(v);

        uint64_t neg = neg_static;
        if (per_row_sign) {
            const int8_t *sg = sign + (size_t)expert_ids[row] * N;
            neg = 0;
#pragma unroll 8
            for (int j = 0; j < 64; ++j)
                if (sg[512 * c2 + b2 + 8 * j] < 0) neg |= (1ull << j);
        }
        // scale, round to fp16 (the dtype the reference's transform returns), sign, range
        __half hv[64];
        float vmax = ASYM ? -FLT_MAX : 0.f, vmin = FLT_MAX;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
            __half h = __float2half_rn(v[j] * scale);
            if ((neg >> j) & 1ull) h = __hneg(h);
            hv[j] = h;
            const float f = __half2float(h);
            if (ASYM) {
                vmax = fmaxf(vmax, f);
                vmin = fminf(vmin, f);
            } else {
                vmax = fmaxf(vmax, fabsf(f));
            }
        }
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
        int zero_i = 0;
        if (!ASYM) {
            __half s = __float2half(vmax / 7.f);
            if (clip != 1.f) s = __float2half(__half2float(s) * clip);
            if (t == 0) q_scale[row] = s;
            rcp = rcp_approx_ftz(__half2float(s));
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
            zero_i = __half2int_rn(zero);
            rcp = rcp_approx_ftz(__half2float(s));
        }

        if (rotated != nullptr) {
            __half *orow = rotated + (size_t)row * N + 512 * c2 + b2;
#pragma unroll
            for (int j = 0; j < 64; ++j) orow[8 * j] = hv[j];
        }

        // ---- codes, eight per register: P[g] nibble i = code of j = 8g + i
        uint32_t P[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            uint32_t w = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int code = ASYM ? asym_code(hv[g * 8 + i], rcp, zero_i, 0, 15) : sym_code(hv[g * 8 + i], rcp);
                w |= (uint32_t)(code & 15) << (4 * i);
            }
            P[g] = w;
        }
        // ---- 8 x 8 nibble transpose across lanes b = 0..7: afterwards lane i holds, in
        // nibble b, the code lane b had at position i (i.e. output word j = 8g + i)
#pragma unroll
        for (int k = 4; k >= 1; k >>= 1) {
            const uint32_t m = k == 4 ? 0xFFFF0000u : (k == 2 ? 0xFF00FF00u : 0xF0F0F0F0u);
            const bool upper = (b2 & k) != 0;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const uint32_t r = __shfl_xor_sync(0xffffffffu, P[g], k);
                P[g] = upper ? ((P[g] & m) | ((r >> (4 * k)) & ~m)) : ((P[g] & ~m) | ((r << (4 * k)) & m));
            }
        }
        uint32_t *qr = reinterpret_cast<uint32_t *>(q + (size_t)row * (N / 2)) + c2 * 64 + b2;
#pragma unroll
        for (int g = 0; g < 8; ++g) qr[8 * g] = P[g];
    }
}

}  // namespace

int launch_rotate_fast(const RotateArgs &a, cudaStream_t st) {
    const bool shape_ok = a.n == 4096 && a.K == 1 && a.stride == 1 && a.S == 4096 && a.q != nullptr &&
                          !a.fp32_mode && (a.in_dtype == SR_F16 || (a.in_dtype == SR_BF16 && a.cast_in_to_f16)) &&
                          aligned16(a.x) && aligned4(a.q) && (a.out == nullptr || a.out_dtype == SR_F16);
    if (!shape_ok) return launch_rotate_had28(a, st);  // the other dedicated shape, or SR_ERR_UNSUPPORTED
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    const uint32_t ctas_needed = cdiv<uint32_t>(a.rows, ROWS_PER_CTA);
    const uint32_t grid = ctas_needed < (uint32_t)(sm_count * 3) ? ctas_needed : (uint32_t)(sm_count * 3);
    constexpr size_t smem = (size_t)ROWS_PER_CTA * 64 * PITCH * sizeof(float);
#define SR_RQ(T, ASYM)                                                                                     \
    do {                                                                                                   \
        auto kfn = rotate_quant_4096_kernel<T, ASYM>;                                                      \
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return fail(SR_ERR_CUDA, "rotate_quant: %s", cudaGetErrorString(e));         \
        kfn<<<grid, ROWS_PER_CTA * 64, smem, st>>>((const T *)a.x, a.sign, a.expert_ids, a.rows, a.scale,   \
                                                   a.clip, a.q, a.q_scale, a.q_zero, (__half *)a.out);     \
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
