// Shared helpers for the signrot_b200 CUDA library (sm_100a only).
//
// Everything exported from this library is a plain C function that takes
// device pointers, sizes and a CUDA stream, returns an int status and never
// allocates, synchronises or reads device memory on the host, so every entry
// point can be captured in a CUDA graph.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/signrot_b200.h"

namespace sr {

// ---------------------------------------------------------------- errors

// Thread-local message of the last failing call; read by sr_last_error().
char *last_error_buffer();
int fail(int code, const char *fmt, ...);

#define SR_REQUIRE(cond, code, ...)                    \
    do {                                               \
        if (!(cond)) return ::sr::fail((code), __VA_ARGS__); \
    } while (0)

// Checks the launch (not the execution) of the kernel just enqueued.
inline int check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(SR_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return SR_OK;
}

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// ---- programmatic dependent launch (decode-graph kernels)
//
// A kernel launched through launch_pdl may be scheduled while the kernel before it on the stream is
// still running; it must execute pdl_wait() (every thread, before any early exit) ahead of its
// first access to memory that an earlier kernel writes or reads, and everything before that point
// may only touch memory no kernel of the stream writes (weights, tables).  pdl_wait() returns once
// all earlier kernels have completed and their writes are visible, so ordering is transitive as
// long as every kernel launched this way waits.  pdl_trigger() lets the next kernel be scheduled
// early; without the launch attribute both are no-ops.  SIGNROT_B200_PDL=0 turns the attribute off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();   // elementwise.cu

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

template <typename T>
__host__ __device__ __forceinline__ T cdiv(T a, T b) { return (a + b - 1) / b; }

// SM count of the CURRENT device (launch grids are sized by it); the runtime answers from its own cache.
inline int current_sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        n <= 0)
        return 148;
    return n;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned4(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

// ---------------------------------------------------------------- device math

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// rcp.approx.ftz.f32: the reciprocal the toolkit's device __hdiv() uses.  Hoisted
// out of per-element loops, so that  q = rn_h(float(x) * rcp)  reproduces
// __hdiv(x, s) for every quotient that can change a 4-bit code (the FMA fix-up
// __hdiv applies to results below 2^-17 cannot move a value across +-0.5).
__device__ __forceinline__ float rcp_approx_ftz(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return max(lo, min(hi, v)); }

// Symmetric code of one fp16 value: clamp(half2int_rn(x / s), -8, 7).
__device__ __forceinline__ int sym_code(__half x, float rcp) {
    __half v = __float2half_rn(__half2float(x) * rcp);
    return clampi(__half2int_rn(v), -8, 7);
}
// Asymmetric code: clamp(half2int_rn(x / s) + zero, lo, hi).
__device__ __forceinline__ int asym_code(__half x, float rcp, int zero, int lo, int hi) {
    __half v = __float2half_rn(__half2float(x) * rcp);
    return clampi(__half2int_rn(v) + zero, lo, hi);
}

// bf16 -> fp16 goes through fp32, the same single rounding torch's .to(float16) does.
__device__ __forceinline__ __half to_half(__half v) { return v; }
__device__ __forceinline__ __half to_half(__nv_bfloat16 v) { return __float2half_rn(__bfloat162float(v)); }

// ---------------------------------------------------------------- bounded mbarrier wait
//
// No wait in this library spins without a limit.  The poll loop touches nothing but the barrier (any other
// shared-memory access would compete with operand traffic); the abort flag (shared by the roles of a CTA) and
// the clock are looked at every 64 polls.  On expiry the waiter raises the abort flag, records `code` in the
// device status word (first failure wins) and returns false; the caller then leaves its loop and the kernel
// returns normally, so the context stays usable.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code,
                                                  long long budget_cycles, int *status_word) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > budget_cycles) {
            *abort_flag = code;
            atomicCAS(status_word, 0, code);
            return false;
        }
    }
}

union Vec16 {
    uint4 u;
    __half h[8];
    __nv_bfloat16 b[8];
    __half2 h2[4];
    uint32_t w[4];
};

}  // namespace sr
