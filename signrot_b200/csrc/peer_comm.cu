// One-shot exchanges between the GPUs of a tensor- or expert-parallel group over peer memory (NVLink).
//
// The reference keeps this path on one device (fake_quant/kernel_utils.py:365-366); a sharded decode step
// adds, per row-parallel linear, an all-gather of a few hundred KB (the online rotation and the per-token
// scale span the whole row) and an all-reduce of the int32 partial sums.  At those sizes the cost is latency,
// not bandwidth, so both are ONE kernel here and the protocol spends exactly one trip across the fabric:
//
//   push     every thread stores its 16-byte pieces of this rank's message into slot [rank] of every rank's
//            exchange buffer as flagged lines: two 16-byte peer stores per piece, each {data, n, data, n} with n
//            the number of this exchange.  An aligned 8-byte half of such a store becomes visible as a whole, so a
//            reader that sees n beside a word has that word: no fence, no separate flag, no second trip;
//   combine  every thread polls the lines it needs in the LOCAL slots until they carry n (bounded: on expiry the
//            kernel records a status code and carries on, so the context stays usable) and writes the caller's
//            output: concatenation (all-gather), integer sum + dequant epilogue (row-parallel W4A4 linear:
//            integer addition is order-free, so every group size gives the bits of one GPU), or fp32 sum in rank
//            order (expert-parallel partial outputs).
// Plain peer stores and local loads only: no multicast loads, no copy engine.
//
// Exchange buffers are double-buffered by the parity of a device-resident exchange counter, so the kernel is
// the same launch every time (capturable in a CUDA graph) and a fast rank that is already pushing exchange
// n + 1 cannot overwrite lines a slow rank is still combining for exchange n (a rank can never be two
// exchanges ahead: finishing n + 1 needs every peer's lines of n + 1, which a peer stores after its own
// exchange n has ended).  Every rank must issue the same sequence of exchanges.
#include "common.cuh"
#include <cstring>

namespace sr {

namespace {

constexpr int PC_MAX_RANKS = 8;
constexpr int PC_THREADS = 256;
constexpr int PC_MAX_CTAS = 128;                // a thread waits only for lines, never for another CTA of its own GPU
constexpr long long PC_WAIT_BUDGET = 3000000000ll;   // about 1.5 s of SM cycles

__device__ int g_peer_status;

// Control block at the start of every rank's region.
struct PeerCtrl {
    uint32_t epoch;                 // exchanges this rank has completed
    uint32_t done;                  // CTAs of the running exchange that have finished
};
constexpr size_t PC_CTRL_BYTES = 256;

struct PeerArgs {
    uint8_t *region[PC_MAX_RANKS];  // region of every rank, mapped into this process (own region at [rank])
    int rank, world;
    unsigned long long slot_bytes;  // bytes of one slot: twice the largest message (every word travels with a flag)
};

__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_line(void *p, uint32_t d0, uint32_t d1, uint32_t n) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(n), "r"(d1), "r"(n) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const void *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// The four data words of piece i of a slot (two flagged lines), once both lines carry exchange number n.
__device__ __forceinline__ uint4 wait_piece(const uint8_t *slot, unsigned long long i, uint32_t n, long long t0, int who) {
    const uint8_t *p = slot + i * 32;
    uint4 a = ld_line(p), b = ld_line(p + 16);
    int spins = 0;
    while (a.y != n || a.w != n || b.y != n || b.w != n) {
        if (++spins == 64) {
            spins = 0;
            if (*reinterpret_cast<volatile int *>(&g_peer_status) != 0) break;      // some wait has already given up
            if (clock64() - t0 > PC_WAIT_BUDGET) {
                atomicCAS(&g_peer_status, 0, 60 + who);                              // code 60 + rank that never arrived
                break;
            }
        }
        a = ld_line(p);
        b = ld_line(p + 16);
    }
    return make_uint4(a.x, a.z, b.x, b.z);
}

enum { PC_GATHER = 0, PC_REDUCE_I32_DEQUANT = 1, PC_REDUCE_F32 = 2 };

struct CombineArgs {
    long long rows, cols;           // GATHER: cols = columns of ONE rank's shard (fp16); REDUCE: cols of the output
    const __half *row_scale;        // REDUCE_I32_DEQUANT: per-row activation scale [rows]
    const __half *col_scale;        //                     per-column weight scale [cols]
    void *out;                      // fp16 [rows, world * cols] (GATHER) or fp16 [rows, cols]
};

template <int MODE>
__global__ void __launch_bounds__(PC_THREADS)
peer_exchange_kernel(PeerArgs a, const uint4 *__restrict__ src, unsigned long long pieces, CombineArgs c) {
    pdl_trigger();
    pdl_wait();                     // src comes from the kernel before this one
    const int tid = threadIdx.x;
    PeerCtrl *me = reinterpret_cast<PeerCtrl *>(a.region[a.rank]);
    __shared__ uint32_t s_epoch;
    if (tid == 0) s_epoch = ld_relaxed_gpu(&me->epoch) + 1;   // rewritten only after every CTA has read it
    __syncthreads();
    const uint32_t n = s_epoch;
    const unsigned long long parity_off = PC_CTRL_BYTES + (unsigned long long)(n & 1) * a.world * a.slot_bytes;
    const unsigned long long stride = (unsigned long long)gridDim.x * PC_THREADS;
    const unsigned long long first = (unsigned long long)blockIdx.x * PC_THREADS + tid;

    // ---- push: this rank's message into slot [rank] of every rank's buffer (its own included), as flagged lines
    {
        const unsigned long long my_slot = parity_off + (unsigned long long)a.rank * a.slot_bytes;
        for (unsigned long long i = first; i < pieces; i += stride) {
            const uint4 v = src[i];
#pragma unroll
            for (int r = 0; r < PC_MAX_RANKS; ++r)
                if (r < a.world) {
                    uint8_t *dst = a.region[r] + my_slot + i * 32;
                    st_line(dst, v.x, v.y, n);
                    st_line(dst + 16, v.z, v.w, n);
                }
        }
    }

    // ---- combine from the local slots, waiting line by line
    const uint8_t *mine = a.region[a.rank] + parity_off;
    const long long t0 = clock64();
    if (MODE == PC_GATHER) {
        // slot r holds rank r's [rows, cols] fp16 shard; out is [rows, world * cols]
        const unsigned long long per_row = (unsigned long long)c.cols / 8;          // 16-byte pieces per shard row
        const unsigned long long total = (unsigned long long)a.world * pieces;
        uint4 *out = reinterpret_cast<uint4 *>(c.out);
        for (unsigned long long i = first; i < total; i += stride) {
            const unsigned long long r = i / pieces, j = i % pieces;
            const unsigned long long row = j / per_row, col = j % per_row;
            out[(row * a.world + r) * per_row + col] = wait_piece(mine + r * a.slot_bytes, j, n, t0, (int)r);
        }
    } else if (MODE == PC_REDUCE_I32_DEQUANT) {
        const unsigned long long per_row = (unsigned long long)c.cols / 4;          // pieces of four int32 per row
        uint2 *out = reinterpret_cast<uint2 *>(c.out);
        for (unsigned long long i = first; i < pieces; i += stride) {
            int4 acc = make_int4(0, 0, 0, 0);
#pragma unroll
            for (int r = 0; r < PC_MAX_RANKS; ++r)
                if (r < a.world) {
                    const uint4 v = wait_piece(mine + (unsigned long long)r * a.slot_bytes, i, n, t0, r);
                    acc.x += (int)v.x;
                    acc.y += (int)v.y;
                    acc.z += (int)v.z;
                    acc.w += (int)v.w;
                }
            const unsigned long long row = i / per_row, col = (i % per_row) * 4;
            const float sr = __half2float(c.row_scale[row]);
            const uint2 sc = *reinterpret_cast<const uint2 *>(c.col_scale + col);
            const __half2 s01 = *reinterpret_cast<const __half2 *>(&sc.x), s23 = *reinterpret_cast<const __half2 *>(&sc.y);
            // the dequant epilogue of the one-GPU linear: rn_h((float(acc) * s_row) * s_col)
            const __half2 o01 = __floats2half2_rn(((float)acc.x * sr) * __low2float(s01), ((float)acc.y * sr) * __high2float(s01));
            const __half2 o23 = __floats2half2_rn(((float)acc.z * sr) * __low2float(s23), ((float)acc.w * sr) * __high2float(s23));
            uint2 o;
            o.x = *reinterpret_cast<const uint32_t *>(&o01);
            o.y = *reinterpret_cast<const uint32_t *>(&o23);
            out[i] = o;
        }
    } else {
        uint2 *out = reinterpret_cast<uint2 *>(c.out);
        for (unsigned long long i = first; i < pieces; i += stride) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < PC_MAX_RANKS; ++r)
                if (r < a.world) {                                 // rank order: the same sum on every rank
                    const uint4 v = wait_piece(mine + (unsigned long long)r * a.slot_bytes, i, n, t0, r);
                    acc.x += __uint_as_float(v.x);
                    acc.y += __uint_as_float(v.y);
                    acc.z += __uint_as_float(v.z);
                    acc.w += __uint_as_float(v.w);
                }
            const __half2 o01 = __floats2half2_rn(acc.x, acc.y), o23 = __floats2half2_rn(acc.z, acc.w);
            uint2 o;
            o.x = *reinterpret_cast<const uint32_t *>(&o01);
            o.y = *reinterpret_cast<const uint32_t *>(&o23);
            out[i] = o;
        }
    }

    // ---- the last CTA to finish publishes the new exchange count
    __syncthreads();
    if (tid == 0) {
        const uint32_t finished = atomicAdd(&me->done, 1u);
        if (finished == gridDim.x - 1) {
            me->done = 0;
            __threadfence();
            atomicExch(&me->epoch, n);
        }
    }
}

}  // namespace

int peer_device_status(int *out, bool clear) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_peer_status, sizeof(int));
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
    if (clear && v != 0) {
        const int z = 0;
        cudaMemcpyToSymbol(g_peer_status, &z, sizeof(int));
    }
    *out = v;
    return SR_OK;
}

}  // namespace sr

using namespace sr;

extern "C" {

int sr_peer_region_bytes(int64_t world, int64_t slot_bytes, int64_t *bytes) {
    SR_REQUIRE(bytes && world >= 1 && world <= PC_MAX_RANKS && slot_bytes > 0 && slot_bytes % 16 == 0, SR_ERR_INVALID,
               "peer_region_bytes: world %lld (1..%d), slot %lld bytes (a positive multiple of 16)", (long long)world,
               PC_MAX_RANKS, (long long)slot_bytes);
    *bytes = (int64_t)PC_CTRL_BYTES + 2 * world * (2 * slot_bytes);      // two parities; every data word travels with a flag
    return SR_OK;
}

int sr_peer_alloc(int64_t bytes, void **ptr, void *ipc_handle) {
    SR_REQUIRE(ptr && ipc_handle && bytes > 0, SR_ERR_INVALID, "peer_alloc: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "peer_alloc: cudaMalloc(%lld): %s", (long long)bytes, cudaGetErrorString(e));
    e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(SR_ERR_CUDA, "peer_alloc: %s", cudaGetErrorString(e));
    }
    memcpy(ipc_handle, &h, sizeof(h));
    *ptr = p;
    return SR_OK;
}

int sr_peer_open(const void *ipc_handle, void **ptr) {
    SR_REQUIRE(ptr && ipc_handle, SR_ERR_INVALID, "peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle, sizeof(h));
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "peer_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    *ptr = p;
    return SR_OK;
}

int sr_peer_close(void *ptr) {
    if (ptr == nullptr) return SR_OK;
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "peer_close: %s", cudaGetErrorString(e));
    return SR_OK;
}

int sr_peer_free(void *ptr) {
    if (ptr == nullptr) return SR_OK;
    cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) return fail(SR_ERR_CUDA, "peer_free: %s", cudaGetErrorString(e));
    return SR_OK;
}

int sr_peer_exchange(int mode, const void *const *regions, int rank, int world, int64_t slot_bytes, const void *src,
                     int64_t rows, int64_t cols, const void *row_scale, const void *col_scale, void *out,
                     void *stream) {
    SR_REQUIRE(regions && src && out, SR_ERR_INVALID, "peer_exchange: null pointer");
    SR_REQUIRE(world >= 1 && world <= PC_MAX_RANKS && rank >= 0 && rank < world, SR_ERR_INVALID,
               "peer_exchange: rank %d of %d", rank, world);
    SR_REQUIRE(rows > 0 && cols > 0, SR_ERR_INVALID, "peer_exchange: empty message");
    SR_REQUIRE(mode >= PC_GATHER && mode <= PC_REDUCE_F32, SR_ERR_INVALID, "peer_exchange: unknown mode %d", mode);
    const int64_t elem = mode == PC_GATHER ? 2 : 4;
    SR_REQUIRE(cols % (16 / elem) == 0, SR_ERR_INVALID, "peer_exchange: %lld columns are not a whole number of 16-byte pieces",
               (long long)cols);
    const int64_t bytes = rows * cols * elem;
    SR_REQUIRE(bytes <= slot_bytes, SR_ERR_UNSUPPORTED, "peer_exchange: message of %lld bytes, slots hold %lld",
               (long long)bytes, (long long)slot_bytes);
    SR_REQUIRE(aligned16(src) && aligned16(out), SR_ERR_INVALID, "peer_exchange: src/out must be 16-byte aligned");
    SR_REQUIRE(mode != PC_REDUCE_I32_DEQUANT || (row_scale && col_scale && (reinterpret_cast<uintptr_t>(col_scale) & 7u) == 0),
               SR_ERR_INVALID, "peer_exchange: the dequant mode needs both scale vectors (column scales 8-byte aligned)");
    PeerArgs a = {};
    for (int r = 0; r < world; ++r) {
        SR_REQUIRE(regions[r] != nullptr, SR_ERR_INVALID, "peer_exchange: region of rank %d is missing", r);
        a.region[r] = (uint8_t *)const_cast<void *>(regions[r]);
    }
    a.rank = rank;
    a.world = world;
    a.slot_bytes = 2ull * (unsigned long long)slot_bytes;
    CombineArgs c = {rows, cols, (const __half *)row_scale, (const __half *)col_scale, out};
    const unsigned long long pieces = (unsigned long long)bytes / 16;
    unsigned long long ctas = cdiv<unsigned long long>(pieces, PC_THREADS);
    if (ctas > PC_MAX_CTAS) ctas = PC_MAX_CTAS;
    cudaStream_t st = as_stream(stream);
    const dim3 grid((unsigned)ctas), block(PC_THREADS);
    if (mode == PC_GATHER) launch_pdl(peer_exchange_kernel<PC_GATHER>, grid, block, 0, st, a, (const uint4 *)src, pieces, c);
    else if (mode == PC_REDUCE_I32_DEQUANT)
        launch_pdl(peer_exchange_kernel<PC_REDUCE_I32_DEQUANT>, grid, block, 0, st, a, (const uint4 *)src, pieces, c);
    else launch_pdl(peer_exchange_kernel<PC_REDUCE_F32>, grid, block, 0, st, a, (const uint4 *)src, pieces, c);
    return check_launch("peer_exchange");
}

}  // extern "C"
