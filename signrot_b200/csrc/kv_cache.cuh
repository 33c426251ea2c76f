// Paged int4 KV cache descriptor shared by the cache kernels.
//
// Cache layout (signrot/transformers/kv_cache.py:185-196, kernels/include/flashinfer/page.cuh:60-95):
//   data  uint8 [pages, layers, 2 (k,v), heads, page_size, head_dim/2]   two 4-bit codes per byte
//   param fp16  [pages, layers, 2,       heads, page_size, 2]            (scale, zero) per vector
//   dequant: float(code) * scale - zero                                  (quantization.cuh:76)
#pragma once
#include "common.cuh"

namespace sr {

struct PagedKV {
    uint8_t *data;
    __half2 *param;
    const int32_t *indptr, *indices, *last_page_offset;
    uint32_t num_layers, layer, heads, page_size;  // head_dim fixed to 128

    __device__ __forceinline__ size_t vec_index(uint32_t page, uint32_t kv, uint32_t head, uint32_t entry) const {
        return ((((size_t)page * num_layers + layer) * 2 + kv) * heads + head) * page_size + entry;
    }
    __device__ __forceinline__ uint32_t seq_len(uint32_t b) const {
        return (uint32_t)(indptr[b + 1] - indptr[b] - 1) * page_size + (uint32_t)last_page_offset[b];
    }
};

constexpr int HD = 128;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Tensor-core decode kernel (kv_decode_tc.cu): same arguments and workspace format as decode_kernel.
// Returns 0 when the geometry is not one it handles (page_size % 16 != 0), 1 when the split-KV states are left in tmp
// for decode_merge_kernel, 2 when the output is complete (one chunk, merged in the cluster, or merged through counters).
int launch_decode_tc(int G, dim3 grid, const __half *q, const PagedKV &kv, __half *o, float *tmp, uint32_t num_chunks,
                      int had_q, float had_scale, cudaStream_t st, int32_t *counters = nullptr);

}  // namespace sr
