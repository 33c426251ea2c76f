// Specialised rotation kernels for the 8B-model shapes.
#include "rotate.cuh"

namespace sr {

int launch_rotate_fast(const RotateArgs &a, cudaStream_t st) {
    (void)a;
    (void)st;
    return SR_ERR_UNSUPPORTED;
}

}  // namespace sr
