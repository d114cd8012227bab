// W2 instantiations of the shape-generic decode GEMV (one translation unit per bit-width so the
// three compile in parallel).
#include "cb_gemv_generic.cuh"

namespace cb {
int launch_gemv_generic_w2(int dtype, const void* x, const GemvParams& P, int64_t rho, cudaStream_t stream) {
    return launch_gemv_generic<2>(dtype, x, P, rho, stream);
}
int occupancy_gemv_generic_w2() { return occupancy_gemv_generic<2>(); }
}  // namespace cb
