// Bit-exact unpack of the packed layout to int32 codes: the device counterpart of
// Crispybits/Kernel/crispybits_kernels/reference.py:58-67, used to check the integer layout
// against the CPU oracle.  One thread per output code; consecutive threads read consecutive
// codes of a row, so both the word reads and the int32 writes coalesce.
#include "cb_bitpack.cuh"
#include "cb_common.cuh"

namespace cb {

__global__ void unpack_codes_kernel(const uint32_t* __restrict__ packed, int64_t n, int K, int wpr, int bits,
                                    int32_t* __restrict__ codes) {
    const int64_t total = n * (int64_t)K;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / K;
        const int k = (int)(i - r * K);
        codes[i] = (int32_t)row_code(packed + r * wpr, k, bits);
    }
}

int launch_unpack(const int32_t* packed, int64_t n, int64_t K, int bits, int32_t* codes, cudaStream_t stream) {
    const int64_t total = n * K;
    if (total == 0) return CB_OK;
    const int wpr = (int)((K + 31) / 32) * bits;
    const int threads = 256;
    const int sms = sm_count_current();
    if (sms <= 0) return CB_ERR_CUDA;
    const int64_t blocks = std::min<int64_t>((total + threads - 1) / threads, (int64_t)sms * 16);
    unpack_codes_kernel<<<(int)blocks, threads, 0, stream>>>(reinterpret_cast<const uint32_t*>(packed), n, (int)K,
                                                             wpr, bits, codes);
    CB_CUDA_TRY(cudaGetLastError());
    return CB_OK;
}

}  // namespace cb
