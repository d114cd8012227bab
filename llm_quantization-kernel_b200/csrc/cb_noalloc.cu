// cb_packed_gemv_static_scratch: the Split-K decode GEMV for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc (or any allocating routine) on the path that
// issues kernels: a serving loop that has handed all device memory to its own arena, a plugin that
// runs under an allocator it does not control, code that runs between the nodes of a captured
// region.  The ordinary entry point asks such a caller to bring its own scratch buffer; this one
// brings the scratch with the library instead, as a fixed array in device memory.
//
// The array below is a file-scope __device__ object: every GPU that loads the library holds
// kStaticScratchBytes of it until the process exits.  In host code its NAME is only a handle; the
// device address is obtained once per device with cudaGetSymbolAddress and that pointer is what the
// kernel receives.  The address is remembered for the life of the process: a caller that destroys the
// device's primary context (cudaDeviceReset) must not use this entry point afterwards.
#include <mutex>

#include "cb_common.cuh"

namespace cb {
namespace {

// Same layout as caller-provided scratch: 256 KiB of arrival counters, then the partial sums.
constexpr size_t kStaticCounterBytes = 65536 * sizeof(int);
constexpr size_t kStaticPartialBytes = 1u << 20;   // room for split_k * B * V <= 262144 floats
constexpr size_t kStaticScratchBytes = kStaticCounterBytes + kStaticPartialBytes;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_ptr[kMaxDevices];   // device address of g_static_scratch on each device, once resolved

// Resolve (once per device, with that device current) the device address of the array.
int static_scratch_address(void** out) {
    int dev = 0;
    CB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        set_error("packed_gemv_static_scratch: device ordinal %d out of range", dev);
        return CB_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        CB_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return CB_OK;
}

}  // namespace
}  // namespace cb

extern "C" {

size_t cb_static_scratch_bytes(void) { return cb::kStaticScratchBytes; }

int cb_packed_gemv_static_scratch(const void* x, int64_t B, const cb_weight* w, void* out, int64_t K, int bits,
                                  int64_t group_size, int dtype, int64_t split_k, int64_t rho, int act,
                                  void* stream) {
    using namespace cb;
    if (w == nullptr || B < 0 || K <= 0 || split_k < 1) {
        set_error("packed_gemv_static_scratch: bad arguments");
        return CB_ERR_INVALID;
    }
    const int64_t nchunks = (K + 31) / 32;
    const int64_t pk = split_k < nchunks ? split_k : nchunks;
    const int64_t tiles = ((B + kMaxBatchBlock - 1) / kMaxBatchBlock) * ((w->n + kTileN - 1) / kTileN);
    if (pk > 1 && tiles > 65536) {
        set_error("packed_gemv_static_scratch: ceil(B/8)*ceil(N/16) = %lld exceeds the 65536 arrival counters of the "
                  "built-in array; call with split_k = 1 or use cb_packed_gemv", (long long)tiles);
        return CB_ERR_INVALID;
    }
    const size_t need = cb_gemv_scratch_bytes(B, w->n, pk);
    if (need > kStaticScratchBytes) {
        set_error("packed_gemv_static_scratch: split_k=%lld x batch=%lld x rows=%lld needs %zu bytes of scratch; the "
                  "built-in array holds %zu (split_k*B*N <= 262144). Lower split_k or use cb_packed_gemv with your "
                  "own buffer", (long long)pk, (long long)B, (long long)w->n, need, kStaticScratchBytes);
        return CB_ERR_INVALID;
    }
    void* scratch = nullptr;
    if (need > 0) {
        const int rc = static_scratch_address(&scratch);
        if (rc != CB_OK) return rc;
        // The array keeps whatever the previous call (or a call that was cut short) left behind.
        // Only the arrival counters have to start at zero; partial sums are fully overwritten.
        const size_t counters = (size_t)((B + kMaxBatchBlock - 1) / kMaxBatchBlock) *
                                (size_t)((w->n + kTileN - 1) / kTileN) * sizeof(int);
        CB_CUDA_TRY(cudaMemsetAsync(scratch, 0, counters, reinterpret_cast<cudaStream_t>(stream)));
    }
    return cb_packed_gemv(x, B, w, out, K, bits, group_size, dtype, pk, rho, act, scratch,
                          need > 0 ? kStaticScratchBytes : 0, stream);
}

}  // extern "C"
