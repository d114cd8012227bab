// Group-wise asymmetric affine quantisation and bit-packing of a weight matrix on the GPU: the device
// counterpart of quantize_affine + pack_codes (Crispybits/Kernel/crispybits_kernels/reference.py:10-27 and
// :37-55), producing the same packed words, scales and zeros bit for bit.
//
//   scale = max((max - min) / qmax, 1e-8)      zero = clamp(rint(-min / scale), 0, qmax)
//   q     = clamp(rint(w / scale) + zero, 0, qmax)            (fp32, IEEE division, round-half-even)
// A ragged last group is completed by repeating the last column (reference.py:18-19); codes past K are zero;
// code j of a 32-code chunk sits at bit j*bits of the chunk's little-endian stream of `bits` words.
//
// One warp per (row, group): lanes stride over the group for min / max (shuffle reduction), then every
// 32-code chunk of the group is quantised one code per lane and its words are assembled with a warp-wide
// OR reduction of the lanes' shifted fields.
#include "cb_common.cuh"

namespace cb {
namespace {

template <typename T>
__global__ void __launch_bounds__(256)
quantize_pack_kernel(const T* __restrict__ w, int64_t n, int K, int bits, int gs, int groups, int chunks,
                     uint32_t* __restrict__ packed, void* __restrict__ scales, void* __restrict__ zeros, int meta_dtype) {
    const int lane = threadIdx.x & 31;
    const int64_t nunits = n * (int64_t)groups;
    const float qmax = (float)((1 << bits) - 1);
    for (int64_t unit = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5); unit < nunits;
         unit += (int64_t)gridDim.x * (blockDim.x >> 5)) {
        const int64_t r = unit / groups;
        const int gi = (int)(unit - r * groups);
        const T* wrow = w + r * (int64_t)K;
        const int k0 = gi * gs;
        float mn = INFINITY, mx = -INFINITY;
        for (int j = lane; j < gs; j += 32) {
            const float v = to_f32(wrow[min(k0 + j, K - 1)]);
            mn = fminf(mn, v); mx = fmaxf(mx, v);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        const float scale = fmaxf(__fdiv_rn(mx - mn, qmax), 1e-8f);
        const float zero = fminf(fmaxf(rintf(__fdiv_rn(-mn, scale)), 0.f), qmax);
        if (lane == 0) {
            const int64_t at = r * groups + gi;
            if (meta_dtype == CB_F32) { reinterpret_cast<float*>(scales)[at] = scale; reinterpret_cast<float*>(zeros)[at] = zero; }
            else if (meta_dtype == CB_F16) {
                reinterpret_cast<__half*>(scales)[at] = __float2half_rn(scale); reinterpret_cast<__half*>(zeros)[at] = __float2half_rn(zero);
            } else {
                reinterpret_cast<__nv_bfloat16*>(scales)[at] = __float2bfloat16_rn(scale);
                reinterpret_cast<__nv_bfloat16*>(zeros)[at] = __float2bfloat16_rn(zero);
            }
        }
        // this lane's field inside a chunk's stream
        const int pos = lane * bits, wi0 = pos >> 5, off = pos & 31;
        const bool spills = off + bits > 32;
        for (int c = 0; c < gs / 32; ++c) {
            const int chunk = (k0 >> 5) + c;
            if (chunk >= chunks) break;                      // warp-uniform
            const int k = k0 + 32 * c + lane;
            uint32_t q = 0u;
            if (k < K) q = (uint32_t)fminf(fmaxf(rintf(__fdiv_rn(to_f32(wrow[k]), scale)) + zero, 0.f), qmax);
            for (int wd = 0; wd < bits; ++wd) {
                uint32_t contrib = 0u;
                if (wi0 == wd) contrib = q << off;
                if (spills && wi0 + 1 == wd) contrib |= q >> (32 - off);
                const uint32_t word = __reduce_or_sync(0xffffffffu, contrib);
                if (lane == wd) packed[r * (int64_t)chunks * bits + (int64_t)chunk * bits + wd] = word;
            }
        }
    }
}

}  // namespace

int launch_quantize_pack(const void* w, int w_dtype, int64_t n, int64_t K, int bits, int64_t gs, int32_t* packed,
                         void* scales, void* zeros, int meta_dtype, cudaStream_t stream) {
    const int groups = (int)((K + gs - 1) / gs), chunks = (int)((K + 31) / 32);
    const int sms = sm_count_current();
    if (sms <= 0) return CB_ERR_CUDA;
    const int64_t units = n * (int64_t)groups;
    const int blocks = (int)std::min<int64_t>((units + 7) / 8, (int64_t)sms * 8);
    uint32_t* p = reinterpret_cast<uint32_t*>(packed);
    if (w_dtype == CB_F32)
        quantize_pack_kernel<float><<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(w), n, (int)K, bits, (int)gs, groups, chunks, p, scales, zeros, meta_dtype);
    else if (w_dtype == CB_F16)
        quantize_pack_kernel<__half><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __half*>(w), n, (int)K, bits, (int)gs, groups, chunks, p, scales, zeros, meta_dtype);
    else
        quantize_pack_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(w), n, (int)K, bits, (int)gs, groups, chunks, p, scales, zeros, meta_dtype);
    CB_CUDA_TRY(cudaGetLastError());
    return CB_OK;
}

}  // namespace cb
