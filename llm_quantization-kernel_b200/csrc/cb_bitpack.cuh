// Device side of the packed bit layout: a row is a little-endian bitstream of 32-bit words with
// code k at bit k*BITS; 32 consecutive codes ("a chunk") occupy exactly BITS words.  The layout is
// the one written by Crispybits/Kernel/crispybits_kernels/reference.py:37-55 and read by
// Crispybits/Kernel/csrc/bitpack.cuh:10-41.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace cb {

// Streaming read-only load: weights are touched once per call, keep them out of L1.
__device__ __forceinline__ uint32_t ld_stream_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_u64(const uint32_t* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_stream_u128(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// The BITS words of one chunk.  W4 chunks are 16 bytes and W2 chunks 8 bytes, and both stay
// aligned to their size when the row base is (rows are whole chunks); W3 chunks are 12 bytes, so
// only 4-byte alignment is guaranteed.
template <int BITS>
__device__ __forceinline__ void load_chunk(const uint32_t* __restrict__ p, uint32_t (&w)[BITS]) {
    if constexpr (BITS == 4) {
        const uint4 v = ld_stream_u128(p);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else if constexpr (BITS == 2) {
        const uint2 v = ld_stream_u64(p);
        w[0] = v.x; w[1] = v.y;
    } else {
        w[0] = ld_stream_u32(p); w[1] = ld_stream_u32(p + 1); w[2] = ld_stream_u32(p + 2);
    }
}

// Code j (0..31) of a chunk held in registers.  With j a compile-time constant (unrolled loops)
// this is one bit-field extract, or one funnel shift + mask for the two 3-bit codes (j = 10, 21)
// that straddle a word boundary.
template <int BITS>
__device__ __forceinline__ uint32_t chunk_code(const uint32_t (&w)[BITS], int j) {
    const int pos = j * BITS, wi = pos >> 5, off = pos & 31;
    constexpr uint32_t mask = (1u << BITS) - 1u;
    if (off + BITS <= 32) return (w[wi] >> off) & mask;
    return __funnelshift_r(w[wi], w[(wi + 1) < BITS ? (wi + 1) : wi], off) & mask;
}

// Small non-negative integer -> float without a conversion instruction: place it in the mantissa
// of 2^23 and subtract 2^23 (exact for q < 2^23).
__device__ __forceinline__ float small_uint_to_float(uint32_t q) {
    return __uint_as_float(q | 0x4B000000u) - 8388608.0f;
}

// Arbitrary code k of a row in global memory (slow path: unpack kernel, SIMT GEMM).
__device__ __forceinline__ uint32_t row_code(const uint32_t* __restrict__ row, int k, int bits) {
    const int pos = k * bits, wi = pos >> 5, off = pos & 31;
    uint32_t v = row[wi] >> off;
    if (off + bits > 32) v |= row[wi + 1] << (32 - off);
    return v & ((1u << bits) - 1u);
}

}  // namespace cb
