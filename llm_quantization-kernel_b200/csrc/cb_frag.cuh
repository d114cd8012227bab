// Register-level pieces shared by the fp16 decode kernels: packed words -> exact fp16 integers in the
// operand order of mma.sync m16n8k16, and the MMA itself.
#pragma once
#include "cb_common.cuh"

namespace cb {

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
    return r;
}
__device__ __forceinline__ uint32_t h2fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t h2add(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t a0, const uint32_t a1, const uint32_t a2,
                                         const uint32_t a3, const uint32_t b0, const uint32_t b1, const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

constexpr uint32_t kMagic = 0x64006400u;      // half2(1024, 1024)

__device__ __forceinline__ uint32_t h2sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// The 32 codes of one chunk -> 16 half2 registers holding the exact integers (code - zero).  e[m] holds
// the code pair (pair_lo(m), pair_lo(m) + pair_gap()) in its (low, high) half.  A field that sits at
// bit p of a half is extracted in place: (w & mask) | 0x6400 reads as 1024 + code * 2^p, and one
// fused multiply-add with 2^-p and the constant -(1024 * 2^-p + zero) leaves code - zero, exactly.
// `consts()` prepares those constants for one (row, group) from the group's zero point.
template <int BITS> struct Unpack;

template <> struct Unpack<4> {
    static constexpr int kConsts = 2;
    __device__ static __forceinline__ int pair_lo(int m) { return 8 * (m >> 2) + (m & 3); }   // word i: e[4i+j] = (8i+j, 8i+j+4)
    __device__ static __forceinline__ int pair_gap() { return 4; }
    __device__ static __forceinline__ void consts(uint32_t zz, uint32_t (&k)[kConsts]) {
        k[0] = h2sub(0xE400E400u, zz);     // -(1024 + z)
        k[1] = h2sub(0xD400D400u, zz);     // -(64 + z)
    }
    __device__ static __forceinline__ void run(const uint32_t (&w)[4], const uint32_t (&k)[kConsts], uint32_t (&e)[16]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t lo = w[i], hi = w[i] >> 8;
            e[4 * i + 0] = h2add(lop3_and_or(lo, 0x000F000Fu, kMagic), k[0]);
            e[4 * i + 1] = h2fma(lop3_and_or(lo, 0x00F000F0u, kMagic), 0x2C002C00u, k[1]);   // * 1/16
            e[4 * i + 2] = h2add(lop3_and_or(hi, 0x000F000Fu, kMagic), k[0]);
            e[4 * i + 3] = h2fma(lop3_and_or(hi, 0x00F000F0u, kMagic), 0x2C002C00u, k[1]);
        }
    }
};

template <> struct Unpack<2> {
    static constexpr int kConsts = 5;
    __device__ static __forceinline__ int pair_lo(int m) { return 16 * (m >> 3) + (m & 7); }  // word i: e[8i+j] = (16i+j, 16i+j+8)
    __device__ static __forceinline__ int pair_gap() { return 8; }
    __device__ static __forceinline__ void consts(uint32_t zz, uint32_t (&k)[kConsts]) {
        k[0] = h2sub(0xE400E400u, zz);     // -(1024 + z)
        k[1] = h2sub(0xDC00DC00u, zz);     // -(256 + z)
        k[2] = h2sub(0xD400D400u, zz);     // -(64 + z)
        k[3] = h2sub(0xCC00CC00u, zz);     // -(16 + z)
        k[4] = h2sub(0xC400C400u, zz);     // -(4 + z)
    }
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], const uint32_t (&k)[kConsts], uint32_t (&e)[16]) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t lo = w[i], hi = w[i] >> 10;
            e[8 * i + 0] = h2add(lop3_and_or(lo, 0x00030003u, kMagic), k[0]);
            e[8 * i + 1] = h2fma(lop3_and_or(lo, 0x000C000Cu, kMagic), 0x34003400u, k[1]);   // * 1/4
            e[8 * i + 2] = h2fma(lop3_and_or(lo, 0x00300030u, kMagic), 0x2C002C00u, k[2]);   // * 1/16
            e[8 * i + 3] = h2fma(lop3_and_or(lo, 0x00C000C0u, kMagic), 0x24002400u, k[3]);   // * 1/64
            e[8 * i + 4] = h2fma(lop3_and_or(lo, 0x03000300u, kMagic), 0x1C001C00u, k[4]);   // * 1/256
            e[8 * i + 5] = h2add(lop3_and_or(hi, 0x00030003u, kMagic), k[0]);
            e[8 * i + 6] = h2fma(lop3_and_or(hi, 0x000C000Cu, kMagic), 0x34003400u, k[1]);
            e[8 * i + 7] = h2fma(lop3_and_or(hi, 0x00300030u, kMagic), 0x2C002C00u, k[2]);
        }
    }
};

template <> struct Unpack<3> {
    // e[j] = (code j, code j+16): the chunk is a 96-bit stream; code j sits at bit 3j, code j+16 at bit
    // 3j+48.  Windows of 15 bits (5 codes) of both halves are brought side by side into one register
    // with funnel shifts (which also reassemble the codes that straddle a word) and a byte permute.
    static constexpr int kConsts = 3;
    __device__ static __forceinline__ int pair_lo(int m) { return m; }
    __device__ static __forceinline__ int pair_gap() { return 16; }
    __device__ static __forceinline__ void consts(uint32_t zz, uint32_t (&k)[kConsts]) {
        k[0] = h2sub(0xE400E400u, zz);     // -(1024 + z)
        k[1] = h2sub(0xD800D800u, zz);     // -(128 + z)
        k[2] = h2sub(0xCC00CC00u, zz);     // -(16 + z)
    }
    __device__ static __forceinline__ void five(uint32_t p, const uint32_t (&k)[kConsts], uint32_t* e) {
        const uint32_t q = p >> 9;
        e[0] = h2add(lop3_and_or(p, 0x00070007u, kMagic), k[0]);
        e[1] = h2fma(lop3_and_or(p, 0x00380038u, kMagic), 0x30003000u, k[1]);   // * 1/8
        e[2] = h2fma(lop3_and_or(p, 0x01C001C0u, kMagic), 0x24002400u, k[2]);   // * 1/64
        e[3] = h2add(lop3_and_or(q, 0x00070007u, kMagic), k[0]);
        e[4] = h2fma(lop3_and_or(q, 0x00380038u, kMagic), 0x30003000u, k[1]);
    }
    __device__ static __forceinline__ void run(const uint32_t (&w)[3], const uint32_t (&k)[kConsts], uint32_t (&e)[16]) {
        // stream bits [s, s+16) of the first half next to bits [48+s, 48+s+16) of the second half
        const uint32_t l1 = __funnelshift_r(w[0], w[1], 15), l2 = __funnelshift_r(w[0], w[1], 30);
        const uint32_t u0 = __funnelshift_r(w[1], w[2], 16), u1 = __funnelshift_r(w[1], w[2], 31), u2 = w[2] >> 14;
        five(__byte_perm(w[0], u0, 0x5410), k, e);
        five(__byte_perm(l1, u1, 0x5410), k, e + 5);
        five(__byte_perm(l2, u2, 0x5410), k, e + 10);
        const uint32_t last = __byte_perm(w[1] >> 13, w[2] >> 29, 0x5410);               // codes 15 and 31
        e[15] = h2add(lop3_and_or(last, 0x00070007u, kMagic), k[0]);
    }
};

// ---- bfloat16 counterparts ----------------------------------------------------------------------------------------
// bf16 has seven mantissa bits: (field | 0x4300) reads as 128 + code * 2^p exactly only while code * 2^p <= 127, so
// fields are taken at low bit positions after a few more shifts than the fp16 versions need.  Pairings (which
// two codes share a register) are those of the fp16 versions, so the activation fragments are built the same way.
__device__ __forceinline__ uint32_t b2fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t b2sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ void mma16816_bf16(float (&d)[4], const uint32_t a0, const uint32_t a1, const uint32_t a2,
                                              const uint32_t a3, const uint32_t b0, const uint32_t b1, const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

constexpr uint32_t kMagicB = 0x43004300u;     // bf16x2(128, 128)
constexpr uint32_t kOneB = 0x3F803F80u;       // bf16x2(1, 1)

template <int BITS> struct UnpackB;

template <> struct UnpackB<4> {
    static constexpr int kConsts = 1;
    __device__ static __forceinline__ int pair_lo(int m) { return 8 * (m >> 2) + (m & 3); }
    __device__ static __forceinline__ int pair_gap() { return 4; }
    __device__ static __forceinline__ void consts(uint32_t zz, uint32_t (&k)[kConsts]) {
        k[0] = b2sub(0xC300C300u, zz);     // -(128 + z): at most 143, exact in eight significant bits
    }
    __device__ static __forceinline__ void run(const uint32_t (&w)[4], const uint32_t (&k)[kConsts], uint32_t (&e)[16]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < 4; ++j)      // nibble j of the low half with nibble j of the high half: codes 8i+j, 8i+j+4
                e[4 * i + j] = b2fma(lop3_and_or(w[i] >> (4 * j), 0x000F000Fu, kMagicB), kOneB, k[0]);
        }
    }
};

template <> struct UnpackB<2> {
    static constexpr int kConsts = 3;
    __device__ static __forceinline__ int pair_lo(int m) { return 16 * (m >> 3) + (m & 7); }
    __device__ static __forceinline__ int pair_gap() { return 8; }
    __device__ static __forceinline__ void consts(uint32_t zz, uint32_t (&k)[kConsts]) {
        k[0] = b2sub(0xC300C300u, zz);     // -(128 + z)
        k[1] = b2sub(0xC200C200u, zz);     // -(32 + z)
        k[2] = b2sub(0xC100C100u, zz);     // -(8 + z)
    }
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], const uint32_t (&k)[kConsts], uint32_t (&e)[16]) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t v0 = w[i], v1 = w[i] >> 6, v2 = w[i] >> 12;       // fields 0-2, 3-5, 6-7 of each half at bits 0, 2, 4
            e[8 * i + 0] = b2fma(lop3_and_or(v0, 0x00030003u, kMagicB), kOneB, k[0]);
            e[8 * i + 1] = b2fma(lop3_and_or(v0, 0x000C000Cu, kMagicB), 0x3E803E80u, k[1]);   // * 1/4
            e[8 * i + 2] = b2fma(lop3_and_or(v0, 0x00300030u, kMagicB), 0x3D803D80u, k[2]);   // * 1/16
            e[8 * i + 3] = b2fma(lop3_and_or(v1, 0x00030003u, kMagicB), kOneB, k[0]);
            e[8 * i + 4] = b2fma(lop3_and_or(v1, 0x000C000Cu, kMagicB), 0x3E803E80u, k[1]);
            e[8 * i + 5] = b2fma(lop3_and_or(v1, 0x00300030u, kMagicB), 0x3D803D80u, k[2]);
            e[8 * i + 6] = b2fma(lop3_and_or(v2, 0x00030003u, kMagicB), kOneB, k[0]);
            e[8 * i + 7] = b2fma(lop3_and_or(v2, 0x000C000Cu, kMagicB), 0x3E803E80u, k[1]);
        }
    }
};

template <> struct UnpackB<3> {
    // Same windows as Unpack<3> (stream bits [s, s+16) beside [48+s, 48+s+16)); a window gives its five codes at
    // bits 0 and 3 of three 6-bit steps.
    static constexpr int kConsts = 2;
    __device__ static __forceinline__ int pair_lo(int m) { return m; }
    __device__ static __forceinline__ int pair_gap() { return 16; }
    __device__ static __forceinline__ void consts(uint32_t zz, uint32_t (&k)[kConsts]) {
        k[0] = b2sub(0xC300C300u, zz);     // -(128 + z)
        k[1] = b2sub(0xC180C180u, zz);     // -(16 + z)
    }
    __device__ static __forceinline__ void five(uint32_t p, const uint32_t (&k)[kConsts], uint32_t* e) {
        const uint32_t q = p >> 6, r = p >> 12;
        e[0] = b2fma(lop3_and_or(p, 0x00070007u, kMagicB), kOneB, k[0]);
        e[1] = b2fma(lop3_and_or(p, 0x00380038u, kMagicB), 0x3E003E00u, k[1]);   // * 1/8
        e[2] = b2fma(lop3_and_or(q, 0x00070007u, kMagicB), kOneB, k[0]);
        e[3] = b2fma(lop3_and_or(q, 0x00380038u, kMagicB), 0x3E003E00u, k[1]);
        e[4] = b2fma(lop3_and_or(r, 0x00070007u, kMagicB), kOneB, k[0]);
    }
    __device__ static __forceinline__ void run(const uint32_t (&w)[3], const uint32_t (&k)[kConsts], uint32_t (&e)[16]) {
        const uint32_t l1 = __funnelshift_r(w[0], w[1], 15), l2 = __funnelshift_r(w[0], w[1], 30);
        const uint32_t u0 = __funnelshift_r(w[1], w[2], 16), u1 = __funnelshift_r(w[1], w[2], 31), u2 = w[2] >> 14;
        five(__byte_perm(w[0], u0, 0x5410), k, e);
        five(__byte_perm(l1, u1, 0x5410), k, e + 5);
        five(__byte_perm(l2, u2, 0x5410), k, e + 10);
        const uint32_t last = __byte_perm(w[1] >> 13, w[2] >> 29, 0x5410);               // codes 15 and 31
        e[15] = b2fma(lop3_and_or(last, 0x00070007u, kMagicB), kOneB, k[0]);
    }
};

// Even split of n items into `parts`: part i starts at i*q + min(i, r) with q = n / parts, r = n % parts
// (q and r come from the host, so the kernel does no division on its way to the first copy).
__device__ __forceinline__ int split_begin(int i, int q, int r) { return i * q + min(i, r); }

}  // namespace cb
