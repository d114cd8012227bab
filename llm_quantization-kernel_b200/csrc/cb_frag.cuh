// Register-level pieces of the decode ring kernel: packed words -> MMA A operands in the operand order of
// mma.sync m16n8k16, and the MMA itself.
#pragma once
#include "cb_common.cuh"

namespace cb {

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
    return r;
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t a0, const uint32_t a1, const uint32_t a2,
                                         const uint32_t a3, const uint32_t b0, const uint32_t b1, const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

constexpr uint32_t kMagic = 0x64006400u;      // half2(1024, 1024)

__device__ __forceinline__ void mma16816_bf16(float (&d)[4], const uint32_t a0, const uint32_t a1, const uint32_t a2,
                                              const uint32_t a3, const uint32_t b0, const uint32_t b1, const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

constexpr uint32_t kMagicB = 0x43004300u;     // bf16x2(128, 128)

// ---- offset-free operands for the ring kernel ----------------------------------------------------------------------
// Frag<BITS, KIND>::run turns one 32-code chunk into 16 MMA A registers with ONE logic instruction per code pair and
// no arithmetic: register m holds the code pair (pair_lo(m), pair_lo(m) + pair_gap()) as the two numbers
//     base + code * 2^shift(m) * unit          (low half, high half)
// and the kernel multiplies the matching activations by 2^-shift(m) once per group (exact: a power of two), so that
// the MMA yields  base * sum(x * 2^-shift) + unit * sum(code * x).
//   KIND 0 (fp16): the masked field is used as it stands.  With a zero exponent field an fp16 bit pattern is a
//           subnormal number, field * 2^-24: base = 0, unit = 2^-24, nothing to subtract afterwards.  A field must
//           lie inside the ten mantissa bits.
//   KIND 1 (fp16): (field | 0x6400) = 1024 + field: base = 1024, unit = 1 (the kernel subtracts base * sum(x')).
//   KIND 2 (bf16): (field | 0x4300) = 128 + field, fields inside the seven mantissa bits: base = 128, unit = 1.
// The zero point is not touched here either: per group the kernel uses  s * (sum(code * x) - z * sum(x)).
constexpr int kFragSubnormal = 0, kFragMagicH = 1, kFragMagicB = 2;

template <int KIND> struct FragKind {
    static constexpr bool kBf = KIND == kFragMagicB;
    static constexpr float kBase = KIND == kFragSubnormal ? 0.f : (KIND == kFragMagicH ? 1024.f : 128.f);
    static constexpr float kInvUnit = KIND == kFragSubnormal ? 16777216.f : 1.f;      // 1 / unit
    static constexpr uint32_t kOnes = kBf ? 0x3F803F80u : 0x3C003C00u;                 // (1, 1) in the operand type
    __device__ static __forceinline__ uint32_t field(uint32_t v, uint32_t mask) {
        if constexpr (KIND == kFragSubnormal) return v & mask;
        else return lop3_and_or(v, mask, KIND == kFragMagicH ? kMagic : kMagicB);
    }
    // (2^-e, 2^-e) in the operand type
    __device__ static __forceinline__ constexpr uint32_t pow2neg(int e) {
        return kBf ? (uint32_t)(((127 - e) << 7) * 0x10001u) : (uint32_t)(((15 - e) << 10) * 0x10001u);
    }
    // (2^-lo, 2^-hi) in the operand type: low half first
    __device__ static __forceinline__ constexpr uint32_t pow2neg2(int lo, int hi) {
        return kBf ? (uint32_t)((127 - lo) << 7) | ((uint32_t)((127 - hi) << 7) << 16)
                   : (uint32_t)((15 - lo) << 10) | ((uint32_t)((15 - hi) << 10) << 16);
    }
    __device__ static __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
        uint32_t r;
        if constexpr (kBf) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        else asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
};

template <int BITS, int KIND> struct Frag;

template <int KIND> struct Frag<4, KIND> : FragKind<KIND> {
    using F = FragKind<KIND>;
    __device__ static __forceinline__ constexpr int pair_lo(int m) { return 8 * (m >> 2) + (m & 3); }   // word i: e[4i+j] = (8i+j, 8i+j+4)
    __device__ static __forceinline__ constexpr int pair_hi(int m) { return pair_lo(m) + 4; }
    __device__ static __forceinline__ constexpr int shift(int m) { return F::kBf ? 0 : ((m & 1) ? 4 : 0); }
    // what the activations of pair m are multiplied by when they are staged: (2^-p, 2^-p') for fields at bits p, 16 + p'
    __device__ static __forceinline__ constexpr uint32_t scale2(int m) { return F::pow2neg2(shift(m), shift(m)); }
    __device__ static __forceinline__ void run(const uint32_t (&w)[4], uint32_t (&e)[16]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if constexpr (F::kBf) {
#pragma unroll
                for (int j = 0; j < 4; ++j) e[4 * i + j] = F::field(w[i] >> (4 * j), 0x000F000Fu);
            } else {
                const uint32_t lo = w[i], hi = w[i] >> 8;
                e[4 * i + 0] = F::field(lo, 0x000F000Fu);
                e[4 * i + 1] = F::field(lo, 0x00F000F0u);
                e[4 * i + 2] = F::field(hi, 0x000F000Fu);
                e[4 * i + 3] = F::field(hi, 0x00F000F0u);
            }
        }
    }
};

template <int KIND> struct Frag<2, KIND> : FragKind<KIND> {
    using F = FragKind<KIND>;
    __device__ static __forceinline__ constexpr int pair_lo(int m) { return 16 * (m >> 3) + (m & 7); }  // word i: e[8i+j] = (16i+j, 16i+j+8)
    __device__ static __forceinline__ constexpr int pair_hi(int m) { return pair_lo(m) + 8; }
    __device__ static __forceinline__ constexpr int shift(int m) {
        const int j = m & 7;
        return F::kBf ? 2 * (j % 3) : (j < 5 ? 2 * j : 2 * (j - 5));
    }
    __device__ static __forceinline__ constexpr uint32_t scale2(int m) { return F::pow2neg2(shift(m), shift(m)); }
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t (&e)[16]) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if constexpr (F::kBf) {
                const uint32_t v0 = w[i], v1 = w[i] >> 6, v2 = w[i] >> 12;    // fields 0-2, 3-5, 6-7 of each half at bits 0, 2, 4
                e[8 * i + 0] = F::field(v0, 0x00030003u);
                e[8 * i + 1] = F::field(v0, 0x000C000Cu);
                e[8 * i + 2] = F::field(v0, 0x00300030u);
                e[8 * i + 3] = F::field(v1, 0x00030003u);
                e[8 * i + 4] = F::field(v1, 0x000C000Cu);
                e[8 * i + 5] = F::field(v1, 0x00300030u);
                e[8 * i + 6] = F::field(v2, 0x00030003u);
                e[8 * i + 7] = F::field(v2, 0x000C000Cu);
            } else {
                const uint32_t lo = w[i], hi = w[i] >> 10;                   // fields 0-4 in place, fields 5-7 at bits 0, 2, 4
                e[8 * i + 0] = F::field(lo, 0x00030003u);
                e[8 * i + 1] = F::field(lo, 0x000C000Cu);
                e[8 * i + 2] = F::field(lo, 0x00300030u);
                e[8 * i + 3] = F::field(lo, 0x00C000C0u);
                e[8 * i + 4] = F::field(lo, 0x03000300u);
                e[8 * i + 5] = F::field(hi, 0x00030003u);
                e[8 * i + 6] = F::field(hi, 0x000C000Cu);
                e[8 * i + 7] = F::field(hi, 0x00300030u);
            }
        }
    }
};

template <int KIND> struct Frag<3, KIND> : FragKind<KIND> {
    // The chunk is a 96-bit stream with code j at bit 3j.
    //
    // fp16 subnormal operands (KIND 0).  A field may sit anywhere in bits 0..10 of its half (values with exponent field
    // 0 or 1 are linear in the bit pattern), and the two codes of a register need not be 16 positions apart: the
    // activations are arranged to match.  So six windows of the stream -- one word as it is, three funnel shifts, two
    // shifts -- hold all 32 codes with three (two) low-half and three (two) high-half fields each, and 16 ANDs finish:
    //   w0               codes (0,6) (1,7) (2,8)          low fields at bits 0, 3, 6; high fields at 16 + 2, 5, 8
    //   stream >> 9      codes (3,9) (4,10) (5,11)        the same masks
    //   stream >> 36     codes (12,18) (13,19) (14,20)
    //   stream >> 45     codes (15,21) (16,22) (17,23)
    //   w2 >> 4          codes (24,28) (25,29)            low fields at bits 4, 7; high fields at 16 + 0, 3
    //   w2 >> 10         codes (26,30) (27,31)
    // 21 integer instructions per 32 codes.
    //
    // Offset operands (KIND 1, 2).  e[j] = (code j, code j+16): windows of 15 bits (5 codes) of both halves are brought
    // side by side into one register with funnel shifts (which also reassemble the codes that straddle a word) and a
    // byte permute; fields stay inside the mantissa of the offset.  30 instructions per 32 codes.
    using F = FragKind<KIND>;
    static constexpr bool kWindows = KIND == kFragSubnormal;
    __device__ static __forceinline__ constexpr int pair_lo(int m) {
        if (!kWindows) return m;
        return m < 12 ? 12 * (m / 6) + (m % 6) : 24 + (m - 12);           // 0..5, 12..17, 24..27
    }
    __device__ static __forceinline__ constexpr int pair_hi(int m) {
        if (!kWindows) return m + 16;
        return m < 12 ? pair_lo(m) + 6 : pair_lo(m) + 4;
    }
    __device__ static __forceinline__ constexpr int shift(int m) {
        if (m == 15) return 0;
        const int j = m % 5;
        return F::kBf ? 3 * (j & 1) : (j < 3 ? 3 * j : 3 * (j - 3));
    }
    __device__ static __forceinline__ constexpr uint32_t scale2(int m) {
        if (!kWindows) return F::pow2neg2(shift(m), shift(m));
        if (m < 12) return F::pow2neg2(3 * (m % 3), 2 + 3 * (m % 3));
        return (m & 1) ? F::pow2neg2(7, 3) : F::pow2neg2(4, 0);
    }
    __device__ static __forceinline__ void five(uint32_t p, uint32_t* e) {
        if constexpr (F::kBf) {
            const uint32_t q = p >> 6, r = p >> 12;
            e[0] = F::field(p, 0x00070007u);
            e[1] = F::field(p, 0x00380038u);
            e[2] = F::field(q, 0x00070007u);
            e[3] = F::field(q, 0x00380038u);
            e[4] = F::field(r, 0x00070007u);
        } else {
            const uint32_t q = p >> 9;
            e[0] = F::field(p, 0x00070007u);
            e[1] = F::field(p, 0x00380038u);
            e[2] = F::field(p, 0x01C001C0u);
            e[3] = F::field(q, 0x00070007u);
            e[4] = F::field(q, 0x00380038u);
        }
    }
    __device__ static __forceinline__ void run(const uint32_t (&w)[3], uint32_t (&e)[16]) {
        if constexpr (kWindows) {
            const uint32_t win[4] = {w[0], __funnelshift_r(w[0], w[1], 9), __funnelshift_r(w[1], w[2], 4),
                                     __funnelshift_r(w[1], w[2], 13)};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                e[3 * i + 0] = win[i] & 0x001C0007u;
                e[3 * i + 1] = win[i] & 0x00E00038u;
                e[3 * i + 2] = win[i] & 0x070001C0u;
            }
            const uint32_t t4 = w[2] >> 4, t10 = w[2] >> 10;
            e[12] = t4 & 0x00070070u;
            e[13] = t4 & 0x00380380u;
            e[14] = t10 & 0x00070070u;
            e[15] = t10 & 0x00380380u;
        } else {
            // stream bits [s, s+16) of the first half next to bits [48+s, 48+s+16) of the second half
            const uint32_t l1 = __funnelshift_r(w[0], w[1], 15), l2 = __funnelshift_r(w[0], w[1], 30);
            const uint32_t u0 = __funnelshift_r(w[1], w[2], 16), u1 = __funnelshift_r(w[1], w[2], 31), u2 = w[2] >> 14;
            five(__byte_perm(w[0], u0, 0x5410), e);
            five(__byte_perm(l1, u1, 0x5410), e + 5);
            five(__byte_perm(l2, u2, 0x5410), e + 10);
            const uint32_t last = __byte_perm(w[1] >> 13, w[2] >> 29, 0x5410);               // codes 15 and 31
            e[15] = F::field(last, 0x00070007u);
        }
    }
};

// Even split of n items into `parts`: part i starts at i*q + min(i, r) with q = n / parts, r = n % parts
// (q and r come from the host, so the kernel does no division on its way to the first copy).
__device__ __forceinline__ int split_begin(int i, int q, int r) { return i * q + min(i, r); }

}  // namespace cb
