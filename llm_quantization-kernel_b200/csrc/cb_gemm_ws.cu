// Prefill GEMM on tcgen05 with the dequantised weights held in tensor memory ("weight-stationary").
//
//   out[M, N] = act( x[M, K] * Wdq[N, K]^T + bias ),   Wdq = round_fp16((q - zero) * scale)
//
// Same numerics as the shared-memory-operand kernel (Crispybits/Kernel/csrc/packed_gemm.cu:47-61: weight
// rounded to the storage type before the product, fp32 accumulation).  What differs is where the expanded
// weights live.  With both MMA operands in shared memory, one SM's shared-memory port carries the TMA
// writes of x, the dequantisers' stores, and the tensor core's reads of both operands -- about 135 KB per
// 64-code stage, which at 128 bytes per cycle is as long as the MMAs themselves and was measured to bound
// the kernel.  Here the product is computed transposed, D[n, m] = sum_k Wdq[n, k] * x[m, k]:
//   * the weight tile is the A operand and is read from TENSOR MEMORY: the dequantiser of weight row n
//     writes its fp16 values with tcgen05.st into TMEM lane n -- they never touch shared memory;
//   * the activation tile (256 tokens x 64 codes, TMA, 128-byte swizzle) is the B operand from shared memory;
//   * the accumulator is 128 weight rows (lanes) x 256 tokens (columns) of fp32 in TMEM, so each packed word is
//     expanded once per 256 tokens.
// TMEM map (512 columns): [0, 256) accumulator, [256 + 32 s, 256 + 32 s + 32) A stage s (64 fp16 per lane).
//
// One persistent CTA per SM, 27 warps: warp 0 TMA producer of x; warp 1 TMEM owner and MMA issuer
// (kind::f16, 128 x 256 x 16, four per stage); warps 2-17 dequantisers (TMEM lane quadrant = warp % 4, the
// four warps of a quadrant take 16 codes each of the stage's 64); warps 18-25 epilogue, two per lane quadrant
// (tcgen05.ld of their quadrant, bias, activation, fp16 stores: lane = weight row, so the 32 lanes of a store are
// 64 contiguous bytes of one token's output row; there is one accumulator, so the drain is not overlapped with the
// next tile's MMAs, and eight warps instead of four were measured 5-17 % faster end to end); warp 26 TMA producer
// of the packed words (128 rows x 128 codes per box).
// Every mbarrier wait is bounded; a wait that runs out raises a flag in shared memory and in the status word,
// every role leaves its loops, TMEM is released, and the kernel returns.
#include <algorithm>

#include <cuda.h>

#include "cb_common.cuh"

namespace cb {
namespace {

constexpr int kBN = 128;                            // weight rows per tile (UMMA M)
constexpr int kBT = 256;                            // tokens per tile (UMMA N)
constexpr int kBK = 64;                             // codes per stage
constexpr int kStages = 6;
constexpr int kPackedSlots = 4;                     // ring of packed super-blocks (128 codes = two stages each)
constexpr int kEpiWarps = 8;                        // two per TMEM lane quadrant, each draining every other 32-column chunk
constexpr int kDequantWarps = 16, kFirstDequantWarp = 2, kFirstEpiWarp = 18, kPackedWarp = kFirstEpiWarp + kEpiWarps;
constexpr int kThreads = (kPackedWarp + 1) * 32;
constexpr uint32_t kXBytes = kBT * kBK * 2;         // 32 KB: one stage of activations
constexpr uint32_t kPackedSlotBytes = kBN * 64;     // 128 rows x 128 codes at 4 bits; narrower rows use less of it
constexpr uint32_t kSmemBytes = kStages * kXBytes + kPackedSlots * kPackedSlotBytes + 1024 /*align*/ + 256 /*barriers*/;
constexpr uint32_t kAccCols = 256, kAStageCols = 32;
constexpr long long kWaitCycles = 2000000000ll;     // about a second at boost clock
// instruction descriptor: fp32 accumulator, A and B both fp16 (format 0) or both bf16 (format 1), K-major, N = 256, M = 128
constexpr uint32_t kIdescF16 = (1u << 4) | ((uint32_t)(kBT >> 3) << 17) | ((uint32_t)(kBN >> 4) << 24);
constexpr uint32_t kIdescBF16 = kIdescF16 | (1u << 7) | (1u << 10);

__device__ int g_gemm_ws_status;   // 0 = ok, else the role that gave up waiting (1 x producer, 2 mma, 3 dequant, 4 epilogue, 5 packed producer)

// Fused Q/K/V only: projections 2 and 3 (K, V); GemmParams' scales / zeros / scales2 / zeros2 / bias / out are Q's and
// K's.  A kernel parameter of its own: with these fields inside GemmParams the compiler generated other code for the
// plain kernel (80 instead of 72 registers), measured a fifth slower on shapes with several tiles per CTA.
struct QkvParams {
    const __half* scales3; const __half* zeros3; const __half* bias2; const __half* bias3; __half* out2; __half* out3;
    int n1, n2, n3;                                  // rows of Q, K, V (each a multiple of 128)
    const float* rope_cos; const float* rope_sin;    // [M, head_dim] fp32 or nullptr
    int head_dim, perm_hd;
};

struct GemmParams {
    const __half* scales; const __half* zeros; const __half* bias; __half* out;
    const __half* scales2; const __half* zeros2;     // fused gate/up: the up projection's metadata (scales / zeros are the gate's)
    int M, N, K, groups, group_size, act;
    int tiles_m, tiles_n, kblocks;
    // K split (plain mode only): a work item is (tile, one of `splits` ranges of `kper` stages); with splits > 1 the
    // items store fp32 partial sums [splits, M, N] and a second kernel adds them up
    int splits, kper;
    float* partial;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns = 20000u) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}
// Bounded wait: false when the phase did not complete in time or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag != 0 || clock64() - t0 > kWaitCycles) return false;
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
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
__device__ __forceinline__ uint32_t h2mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
constexpr uint32_t kMagic = 0x64006400u;

// Dequantise 16 consecutive codes of one row into eight half2 registers (codes 2j, 2j+1 in t[j]).  `w` holds the
// codes as a bit stream that starts at bit 0 of w[0].  Both fields of a pair are masked in place from a copy of
// their byte(s): (field | 0x6400) reads as 1024 + code * 2^p, one fused multiply-add with 2^-p and
// -(1024 * 2^-p + zero) leaves code - zero exactly, one multiply applies the scale (a single rounding of the
// exact product, i.e. the fp16 rounding of the fp32 value the reference rounds).
template <int BITS> struct Dequant16;

template <> struct Dequant16<4> {
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t zz, uint32_t ss, uint32_t (&t)[8]) {
        const uint32_t add = h2sub(0xD400E400u, zz);                 // (-1024 - z, -64 - z)
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = __byte_perm(w[j >> 2], 0u, (j & 3) | ((j & 3) << 8));   // byte -> bytes 0 and 2
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = lop3_and_or(t[j], 0x00F0000Fu, kMagic);
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = h2fma(t[j], 0x2C003C00u, add);                          // * (1, 1/16)
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = h2mul(t[j], ss);
    }
};

template <> struct Dequant16<2> {
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t zz, uint32_t ss, uint32_t (&t)[8]) {
        const uint32_t add01 = h2sub(0xDC00E400u, zz);               // (-1024 - z, -256 - z)   fields at bits 0, 2
        const uint32_t add23 = h2sub(0xCC00D400u, zz);               // (-64 - z,  -16 - z)     fields at bits 4, 6
        uint32_t b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = __byte_perm(w[0], 0u, j | (j << 8));                    // byte j = codes 4j..4j+3
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            t[2 * j] = lop3_and_or(b[j], 0x000C0003u, kMagic);
            t[2 * j + 1] = lop3_and_or(b[j], 0x00C00030u, kMagic);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            t[2 * j] = h2fma(t[2 * j], 0x34003C00u, add01);                                          // * (1, 1/4)
            t[2 * j + 1] = h2fma(t[2 * j + 1], 0x24002C00u, add23);                                  // * (1/16, 1/64)
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = h2mul(t[j], ss);
    }
};

template <> struct Dequant16<3> {
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t zz, uint32_t ss, uint32_t (&t)[8]) {
        const uint32_t add = h2sub(0xE400E400u, zz);                 // (-1024 - z) twice
#pragma unroll
        for (int j = 0; j < 8; ++j) {                                // codes 2j, 2j+1 at stream bit 6j (48 bits in all)
            const int pos = 6 * j, wi = pos >> 5, off = pos & 31;
            if (off + 6 <= 32) t[j] = w[wi] >> off;
            else t[j] = __funnelshift_r(w[0], w[1], off);            // the pair that straddles the two words
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = (t[j] & 0x3Fu) * 0x2001u;   // low code stays at bit 0, high code moves to bit 16
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = lop3_and_or(t[j], 0x00070007u, kMagic);
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = h2fma(t[j], 0x3C003C00u, add);
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = h2mul(t[j], ss);
    }
};

// ---- the same for bfloat16 activations: the expanded weight is round_bf16((q - zero) * scale) -------------------------
// bf16 has seven mantissa bits, so a field is only exact at bits 0..6 of its half: (field | 0x4300) reads as
// 128 + code * 2^p for p <= 4.  A multiply by 2^a + 1 first copies the byte's upper codes into the upper half.
__device__ __forceinline__ uint32_t b2fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t b2mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t b2sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
constexpr uint32_t kMagicB = 0x43004300u;      // bf16x2(128, 128)
constexpr uint32_t kOneB = 0x3F803F80u;        // bf16x2(1, 1)

template <int BITS> struct Dequant16B;

template <> struct Dequant16B<4> {
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t zz, uint32_t ss, uint32_t (&t)[8]) {
        const uint32_t add = b2sub(0xC300C300u, zz);                 // -(128 + z), exact: 128 + 15 needs eight bits
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = __byte_perm(w[j >> 2], 0u, 0x4440 | (j & 3)) * 0x1001u;   // byte j: its low code at bits 0-3 of the low half, its high code at bits 0-3 of the high half
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = lop3_and_or(t[j], 0x000F000Fu, kMagicB);
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = b2fma(t[j], kOneB, add);
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = b2mul(t[j], ss);
    }
};

template <> struct Dequant16B<2> {
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t zz, uint32_t ss, uint32_t (&t)[8]) {
        const uint32_t add0 = b2sub(0xC300C300u, zz);                // -(128 + z)    fields at bit 0
        const uint32_t add4 = b2sub(0xC100C100u, zz);                // -(8 + z)      fields at bit 4, scaled by 1/16
        uint32_t b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = __byte_perm(w[0], 0u, 0x4440 | j) * 0x4001u;   // low half: code 4j at bits 0-1, 4j+2 at bits 4-5; high half: 4j+1 at bits 0-1, 4j+3 at bits 4-5
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            t[2 * j] = lop3_and_or(b[j], 0x00030003u, kMagicB);      // codes 4j, 4j+1
            t[2 * j + 1] = lop3_and_or(b[j], 0x00300030u, kMagicB);  // codes 4j+2, 4j+3 (as 128 + 16 * code)
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            t[2 * j] = b2fma(t[2 * j], kOneB, add0);
            t[2 * j + 1] = b2fma(t[2 * j + 1], 0x3D803D80u, add4);   // * 1/16
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = b2mul(t[j], ss);
    }
};

template <> struct Dequant16B<3> {
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t zz, uint32_t ss, uint32_t (&t)[8]) {
        const uint32_t add = b2sub(0xC300C300u, zz);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int pos = 6 * j, wi = pos >> 5, off = pos & 31;
            if (off + 6 <= 32) t[j] = w[wi] >> off;
            else t[j] = __funnelshift_r(w[0], w[1], off);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = (t[j] & 0x3Fu) * 0x2001u;
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = lop3_and_or(t[j], 0x00070007u, kMagicB);
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = b2fma(t[j], kOneB, add);
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = b2mul(t[j], ss);
    }
};

// GU: fused gate/up.  The 128 TMEM lanes of a tile are 64 gate rows and the 64 up rows of the same indices,
// interleaved (lane 2i = gate row n0 + i, lane 2i + 1 = up row n0 + i), so that silu(gate) * up is a product of
// neighbouring lanes in the epilogue (the virtual-row trick of the decode kernel,
// Crispybits/Kernel/csrc/packed_gemv.cu:33-42, 61-64); a tile then covers 64 output columns.
// MODE 2: fused Q/K/V.  Tiles run over the rows of Q, then K, then V (each projection a whole number of tiles);
// the epilogue adds the bias, rotates Q and K (RoPE with the partner row in the neighbouring lane -- the rows are
// stored pair-interleaved, Crispybits/Kernel/csrc/common.cuh:61-70) and writes at the un-permuted column of the
// projection's own output.
template <int BITS, bool BF, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_ws_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
               const __grid_constant__ CUtensorMap wmap2, const __grid_constant__ CUtensorMap wmap3, const GemmParams P, const QkvParams Q) {
    constexpr bool GU = MODE == 1, QKV = MODE == 2;
    // fused Q/K/V: projection and first row (inside the projection) of weight tile tn
    auto tile_proj = [&](int tn, int& proj, int& n0) {
        const int tq = Q.n1 / kBN, tk = Q.n2 / kBN;
        if (tn < tq) { proj = 0; n0 = tn * kBN; }
        else if (tn < tq + tk) { proj = 1; n0 = (tn - tq) * kBN; }
        else { proj = 2; n0 = (tn - tq - tk) * kBN; }
    };
    constexpr int kOutCols = GU ? kBN / 2 : kBN;        // output columns (weight rows of one projection) per tile
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                    // swizzled tiles want 1024-byte alignment
    unsigned char* smem = smem_raw + (base - raw);
    constexpr uint32_t kPackedOff = kStages * kXBytes;
    constexpr uint32_t kBarOff = kPackedOff + kPackedSlots * kPackedSlotBytes;
    constexpr int kWords = 2 * BITS;                                 // packed words of one row and stage (64 codes)
    constexpr uint32_t kRowBytes = 2 * kWords * 4;                   // one row of a packed super-block (128 codes)
    const uint32_t s_bar = base + kBarOff;
    // barriers: full_x[s], full_w[s], empty[s], tmem_full, tmem_empty, full_p[slot], empty_p[slot]
    auto full_x = [&](int s) { return s_bar + 8u * s; };
    auto full_w = [&](int s) { return s_bar + 8u * (kStages + s); };
    auto empty = [&](int s) { return s_bar + 8u * (2 * kStages + s); };
    const uint32_t tmem_full = s_bar + 8u * (3 * kStages), tmem_empty = s_bar + 8u * (3 * kStages + 1);
    auto full_p = [&](int s) { return s_bar + 8u * (3 * kStages + 2 + s); };
    auto empty_p = [&](int s) { return s_bar + 8u * (3 * kStages + 2 + kPackedSlots + s); };
    const uint32_t final_full = s_bar + 8u * (3 * kStages + 2 + 2 * kPackedSlots);   // the CTA's last accumulator is complete
    constexpr uint32_t kNumBars = 3 * kStages + 3 + 2 * kPackedSlots;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kBarOff + 8 * kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kBarOff + 8 * kNumBars + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_x(s), 1);
            mbar_init(full_w(s), 4);                 // the four warps (lane quadrants) of one dequantiser group
            mbar_init(empty(s), 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, kEpiWarps);
        mbar_init(final_full, 1);
        for (int s = 0; s < kPackedSlots; ++s) { mbar_init(full_p(s), 1); mbar_init(empty_p(s), kDequantWarps); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // all 512 TMEM columns: the accumulator and the weight stages
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32((const void*)tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int nitems = P.tiles_m * P.tiles_n * P.splits;            // work item = (tile, K range): item / splits, item % splits
    int gave_up = 0;

    // Accumulator chunks (32 token columns each) cbegin, cbegin + cstep, ... of `tile` -> bias, activation, fp16, global.
    // Lane = weight row of this warp's TMEM lane quadrant, so the 32 lanes of a store are 64 contiguous bytes of
    // one token's output row.
    // release_bar != 0: arrive on that barrier as soon as this warp's last chunk is in registers -- the accumulator may
    // then be overwritten; the conversion and the stores of that chunk follow the arrival.
    auto drain = [&](int item, int cbegin, int cstep, uint32_t release_bar) {
        const int tile = item / P.splits, split = item - tile * P.splits;
        const int q = warp & 3;
        const int m0 = (tile % P.tiles_m) * kBT;
        const int row = q * 32 + lane;                              // TMEM lane
        int n = (tile / P.tiles_m) * kOutCols + (GU ? (row >> 1) : row);
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
        bool nlive = n < P.N;
        auto load_bias = [&](const __half* b, int r) {
            return b == nullptr ? 0.f
                   : BF ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(b)[r]) : __half2float(b[r]);
        };
        float bias = 0.f;
        __half* obase = P.out;
        int ld = P.N;                                               // row stride of the output
        // fused Q/K/V: the projection's output, the un-permuted column, the partner's bias and the RoPE column
        float bias_partner = 0.f;
        int rope_d = -1;
        // Two lanes that hold neighbouring output columns pair up for the stores (below): lanes one apart, or two apart
        // where the rows are stored pair-interleaved (then rows r and r + 2 of equal parity are columns c and c + 1).
        int pair_dist = 1;
        bool pair_ok = true;
        if constexpr (QKV) {
            int proj, pn0;
            tile_proj(tile / P.tiles_m, proj, pn0);
            const int r = pn0 + row;
            const __half* b = proj == 0 ? P.bias : proj == 1 ? Q.bias2 : Q.bias3;
            obase = proj == 0 ? P.out : proj == 1 ? Q.out2 : Q.out3;
            ld = proj == 0 ? Q.n1 : proj == 1 ? Q.n2 : Q.n3;
            bias = load_bias(b, r);
            n = unpermute_row(r, proj < 2 ? Q.perm_hd : 0);
            nlive = true;
            if (proj < 2 && Q.perm_hd > 0) { pair_dist = 2; pair_ok = Q.perm_hd % 4 == 0; }
            if (Q.rope_cos != nullptr && proj < 2) {
                bias_partner = load_bias(b, r ^ 1);
                rope_d = n % Q.head_dim;
            }
        } else if (!GU && nlive) {
            bias = load_bias(P.bias, n);
        }
        pair_ok = pair_ok && (reinterpret_cast<uintptr_t>(obase) & 3) == 0 && (ld & 1) == 0;
#pragma unroll 1
        for (int c0 = 32 * cbegin; c0 < kBT; c0 += 32 * cstep) {
            uint32_t v[32];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                         "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                         "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                           "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                           "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                           "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                         : "r"(taddr + (uint32_t)c0));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (release_bar != 0u && c0 + 32 * cstep >= kBT) {
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(release_bar);
            }
            if constexpr (MODE == 0) {
                if (P.splits > 1) {      // partial sums of this K range: fp32, [split][token][weight row]
                    if (nlive) {
                        float* pcol = P.partial + ((size_t)split * P.M + m0 + c0) * P.N + n;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (m0 + c0 + j < P.M) pcol[(size_t)j * P.N] = __uint_as_float(v[j]);
                    }
                    continue;
                }
            }
            if constexpr (GU) {
                // silu(gate) * up: the gate lane and the up lane of an output column share the work -- the gate lane
                // finishes the even tokens of the chunk, the up lane the odd ones (one exchange per token pair);
                // the result for token j + (lane & 1) is left in v[j], j even
                const bool odd = (lane & 1) != 0;
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const float mine_even = __uint_as_float(v[j]), mine_odd = __uint_as_float(v[j + 1]);
                    const float other = __shfl_xor_sync(0xffffffffu, odd ? mine_even : mine_odd, 1);
                    const float gate = odd ? other : mine_even, up = odd ? mine_odd : other;
                    v[j] = __float_as_uint(activate(gate, CB_ACT_SILU) * up);
                }
            }
            if constexpr (QKV) {
                if (__any_sync(0xffffffffu, rope_d >= 0)) {          // uniform over the warp: one projection per tile
                    const bool first_half = rope_d < Q.head_dim / 2;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {                   // the rotation partner sits in the next lane
                        const float y = __uint_as_float(v[j]) + bias;
                        const float yp = __shfl_xor_sync(0xffffffffu, __uint_as_float(v[j]), 1) + bias_partner;
                        const int m = min(m0 + c0 + j, P.M - 1);
                        const float c = Q.rope_cos[(size_t)m * Q.head_dim + rope_d];
                        const float sn = Q.rope_sin[(size_t)m * Q.head_dim + rope_d];
                        v[j] = __float_as_uint(first_half ? (y * c - yp * sn) : (y * c + yp * sn));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + bias);
                }
            }
            int pair_hi = 0;
            if constexpr (!GU) {
                if constexpr (!QKV) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(activate(__uint_as_float(v[j]) + bias, P.act));
                }
                if (pair_ok) {
                    // the lower lane of a pair keeps the even tokens, the upper lane the odd ones; v[j] (j even) becomes
                    // the two 16-bit results of columns (c, c + 1) for token j + pair_hi
                    pair_hi = (lane & pair_dist) != 0 ? 1 : 0;
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float a = __uint_as_float(v[j]), b = __uint_as_float(v[j + 1]);
                        const float other = __shfl_xor_sync(0xffffffffu, pair_hi ? a : b, pair_dist);
                        const float lo_val = pair_hi ? other : a, hi_val = pair_hi ? b : other;
                        if constexpr (BF) {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(lo_val, hi_val);
                            v[j] = *reinterpret_cast<const uint32_t*>(&h);
                        } else {
                            const __half2 h = __floats2half2_rn(lo_val, hi_val);
                            v[j] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                    }
                }
            }
            if (nlive) {
                __half* ocol = obase + (size_t)(m0 + c0) * ld + n;
                if constexpr (GU) {
                    const int odd = lane & 1;
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        if (m0 + c0 + j + odd < P.M) {
                            const float y = __uint_as_float(v[j]);
                            if constexpr (BF) reinterpret_cast<__nv_bfloat16*>(ocol)[(size_t)(j + odd) * ld] = __float2bfloat16_rn(y);
                            else ocol[(size_t)(j + odd) * ld] = __float2half_rn(y);
                        }
                    }
                } else if (pair_ok) {
                    // 4-byte stores: this lane writes columns (c, c + 1) of every other token of the chunk
                    uint32_t* o32 = reinterpret_cast<uint32_t*>(ocol - pair_hi);
#pragma unroll
                    for (int j = 0; j < 32; j += 2)
                        if (m0 + c0 + j + pair_hi < P.M) o32[((size_t)(j + pair_hi) * ld) >> 1] = v[j];
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (m0 + c0 + j < P.M) {
                            const float y = __uint_as_float(v[j]);
                            if constexpr (BF) reinterpret_cast<__nv_bfloat16*>(ocol)[(size_t)j * ld] = __float2bfloat16_rn(y);
                            else ocol[(size_t)j * ld] = __float2half_rn(y);
                        }
                    }
                }
            }
        }
    };

    if (warp == 0) {
        // ================= TMA producer: activation tiles, 256 tokens x 64 codes =================
        if (lane == 0) {
            int it = 0;
            for (int item = blockIdx.x; item < nitems && !gave_up; item += gridDim.x) {
                const int tile = item / P.splits, kb0 = (item - tile * P.splits) * P.kper;
                const int m0 = (tile % P.tiles_m) * kBT;
                for (int kb = kb0; kb < kb0 + P.kper; ++kb, ++it) {
                    const int s = it % kStages;
                    if (it >= kStages && !mbar_wait(empty(s), ((it / kStages) - 1) & 1, abort_flag)) { gave_up = 1; break; }
                    mbar_expect_tx(full_x(s), kXBytes);
                    tma_load_2d(base + s * kXBytes, &xmap, kb * kBK, m0, full_x(s));
                }
            }
        }
    } else if (warp == kPackedWarp) {
        // ================= TMA producer: packed words, 128 rows x 128 codes per box =================
        if (lane == 0) {
            int pit = 0;
            for (int item = blockIdx.x; item < nitems && !gave_up; item += gridDim.x) {
                const int tile = item / P.splits, kb0 = (item - tile * P.splits) * P.kper;
                int n0 = (tile / P.tiles_m) * kOutCols;
                const CUtensorMap* map = &wmap;
                if constexpr (QKV) {      // the tile's projection has its own packed tensor
                    int proj;
                    tile_proj(tile / P.tiles_m, proj, n0);
                    map = proj == 0 ? &wmap : proj == 1 ? &wmap2 : &wmap3;
                }
                for (int sb = kb0 >> 1; sb < ((kb0 + P.kper) >> 1); ++sb, ++pit) {      // kper is even
                    const int slot = pit % kPackedSlots;
                    if (pit >= kPackedSlots && !mbar_wait(empty_p(slot), ((pit / kPackedSlots) - 1) & 1, abort_flag)) { gave_up = 5; break; }
                    mbar_expect_tx(full_p(slot), kBN * kRowBytes);
                    const uint32_t dst = base + kPackedOff + slot * kPackedSlotBytes;
                    tma_load_2d(dst, map, sb * 2 * kWords, n0, full_p(slot));
                    if constexpr (GU)     // the up projection's 64 rows behind the gate's 64 rows
                        tma_load_2d(dst + (uint32_t)kOutCols * kRowBytes, &wmap2, sb * 2 * kWords, n0, full_p(slot));
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer: A (weights) from tensor memory, B (activations) from shared memory =================
        if (lane == 0) {
            int it = 0, tcount = 0;
            for (int item = blockIdx.x; item < nitems && !gave_up; item += gridDim.x, ++tcount) {
                // the one accumulator must have been drained by the epilogue of the previous item
                if (tcount >= 1 && !mbar_wait(tmem_empty, (tcount - 1) & 1, abort_flag)) { gave_up = 2; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < P.kper; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!mbar_wait(full_x(s), ph, abort_flag) || !mbar_wait(full_w(s), ph, abort_flag)) { gave_up = 2; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t xa = base + s * kXBytes;
                    const uint32_t a_tmem = tmem_base + kAccCols + (uint32_t)s * kAStageCols;
                    // B descriptor: K-major, 128-byte swizzle, 8-row atoms 1024 bytes apart
                    const uint64_t dhi = (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        const uint64_t bdesc = dhi | (uint64_t)(((xa + k * 32) >> 4) & 0x3FFF);
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                     " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}"
                                     ::"r"(tmem_base), "r"(a_tmem + (uint32_t)k * 8u), "l"(bdesc), "r"(BF ? kIdescBF16 : kIdescF16), "r"(accumulate), "r"(0u) : "memory");
                    }
                    // the stage (shared-memory x tile and TMEM weight columns) may be refilled once these MMAs have read it
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(empty(s)) : "memory");
                }
                if (gave_up) break;
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tmem_full) : "memory");
                if (item + (int)gridDim.x >= nitems)     // also wakes the dequantiser warps, which help drain the last item
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(final_full) : "memory");
            }
        }
    } else if (warp < kFirstEpiWarp) {
        // ================= dequantisers: four groups of four warps; group g expands stages g, g+4, g+8, ... =================
        // A stage's hand-off chain (packed words landed -> expand -> TMEM store -> signal) is several hundred cycles
        // long; with every group on its own stage four such chains overlap, and a group has four stage times to
        // finish one.  Within a group, warp = TMEM lane quadrant, lane = weight row: a thread expands all 64 codes
        // of its row and stage and writes them to its TMEM lane with one 32-column store.
        const int q = warp & 3;                                           // the TMEM lane quadrant this warp may access
        const int grp = (warp - kFirstDequantWarp) >> 2;                  // 0..3
        const int r = q * 32 + lane;                                      // weight row of the tile = TMEM lane
        const int my_tiles = blockIdx.x < nitems ? (nitems - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;   // work items of this CTA
        const int total = my_tiles * P.kper;                              // stages this CTA runs through
        const unsigned short* srow = nullptr;
        const unsigned short* zrow = nullptr;
        int cur_tile_local = -1;
        bool live = false;
        auto meta_of = [&](int it) -> uint32_t {                          // (zero << 16) | scale of (row, stage it), raw fp16 bits
            if (it >= total) return 0u;
            const int tl = it / P.kper;
            const int item = blockIdx.x + tl * gridDim.x;
            const int tile = item / P.splits;
            const int kb = (item - tile * P.splits) * P.kper + (it - tl * P.kper);
            if (tl != cur_tile_local) {
                cur_tile_local = tl;
                int n = (tile / P.tiles_m) * kOutCols + (GU ? (r >> 1) : r);
                live = n < P.N;
                int proj = (GU && (r & 1)) ? 1 : 0;                      // odd lanes of a fused gate/up tile belong to the up projection
                if constexpr (QKV) {
                    int pn0;
                    tile_proj(tile / P.tiles_m, proj, pn0);
                    n = pn0 + r;
                    live = true;
                }
                const __half* sc = proj == 0 ? P.scales : proj == 1 ? P.scales2 : Q.scales3;
                const __half* zr = proj == 0 ? P.zeros : proj == 1 ? P.zeros2 : Q.zeros3;
                srow = reinterpret_cast<const unsigned short*>(sc) + (size_t)(live ? n : 0) * P.groups;
                zrow = reinterpret_cast<const unsigned short*>(zr) + (size_t)(live ? n : 0) * P.groups;
            }
            if (!live) return 0u;                                         // rows past N were zero-filled by the copy and get scale 0
            const int g = (kb * kBK) / P.group_size;
            return (uint32_t)__ldg(srow + g) | ((uint32_t)__ldg(zrow + g) << 16);
        };
        // Every group passes every packed super-block in order (wait for it, read its own stage's words if it has
        // one there, release it): each mbarrier phase is then observed exactly once by each waiter, which is what
        // the parity protocol needs.  Stage index = 2 * super-block + half; group = stage index mod 4.
        const int total_super = total >> 1;                               // kblocks is even
        uint32_t meta_next = meta_of(grp);
        for (int pit = 0; pit < total_super && !gave_up; ++pit) {
            const int slot = pit % kPackedSlots;
            if (!__all_sync(0xffffffffu, mbar_wait(full_p(slot), (pit / kPackedSlots) & 1, abort_flag))) { gave_up = 3; break; }
            const int half = ((2 * pit) & 3) == grp ? 0 : (((2 * pit + 1) & 3) == grp ? 1 : -1);
            uint32_t w[kWords];
            if (half >= 0) {
                const unsigned char* stage_words = smem + kPackedOff + slot * kPackedSlotBytes + (uint32_t)(GU ? ((r & 1) * kOutCols + (r >> 1)) : r) * kRowBytes + half * (kWords * 4);
                if constexpr (BITS == 4) {
                    const uint4 a = reinterpret_cast<const uint4*>(stage_words)[0], b4 = reinterpret_cast<const uint4*>(stage_words)[1];
                    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b4.x; w[5] = b4.y; w[6] = b4.z; w[7] = b4.w;
                } else if constexpr (BITS == 2) {
                    const uint4 a = reinterpret_cast<const uint4*>(stage_words)[0];
                    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
                } else {
                    const uint2 a = reinterpret_cast<const uint2*>(stage_words)[0], b2 = reinterpret_cast<const uint2*>(stage_words)[1],
                                c2 = reinterpret_cast<const uint2*>(stage_words)[2];
                    w[0] = a.x; w[1] = a.y; w[2] = b2.x; w[3] = b2.y; w[4] = c2.x; w[5] = c2.y;
                }
            }
            // A warp that has no stage in this super-block hands the slot back at once; a warp that has one hands it
            // back only after its stage is in tensor memory (below).  Handing it back right after the loads were
            // issued was measured to be unsafe: in a few percent of runs (in all runs once the dequantisers were
            // slowed down artificially) rows were expanded from a mixture of this super-block and the one that the
            // next TMA box brought into the slot.
            __syncwarp();
            if (half < 0) {
                if (lane == 0) mbar_arrive(empty_p(slot));
                continue;
            }
            const int it = 2 * pit + half;
            const int s = it % kStages;
            const uint32_t meta = meta_next;
            meta_next = meta_of(it + 4);                                  // requested one of this group's stages ahead
            const uint32_t ss = (meta & 0xFFFFu) * 0x10001u, zz = (meta >> 16) * 0x10001u;
            uint32_t t[32];
#pragma unroll
            for (int kq = 0; kq < 4; ++kq) {                              // 16 codes at a time
                uint32_t w2[2];
                if constexpr (BITS == 4) { w2[0] = w[2 * kq]; w2[1] = w[2 * kq + 1]; }
                else if constexpr (BITS == 2) { w2[0] = w[kq]; w2[1] = 0u; }
                else {
                    // 48 bits from stream bit 48 * kq: two words, shifted down by 16 for odd quarters
                    const uint32_t lo = w[(3 * kq) >> 1], hi = w[((3 * kq) >> 1) + 1];
                    w2[0] = (kq & 1) ? __funnelshift_r(lo, hi, 16) : lo;
                    w2[1] = (kq & 1) ? (hi >> 16) : hi;
                }
                uint32_t t8[8];
                if constexpr (BF) Dequant16B<BITS>::run(w2, zz, ss, t8);
                else Dequant16<BITS>::run(w2, zz, ss, t8);
#pragma unroll
                for (int j = 0; j < 8; ++j) t[8 * kq + j] = t8[j];
            }
            if (it >= kStages && !__all_sync(0xffffffffu, mbar_wait(empty(s), ((it / kStages) - 1) & 1, abort_flag))) { gave_up = 3; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // lane r, the 32 columns of A stage s: codes 2c, 2c+1 of this stage in column c
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + kAccCols + (uint32_t)s * kAStageCols;
            asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                         "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                         "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                         ::"r"(taddr), "r"(t[0]), "r"(t[1]), "r"(t[2]), "r"(t[3]), "r"(t[4]), "r"(t[5]), "r"(t[6]), "r"(t[7]),
                           "r"(t[8]), "r"(t[9]), "r"(t[10]), "r"(t[11]), "r"(t[12]), "r"(t[13]), "r"(t[14]), "r"(t[15]),
                           "r"(t[16]), "r"(t[17]), "r"(t[18]), "r"(t[19]), "r"(t[20]), "r"(t[21]), "r"(t[22]), "r"(t[23]),
                           "r"(t[24]), "r"(t[25]), "r"(t[26]), "r"(t[27]), "r"(t[28]), "r"(t[29]), "r"(t[30]), "r"(t[31]) : "memory");
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) { mbar_arrive(full_w(s)); mbar_arrive(empty_p(slot)); }
        }
        // All stages are expanded: help the epilogue warps drain the CTA's last accumulator (further workers
        // of each lane quadrant).  A barrier of its own, completed once, tells these warps that it is ready.
        if (my_tiles > 0 && !gave_up) {
            if (!__all_sync(0xffffffffu, mbar_wait(final_full, 0, abort_flag))) gave_up = 3;
            else {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                drain((int)blockIdx.x + (my_tiles - 1) * (int)gridDim.x, grp + kEpiWarps / 4, 4 + kEpiWarps / 4, 0u);
            }
        }
    } else if (warp < kPackedWarp) {
        // ================= epilogue warps: drain every accumulator; on the CTA's last tile the dequantisers help =================
        int tcount = 0;
        for (int tile = blockIdx.x; tile < nitems && !gave_up; tile += gridDim.x, ++tcount) {      // `tile` counts work items here
            if (!__all_sync(0xffffffffu, mbar_wait(tmem_full, tcount & 1, abort_flag))) { gave_up = 4; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool last = tile + (int)gridDim.x >= nitems;
            const int worker = (warp - kFirstEpiWarp) >> 2;             // this warp's place among its quadrant's epilogue warps
            // Plain and gate/up: the arrival that frees the accumulator comes before the last chunk's stores (measured
            // 3-4 % faster); with the Q/K/V epilogue the same order was measured 15 % slower, so there it follows the drain.
            const uint32_t early = QKV ? 0u : tmem_empty;
            if (last) drain(tile, worker, 4 + kEpiWarps / 4, early);        // the four dequantiser groups are further workers
            else drain(tile, worker, kEpiWarps / 4, early);
            if constexpr (QKV) {
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_empty);
            }
        }
    }

    if (gave_up) {
        *abort_flag = 1;
        atomicExch(&g_gemm_ws_status, gave_up);
    }
    // everyone is done with TMEM before it is released
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// out[m, n] = act(sum over the K ranges of partial[s, m, n] + bias[n]) for a K-split launch: four columns per thread.
template <bool BF>
__global__ void gemm_ws_reduce_kernel(const float* __restrict__ partial, const __half* __restrict__ bias, __half* __restrict__ out,
                                      int M, int N, int splits, int act) {
    const size_t quads = (size_t)M * N / 4;
    for (size_t q = blockIdx.x * (size_t)blockDim.x + threadIdx.x; q < quads; q += (size_t)gridDim.x * blockDim.x) {
        float4 acc = reinterpret_cast<const float4*>(partial)[q];
        for (int s = 1; s < splits; ++s) {
            const float4 v = reinterpret_cast<const float4*>(partial + (size_t)s * M * N)[q];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const int n = (int)((q * 4) % N);
        float y[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (bias != nullptr)
                y[i] += BF ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[n + i]) : __half2float(bias[n + i]);
            y[i] = activate(y[i], act);
        }
        if constexpr (BF) {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + q * 4;
            reinterpret_cast<__nv_bfloat162*>(o)[0] = __floats2bfloat162_rn(y[0], y[1]);
            reinterpret_cast<__nv_bfloat162*>(o)[1] = __floats2bfloat162_rn(y[2], y[3]);
        } else {
            __half* o = out + q * 4;
            reinterpret_cast<__half2*>(o)[0] = __floats2half2_rn(y[0], y[1]);
            reinterpret_cast<__half2*>(o)[1] = __floats2half2_rn(y[2], y[3]);
        }
    }
}

template <int BITS, bool BF, int MODE>
int launch_t(const CUtensorMap& xmap, const CUtensorMap& wmap, const CUtensorMap& wmap2, const CUtensorMap& wmap3,
             const GemmParams& P, const QkvParams& Q, int grid, cudaStream_t stream) {
    static bool attr_done[64] = {};
    int dev = 0;
    CB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        CB_CUDA_TRY(cudaFuncSetAttribute(gemm_ws_kernel<BITS, BF, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    gemm_ws_kernel<BITS, BF, MODE><<<grid, kThreads, kSmemBytes, stream>>>(xmap, wmap, wmap2, wmap3, P, Q);
    CB_CUDA_TRY(cudaGetLastError());
    return CB_OK;
}

}  // namespace

namespace {

// w2 == nullptr: out = act(x W^T + bias).  w2 != nullptr: out = silu(x W^T) * (x W2^T), W and W2 of equal shape.
// qkv != nullptr: w, qkv->k, qkv->v are the Q, K, V projections; out is Q's output.
struct WsQkv {
    const cb_weight* k; const cb_weight* v;
    void* out_k; void* out_v;
    const float* rope_cos; const float* rope_sin;
    int head_dim, perm_hd;
};

// How many K ranges a plain launch of this shape is split into when `scratch_bytes` of scratch are available: only where
// the tiles alone would leave more than half of the SMs idle, at least eight stages per range, ranges of equal size.
int ws_splits(int64_t M, int64_t N, int64_t K, int sms, size_t scratch_bytes) {
    const int64_t tiles = ((M + kBT - 1) / kBT) * ((N + kBN - 1) / kBN);
    const int supers = (int)(K / (2 * kBK));
    if (tiles * 2 > sms || N % 4 != 0 || K % 128 != 0) return 1;
    int best = 1;
    for (int sp = 2; sp <= 8 && tiles * sp <= sms && supers / sp >= 4; ++sp)
        if (supers % sp == 0 && (size_t)sp * M * N * sizeof(float) <= scratch_bytes) best = sp;
    return best;
}

int launch_ws(int dtype, const void* x, int64_t M, const cb_weight* w, const cb_weight* w2, void* out, int64_t K, int bits,
              int64_t gs, int act, cudaStream_t stream, const WsQkv* qkv = nullptr, void* scratch = nullptr,
              size_t scratch_bytes = 0) {
    const bool gu = w2 != nullptr && qkv == nullptr;
    if ((dtype != CB_F16 && dtype != CB_BF16) || K % 128 != 0 || gs % kBK != 0 || M < 1) return -1;
    if (!gu && w->n % 8 != 0) return -1;
    if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(w->packed) % 16 ||
        (gu && reinterpret_cast<uintptr_t>(w2->packed) % 16) || reinterpret_cast<uintptr_t>(out) % 2)
        return -1;
    if (qkv != nullptr) {     // every projection a whole number of tiles, so that a tile has one projection
        if (w->n % kBN != 0 || qkv->k->n % kBN != 0 || qkv->v->n % kBN != 0) return -1;
        if (reinterpret_cast<uintptr_t>(qkv->k->packed) % 16 || reinterpret_cast<uintptr_t>(qkv->v->packed) % 16) return -1;
    }
    if (M >= (1ll << 31) / 2 || K >= (1ll << 30)) return -1;
    EncodeTiledFn enc = encode_fn();
    if (enc == nullptr) return -1;
    const int sms = sm_count_current();
    if (sms <= 0) return CB_ERR_CUDA;
    const int out_cols = gu ? kBN / 2 : kBN;                 // weight rows of one projection per tile

    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap xmap, wmap, wmap2, wmap3;
    {   // activations: [M, K] 16-bit, box 64 x 256, 128-byte swizzle (the UMMA K-major layout)
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBT};
        const CUresult cr = enc(&xmap, dtype == CB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                                const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) { set_error("packed_gemm: cuTensorMapEncodeTiled(x) failed (%d)", (int)cr); return CB_ERR_CUDA; }
    }
    auto encode_packed = [&](CUtensorMap* map, const cb_weight* pw) -> int {
        // packed words: [N, K/32*bits] uint32, box (128 codes) x (rows of one projection per tile), no swizzle
        const cuuint64_t wpr = (cuuint64_t)(K / 32) * bits;
        const cuuint64_t dims[2] = {wpr, (cuuint64_t)pw->n};
        const cuuint64_t strides[1] = {wpr * 4};
        const cuuint32_t box[2] = {(cuuint32_t)(4 * bits), (cuuint32_t)out_cols};
        const CUresult cr = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<int32_t*>(pw->packed), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) { set_error("packed_gemm: cuTensorMapEncodeTiled(packed) failed (%d)", (int)cr); return CB_ERR_CUDA; }
        return CB_OK;
    };
    int rc = encode_packed(&wmap, w);
    if (rc != CB_OK) return rc;
    // maps the mode does not use are copies of the first (the kernel takes three): no further encoding on the host
    if (gu || qkv != nullptr) {
        rc = encode_packed(&wmap2, gu ? w2 : qkv->k);
        if (rc != CB_OK) return rc;
    } else {
        wmap2 = wmap;
    }
    if (qkv != nullptr) {
        rc = encode_packed(&wmap3, qkv->v);
        if (rc != CB_OK) return rc;
    } else {
        wmap3 = wmap;
    }

    GemmParams P{};
    QkvParams Q{};
    P.scales = reinterpret_cast<const __half*>(w->scales);
    P.zeros = reinterpret_cast<const __half*>(w->zeros);
    P.scales2 = reinterpret_cast<const __half*>(gu ? w2->scales : w->scales);
    P.zeros2 = reinterpret_cast<const __half*>(gu ? w2->zeros : w->zeros);
    P.bias = gu ? nullptr : reinterpret_cast<const __half*>(w->bias);
    P.out = reinterpret_cast<__half*>(out);
    P.M = (int)M; P.N = (int)w->n; P.K = (int)K;
    P.groups = (int)((K + gs - 1) / gs); P.group_size = (int)gs; P.act = act;
    P.tiles_m = (int)((M + kBT - 1) / kBT); P.tiles_n = (int)((w->n + out_cols - 1) / out_cols); P.kblocks = (int)(K / kBK);
    if (qkv != nullptr) {
        P.bias = reinterpret_cast<const __half*>(w->bias);
        P.scales2 = reinterpret_cast<const __half*>(qkv->k->scales); P.zeros2 = reinterpret_cast<const __half*>(qkv->k->zeros);
        Q.scales3 = reinterpret_cast<const __half*>(qkv->v->scales); Q.zeros3 = reinterpret_cast<const __half*>(qkv->v->zeros);
        Q.bias2 = reinterpret_cast<const __half*>(qkv->k->bias); Q.bias3 = reinterpret_cast<const __half*>(qkv->v->bias);
        Q.out2 = reinterpret_cast<__half*>(qkv->out_k); Q.out3 = reinterpret_cast<__half*>(qkv->out_v);
        Q.n1 = (int)w->n; Q.n2 = (int)qkv->k->n; Q.n3 = (int)qkv->v->n;
        P.N = Q.n1 + Q.n2 + Q.n3;
        P.tiles_n = P.N / kBN;
        Q.rope_cos = qkv->rope_cos; Q.rope_sin = qkv->rope_sin;
        Q.head_dim = qkv->head_dim; Q.perm_hd = qkv->perm_hd;
        P.act = 0;
    }
    const bool bf = dtype == CB_BF16;
    const int mode = qkv != nullptr ? 2 : gu ? 1 : 0;
    P.splits = 1;
    if (mode == 0 && scratch != nullptr && reinterpret_cast<uintptr_t>(scratch) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0)
        P.splits = ws_splits(M, w->n, K, sms, scratch_bytes);
    P.kper = P.kblocks / P.splits;
    P.partial = P.splits > 1 ? reinterpret_cast<float*>(scratch) : nullptr;
    const int grid = std::min(sms, P.tiles_m * P.tiles_n * P.splits);
    int rc_launch;
#define CB_WS_LAUNCH_M(B, MD) \
    (bf ? launch_t<B, true, MD>(xmap, wmap, wmap2, wmap3, P, Q, grid, stream) : launch_t<B, false, MD>(xmap, wmap, wmap2, wmap3, P, Q, grid, stream))
#define CB_WS_LAUNCH(B) (mode == 2 ? CB_WS_LAUNCH_M(B, 2) : mode == 1 ? CB_WS_LAUNCH_M(B, 1) : CB_WS_LAUNCH_M(B, 0))
    switch (bits) {
        case 2: rc_launch = CB_WS_LAUNCH(2); break;
        case 3: rc_launch = CB_WS_LAUNCH(3); break;
        default: rc_launch = CB_WS_LAUNCH(4); break;
    }
#undef CB_WS_LAUNCH
#undef CB_WS_LAUNCH_M
    if (rc_launch != CB_OK || P.splits == 1) return rc_launch;
    const int rthreads = 256;
    const int rgrid = (int)std::min<size_t>(((size_t)M * w->n / 4 + rthreads - 1) / rthreads, (size_t)sms * 8);
    if (bf) gemm_ws_reduce_kernel<true><<<rgrid, rthreads, 0, stream>>>(P.partial, P.bias, P.out, P.M, P.N, P.splits, P.act);
    else gemm_ws_reduce_kernel<false><<<rgrid, rthreads, 0, stream>>>(P.partial, P.bias, P.out, P.M, P.N, P.splits, P.act);
    CB_CUDA_TRY(cudaGetLastError());
    return CB_OK;
}

}  // namespace

// CB_OK after launching; a CB_ERR_* code on a CUDA error; -1 when the problem is outside this kernel's
// domain (fp16 or bf16, K a multiple of 128, group size a multiple of 64, N a multiple of 8, 16-byte aligned
// x / packed) and the caller should use another kernel.
int launch_gemm_ws(int dtype, const void* x, int64_t M, const cb_weight* w, void* out, int64_t K, int bits,
                   int64_t gs, int act, cudaStream_t stream, void* scratch, size_t scratch_bytes) {
    return launch_ws(dtype, x, M, w, nullptr, out, K, bits, gs, act, stream, nullptr, scratch, scratch_bytes);
}

// Splits a plain launch of this shape would use with unlimited scratch (1 = no split), for sizing that scratch.
int gemm_ws_splits(int64_t M, int64_t N, int64_t K) {
    const int sms = sm_count_current();
    return sms <= 0 ? 1 : ws_splits(M, N, K, sms, ~(size_t)0);
}

// Fused prefill gate/up: out[M, n] = silu(x Wg^T) * (x Wu^T) in one launch; same return convention.
int launch_gemm_ws_gate_up(int dtype, const void* x, int64_t M, const cb_weight* gate, const cb_weight* up, void* out,
                           int64_t K, int bits, int64_t gs, cudaStream_t stream) {
    if (gate->n != up->n) return -1;
    return launch_ws(dtype, x, M, gate, up, out, K, bits, gs, 0, stream);
}

// Fused prefill Q/K/V (+ bias, + RoPE on Q and K, un-permuted stores) in one launch; same return convention.
// Needs every projection's row count to be a multiple of 128.
int launch_gemm_ws_qkv(int dtype, const void* x, int64_t M, const cb_weight* q, const cb_weight* k, const cb_weight* v,
                       void* out_q, void* out_k, void* out_v, const float* rope_cos, const float* rope_sin, int head_dim,
                       int perm_hd, int64_t K, int bits, int64_t gs, cudaStream_t stream) {
    const WsQkv spec{k, v, out_k, out_v, rope_cos, rope_sin, head_dim, perm_hd};
    return launch_ws(dtype, x, M, q, k, out_q, K, bits, gs, 0, stream, &spec);
}

int gemm_ws_status_read_and_clear(int* out) {
    int v = 0, zero = 0;
    CB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_gemm_ws_status, sizeof(int)));
    CB_CUDA_TRY(cudaMemcpyToSymbol(g_gemm_ws_status, &zero, sizeof(int)));
    *out = v;
    return CB_OK;
}

}  // namespace cb
