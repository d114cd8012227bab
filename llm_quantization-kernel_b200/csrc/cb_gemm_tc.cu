// Prefill GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) with in-kernel dequantisation.
//
//   out[M, N] = act( x[M, K] * Wdq[N, K]^T + bias ),   Wdq = round_fp16((q - zero) * scale)
//
// The weight numerics are those of the reference's tensor-core path (the dequantised weight is
// rounded to the storage type before the product, fp32 accumulation:
// Crispybits/Kernel/csrc/packed_gemm.cu:47-61): (q - zero) is an exact fp16 integer and one fp16
// multiply by the scale rounds the exact product once, which is the same value as rounding the fp32
// product.
//
// Shape of the kernel (one persistent CTA per SM, 23 warps, no cluster):
//   tile        128 tokens (UMMA M) x 256 weight rows (UMMA N) x 64 codes per pipeline stage;
//               tokens are the M side because the activation tile is what travels from L2 for every
//               tile, and 128 x 64 fp16 is half of what a 256-token tile would cost; the packed
//               weights are 4-8x smaller than fp16 and are expanded inside the SM.
//   warp 0      TMA producer of the x tile of each stage (2-D tensor map, 128-byte swizzle).
//   warp 1      allocates TMEM, and one lane issues tcgen05.mma (kind::f16, 128x256x16, four per stage)
//               with shared-memory descriptors; tcgen05.commit hands stages back and publishes finished
//               accumulators.
//   warps 2-17  dequantisers: half a weight row (32 codes) per thread and stage.  The row's packed words are read from
//               a shared-memory ring, expanded with the (w & mask) | 0x6400 trick, and stored as fp16 in
//               the K-major 128-byte-swizzled layout the MMA reads (16-byte chunk c of row r lands at
//               chunk c ^ (r & 7)).
//   warps 18-21 epilogue: tcgen05.ld of their 32 TMEM lanes (= 32 tokens), bias, activation, fp16, and
//               64-byte row segments to global memory.  Two 256-column accumulators alternate, so the
//               epilogue of one tile overlaps the main loop of the next.
//   warp 22     TMA producer of the packed words: one 2-D box of 256 rows x 128 codes per two stages
//               into a three-deep ring.  (Thread-per-row loads straight from global memory touch 32
//               different cache lines per warp instruction and were measured to bound the whole
//               pipeline; the bulk copy does the strided gather in the copy engine.)
// Every mbarrier wait is bounded; a wait that runs out raises a flag in shared memory and in the
// status word, every role leaves its loops, TMEM is released, and the kernel returns.
#include <algorithm>

#include <cuda.h>

#include "cb_common.cuh"

namespace cb {
namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 3;
constexpr int kPackedSlots = 3;                     // ring of packed super-blocks (128 codes = two stages each)
constexpr int kThreads = 23 * 32;
constexpr int kDequantWarps = 16, kFirstDequantWarp = 2, kFirstEpiWarp = 18, kPackedWarp = 22;
constexpr uint32_t kXBytes = kBM * kBK * 2, kWBytes = kBN * kBK * 2;
constexpr uint32_t kStageBytes = kXBytes + kWBytes;
constexpr uint32_t kPackedSlotBytes = kBN * 64;     // 256 rows x 128 codes at 4 bits; narrower rows use less of it
constexpr uint32_t kSmemBytes = kStages * kStageBytes + kPackedSlots * kPackedSlotBytes + 1024 /*align*/ + 256 /*barriers*/;
constexpr long long kWaitCycles = 2000000000ll;     // about a second at boost clock
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);   // f16 x f16 -> f32, K-major A and B

__device__ int g_gemm_status;   // 0 = ok, else the role that gave up waiting (1 x producer, 2 mma, 3 dequant, 4 epilogue, 5 packed producer)

struct GemmParams {
    const __half* scales; const __half* zeros; const __half* bias; __half* out;
    int M, N, K, groups, group_size, act;
    int tiles_m, tiles_n, kblocks;
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
// try_wait with a suspend-time hint: the thread sleeps in hardware until the phase completes or
// roughly `hint_ns` have passed.
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

// Dequantise 32 codes (BITS words) of one row into four 16-byte chunks (8 consecutive fp16 each).
// Codes 2i, 2i+1 are taken together: both fields are masked in place from a copy of their byte(s),
// (field | 0x6400) reads as 1024 + code * 2^p, one fused multiply-add with (2^-p) and
// -(1024 * 2^-p + zero) leaves code - zero exactly, one multiply applies the scale.  The four steps of a
// pair depend on each other; they are written stage by stage over eight pairs so that eight
// independent chains are in flight.
template <int BITS> struct Dequant32;

template <> struct Dequant32<4> {
    __device__ static __forceinline__ void run(const uint32_t (&w)[4], uint32_t zz, uint32_t ss, uint4 (&chunk)[4]) {
        const uint32_t add = h2sub(0xD400E400u, zz);                 // (-1024 - z, -64 - z)
#pragma unroll
        for (int i = 0; i < 4; i += 2) {                             // word i = codes 8i..8i+7 = chunk i
            uint32_t t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = __byte_perm(w[i + (j >> 2)], 0u, (j & 3) | ((j & 3) << 8));   // byte -> bytes 0 and 2
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = lop3_and_or(t[j], 0x00F0000Fu, kMagic);
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = h2fma(t[j], 0x2C003C00u, add);                                 // * (1, 1/16)
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = h2mul(t[j], ss);
            chunk[i] = make_uint4(t[0], t[1], t[2], t[3]);
            chunk[i + 1] = make_uint4(t[4], t[5], t[6], t[7]);
        }
    }
};

template <> struct Dequant32<2> {
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t zz, uint32_t ss, uint4 (&chunk)[4]) {
        const uint32_t add01 = h2sub(0xDC00E400u, zz);               // (-1024 - z, -256 - z)   fields at bits 0, 2
        const uint32_t add23 = h2sub(0xCC00D400u, zz);               // (-64 - z,  -16 - z)     fields at bits 4, 6
#pragma unroll
        for (int i = 0; i < 2; ++i) {                                // word i = codes 16i..16i+15 = chunks 2i, 2i+1
            uint32_t b[4], t[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = __byte_perm(w[i], 0u, j | (j << 8));                           // byte j = codes 4j..4j+3
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                t[2 * j] = lop3_and_or(b[j], 0x000C0003u, kMagic);
                t[2 * j + 1] = lop3_and_or(b[j], 0x00C00030u, kMagic);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                t[2 * j] = h2fma(t[2 * j], 0x34003C00u, add01);                                                 // * (1, 1/4)
                t[2 * j + 1] = h2fma(t[2 * j + 1], 0x24002C00u, add23);                                         // * (1/16, 1/64)
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = h2mul(t[j], ss);
            chunk[2 * i] = make_uint4(t[0], t[1], t[2], t[3]);
            chunk[2 * i + 1] = make_uint4(t[4], t[5], t[6], t[7]);
        }
    }
};

template <> struct Dequant32<3> {
    __device__ static __forceinline__ void run(const uint32_t (&w)[3], uint32_t zz, uint32_t ss, uint4 (&chunk)[4]) {
        const uint32_t add = h2sub(0xE400E400u, zz);                 // (-1024 - z) twice
#pragma unroll
        for (int c = 0; c < 4; c += 2) {                             // 16 codes -> two chunks
            uint32_t t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {                            // codes 2i, 2i+1 at stream bit 6i
                const int i = 4 * c + j, pos = 6 * i, wi = pos >> 5, off = pos & 31;
                if (off + 6 <= 32) t[j] = w[wi] >> off;
                else t[j] = __funnelshift_r(w[wi], w[wi + 1], off);  // codes that straddle a word
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = (t[j] & 0x3Fu) * 0x2001u;   // low code stays at bit 0, high code moves to bit 16
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = lop3_and_or(t[j], 0x00070007u, kMagic);
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = h2fma(t[j], 0x3C003C00u, add);
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = h2mul(t[j], ss);
            chunk[c] = make_uint4(t[0], t[1], t[2], t[3]);
            chunk[c + 1] = make_uint4(t[4], t[5], t[6], t[7]);
        }
    }
};

template <int BITS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const GemmParams P) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                    // swizzled tiles want 1024-byte alignment
    unsigned char* smem = smem_raw + (base - raw);
    constexpr uint32_t kPackedOff = kStages * kStageBytes;
    constexpr uint32_t kBarOff = kPackedOff + kPackedSlots * kPackedSlotBytes;
    constexpr int kWords = 2 * BITS;                                 // packed words of one row and stage (64 codes)
    constexpr uint32_t kRowBytes = 2 * kWords * 4;                   // one row of a packed super-block (128 codes)
    const uint32_t s_bar = base + kBarOff;
    // barriers: full_x[s], full_w[s], empty[s], tmem_full[2], tmem_empty[2], full_p[slot], empty_p[slot]
    auto full_x = [&](int s) { return s_bar + 8u * s; };
    auto full_w = [&](int s) { return s_bar + 8u * (kStages + s); };
    auto empty = [&](int s) { return s_bar + 8u * (2 * kStages + s); };
    auto tmem_full = [&](int a) { return s_bar + 8u * (3 * kStages + a); };
    auto tmem_empty = [&](int a) { return s_bar + 8u * (3 * kStages + 2 + a); };
    auto full_p = [&](int s) { return s_bar + 8u * (3 * kStages + 4 + s); };
    auto empty_p = [&](int s) { return s_bar + 8u * (3 * kStages + 4 + kPackedSlots + s); };
    constexpr uint32_t kNumBars = 3 * kStages + 4 + 2 * kPackedSlots;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kBarOff + 8 * kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kBarOff + 8 * kNumBars + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_x(s), 1);
            mbar_init(full_w(s), kDequantWarps);
            mbar_init(empty(s), 1);
        }
        for (int a = 0; a < 2; ++a) { mbar_init(tmem_full(a), 1); mbar_init(tmem_empty(a), 4); }
        for (int s = 0; s < kPackedSlots; ++s) { mbar_init(full_p(s), 1); mbar_init(empty_p(s), kDequantWarps); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // all 512 TMEM columns: two 128 x 256 fp32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32((const void*)tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int ntiles = P.tiles_m * P.tiles_n;
    const int nsuper = (P.kblocks + 1) >> 1;                         // packed super-blocks per tile
    int gave_up = 0;

    if (warp == 0) {
        // ================= TMA producer: x tiles =================
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < ntiles && !gave_up; tile += gridDim.x) {
                const int m0 = (tile % P.tiles_m) * kBM;
                for (int kb = 0; kb < P.kblocks; ++kb, ++it) {
                    const int s = it % kStages;
                    if (it >= kStages && !mbar_wait(empty(s), ((it / kStages) - 1) & 1, abort_flag)) { gave_up = 1; break; }
                    mbar_expect_tx(full_x(s), kXBytes);
                    tma_load_2d(base + s * kStageBytes, &xmap, kb * kBK, m0, full_x(s));
                }
            }
        }
    } else if (warp == kPackedWarp) {
        // ================= TMA producer: packed words, 256 rows x 128 codes per box =================
        if (lane == 0) {
            int pit = 0;
            for (int tile = blockIdx.x; tile < ntiles && !gave_up; tile += gridDim.x) {
                const int n0 = (tile / P.tiles_m) * kBN;
                for (int sb = 0; sb < nsuper; ++sb, ++pit) {
                    const int slot = pit % kPackedSlots;
                    if (pit >= kPackedSlots && !mbar_wait(empty_p(slot), ((pit / kPackedSlots) - 1) & 1, abort_flag)) { gave_up = 5; break; }
                    mbar_expect_tx(full_p(slot), kBN * kRowBytes);
                    tma_load_2d(base + kPackedOff + slot * kPackedSlotBytes, &wmap, sb * 2 * kWords, n0, full_p(slot));
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            int it = 0, tcount = 0;
            for (int tile = blockIdx.x; tile < ntiles && !gave_up; tile += gridDim.x, ++tcount) {
                const int acc = tcount & 1;
                if (tcount >= 2 && !mbar_wait(tmem_empty(acc), ((tcount >> 1) - 1) & 1, abort_flag)) { gave_up = 2; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)acc * kBN;
                for (int kb = 0; kb < P.kblocks; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!mbar_wait(full_x(s), ph, abort_flag) || !mbar_wait(full_w(s), ph, abort_flag)) { gave_up = 2; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t xa = base + s * kStageBytes, wa = xa + kXBytes;
                    // descriptors: K-major, 128-byte swizzle, 8-row atoms 1024 bytes apart
                    const uint64_t dhi = (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        const uint64_t adesc = dhi | (uint64_t)(((xa + k * 32) >> 4) & 0x3FFF);
                        const uint64_t bdesc = dhi | (uint64_t)(((wa + k * 32) >> 4) & 0x3FFF);
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                     " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                                     ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate), "r"(0u) : "memory");
                    }
                    // the stage may be refilled once these MMAs have read it
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(empty(s)) : "memory");
                }
                if (gave_up) break;
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tmem_full(acc)) : "memory");
            }
        }
    } else if (warp < kFirstEpiWarp) {
        // ================= dequantisers: half a weight row (32 codes) per thread and stage =================
        const int dq = (warp - kFirstDequantWarp) * 32 + lane;            // 0..511
        const int r = dq & 255, kh = dq >> 8;                             // row of the 256-row tile, which 32-code half
        const uint32_t row_off = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
        int it = 0, pit = 0;
        for (int tile = blockIdx.x; tile < ntiles && !gave_up; tile += gridDim.x) {
            const int n = (tile / P.tiles_m) * kBN + r;
            const bool live = n < P.N;
            const unsigned short* srow = reinterpret_cast<const unsigned short*>(P.scales) + (size_t)(live ? n : 0) * P.groups;
            const unsigned short* zrow = reinterpret_cast<const unsigned short*>(P.zeros) + (size_t)(live ? n : 0) * P.groups;
            // Scale and zero point of the two stages of a super-block, requested two super-blocks (four
            // stages) before their use: (zero << 16) | scale as raw fp16 bits, one word per stage.
            const bool one_group = (P.group_size % (2 * kBK)) == 0;   // both stages of a super-block share a group
            auto load_meta = [&](int sb, uint32_t& ma, uint32_t& mb) {
                ma = 0u; mb = 0u;
                if (live && sb < nsuper) {
                    const int ga = (2 * sb * kBK) / P.group_size;
                    ma = (uint32_t)__ldg(srow + ga) | ((uint32_t)__ldg(zrow + ga) << 16);
                    mb = ma;
                    if (!one_group) {
                        const int gb = ((2 * sb + 1) * kBK) / P.group_size;
                        mb = (uint32_t)__ldg(srow + gb) | ((uint32_t)__ldg(zrow + gb) << 16);
                    }
                }
            };
            uint32_t m0a, m0b, m1a, m1b, m2a, m2b;
            load_meta(0, m0a, m0b);
            load_meta(1, m1a, m1b);
            for (int sb = 0; sb < nsuper && !gave_up; ++sb, ++pit) {
                load_meta(sb + 2, m2a, m2b);
                const int slot = pit % kPackedSlots;
                if (!mbar_wait(full_p(slot), (pit / kPackedSlots) & 1, abort_flag)) { gave_up = 3; break; }
                const unsigned char* prow = smem + kPackedOff + slot * kPackedSlotBytes + (uint32_t)r * kRowBytes;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int kb = 2 * sb + half;
                    if (kb >= P.kblocks) break;
                    const int s = it % kStages;
                    const uint32_t meta = half == 0 ? m0a : m0b;
                    const uint32_t ss = (meta & 0xFFFFu) * 0x10001u, zz = (meta >> 16) * 0x10001u;
                    uint32_t w[BITS];
                    const unsigned char* src = prow + half * (kWords * 4) + kh * (BITS * 4);
                    if constexpr (BITS == 4) {
                        const uint4 a = *reinterpret_cast<const uint4*>(src);
                        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
                    } else if constexpr (BITS == 2) {
                        const uint2 a = *reinterpret_cast<const uint2*>(src);
                        w[0] = a.x; w[1] = a.y;
                    } else {
#pragma unroll
                        for (int i = 0; i < 3; ++i) w[i] = reinterpret_cast<const uint32_t*>(src)[i];
                    }
                    uint4 chunk[4];
                    Dequant32<BITS>::run(w, zz, ss, chunk);           // rows past N were zero-filled by the copy and get scale 0
                    if (it >= kStages && !mbar_wait(empty(s), ((it / kStages) - 1) & 1, abort_flag)) { gave_up = 3; break; }
                    unsigned char* wtile = smem + s * kStageBytes + kXBytes + row_off;
#pragma unroll
                    for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(wtile + (((4 * kh + c) ^ (r & 7)) << 4)) = chunk[c];
                    // make the generic-proxy writes visible to the tensor core's async-proxy reads, then signal
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_w(s));
                    ++it;
                }
                // the packed slot has been read by this warp
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_p(slot));
                m0a = m1a; m0b = m1b; m1a = m2a; m1b = m2b;
            }
        }
    } else if (warp < kPackedWarp) {
        // ================= epilogue: TMEM -> registers -> global =================
        const int q = warp & 3;                                       // the TMEM lane quadrant this warp may read
        int tcount = 0;
        for (int tile = blockIdx.x; tile < ntiles && !gave_up; tile += gridDim.x, ++tcount) {
            const int acc = tcount & 1;
            const int m = (tile % P.tiles_m) * kBM + q * 32 + lane;
            const int n0 = (tile / P.tiles_m) * kBN;
            if (!mbar_wait(tmem_full(acc), (tcount >> 1) & 1, abort_flag)) { gave_up = 4; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * kBN;
#pragma unroll 1
            for (int c0 = 0; c0 < kBN; c0 += 32) {
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
                if (m < P.M) {
                    __half* orow = P.out + (size_t)m * P.N + n0 + c0;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (n0 + c0 + j < P.N) {                          // N is a multiple of 8 on this path
                            uint32_t pk[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float a = __uint_as_float(v[j + 2 * e]), b = __uint_as_float(v[j + 2 * e + 1]);
                                if (P.bias != nullptr) {
                                    a += __half2float(P.bias[n0 + c0 + j + 2 * e]);
                                    b += __half2float(P.bias[n0 + c0 + j + 2 * e + 1]);
                                }
                                const __half2 h = __floats2half2_rn(activate(a, P.act), activate(b, P.act));
                                pk[e] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                            *reinterpret_cast<uint4*>(orow + j) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty(acc));
        }
    }

    if (gave_up) {
        *abort_flag = 1;
        atomicExch(&g_gemm_status, gave_up);
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

template <int BITS>
int launch_t(const CUtensorMap& xmap, const CUtensorMap& wmap, const GemmParams& P, int grid, cudaStream_t stream) {
    static bool attr_done[64] = {};
    int dev = 0;
    CB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        CB_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    gemm_tc_kernel<BITS><<<grid, kThreads, kSmemBytes, stream>>>(xmap, wmap, P);
    CB_CUDA_TRY(cudaGetLastError());
    return CB_OK;
}

}  // namespace

// CB_OK after launching; a CB_ERR_* code on a CUDA error; -1 when the problem is outside this kernel's
// domain (fp16, K a multiple of 128, group size a multiple of 64, N a multiple of 8, 16-byte aligned
// x / packed / out) and the caller should use the CUDA-core kernel.
int launch_gemm_tc(int dtype, const void* x, int64_t M, const cb_weight* w, void* out, int64_t K, int bits,
                   int64_t gs, int act, cudaStream_t stream) {
    if (dtype != CB_F16 || K % 128 != 0 || gs % kBK != 0 || w->n % 8 != 0 || M < 1) return -1;
    if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(w->packed) % 16 ||
        reinterpret_cast<uintptr_t>(out) % 16)
        return -1;
    if (M >= (1ll << 31) / 2 || K >= (1ll << 30)) return -1;
    EncodeTiledFn enc = encode_fn();
    if (enc == nullptr) return -1;
    const int sms = sm_count_current();
    if (sms <= 0) return CB_ERR_CUDA;

    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap xmap, wmap;
    {   // activations: [M, K] fp16, box 64 x 128, 128-byte swizzle (the UMMA K-major layout)
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBM};
        const CUresult cr = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) { set_error("packed_gemm: cuTensorMapEncodeTiled(x) failed (%d)", (int)cr); return CB_ERR_CUDA; }
    }
    {   // packed words: [N, K/32*bits] uint32, box (128 codes) x 256 rows, no swizzle
        const cuuint64_t wpr = (cuuint64_t)(K / 32) * bits;
        const cuuint64_t dims[2] = {wpr, (cuuint64_t)w->n};
        const cuuint64_t strides[1] = {wpr * 4};
        const cuuint32_t box[2] = {(cuuint32_t)(4 * bits), (cuuint32_t)kBN};
        const CUresult cr = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<int32_t*>(w->packed), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) { set_error("packed_gemm: cuTensorMapEncodeTiled(packed) failed (%d)", (int)cr); return CB_ERR_CUDA; }
    }

    GemmParams P{};
    P.scales = reinterpret_cast<const __half*>(w->scales);
    P.zeros = reinterpret_cast<const __half*>(w->zeros);
    P.bias = reinterpret_cast<const __half*>(w->bias);
    P.out = reinterpret_cast<__half*>(out);
    P.M = (int)M; P.N = (int)w->n; P.K = (int)K;
    P.groups = (int)((K + gs - 1) / gs); P.group_size = (int)gs; P.act = act;
    P.tiles_m = (int)((M + kBM - 1) / kBM); P.tiles_n = (int)((w->n + kBN - 1) / kBN); P.kblocks = (int)(K / kBK);
    const int grid = std::min(sms, P.tiles_m * P.tiles_n);
    switch (bits) {
        case 2: return launch_t<2>(xmap, wmap, P, grid, stream);
        case 3: return launch_t<3>(xmap, wmap, P, grid, stream);
        default: return launch_t<4>(xmap, wmap, P, grid, stream);
    }
}

int gemm_status_read_and_clear(int* out) {
    int v = 0, zero = 0;
    CB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)));
    CB_CUDA_TRY(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)));
    *out = v;
    return CB_OK;
}

}  // namespace cb
