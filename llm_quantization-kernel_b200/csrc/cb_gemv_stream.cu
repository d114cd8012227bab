// Streamlined fp16 decode GEMV for sm_100a: the memory-bound fast path (group size 128, K a multiple
// of 128, batch <= 8, all three modes).
//
// Why it looks the way it does.  A 4096x4096 W4 matrix is 8.9 MB: at B200's HBM rate that is ~1.4 us
// of traffic, the same order as one DRAM round trip, so (1) every byte a CTA needs must be in flight
// at once, and (2) the per-code ALU work must stay far below one instruction per code.
//
//  (1) Each CTA owns a contiguous slab of virtual output rows (V / #slabs of them, not a multiple of a
//      tile) and one of split_k K-partitions.  Rows of a slab are fetched 32 at a time ("a pass") with
//      one cp.async.bulk per row into a shared-memory ring guarded by mbarriers; the copies of the
//      first passes are issued before anything else, also before the programmatic-dependent-launch
//      wait, so they overlap the tail of the previous kernel in the stream.  Packed weights are
//      assumed constant for the duration of the call.
//  (2) The 8 warps of the CTA split the K-partition by quantisation group.  A warp turns packed words
//      into exact fp16 integers with the (w & mask) | 0x6400 trick (two codes per LOP3, one HFMA2 to
//      remove the 1024 offset and the field's power-of-two scale; 3-bit codes are first aligned with
//      funnel shifts and byte permutes) and feeds them straight to mma.sync m16n8k16 as the A operand:
//      16 weight rows x 16 codes per instruction, activations of up to 8 batch rows as the B operand,
//      fp32 accumulation.  Products q*x are exact and sums are fp32, like the reference's
//      fmaf loop; per group the result enters the row accumulator as  s*D - (s*z)*sum(x)
//      (Crispybits/Kernel/csrc/packed_gemv.cu:131-135).  Partial sums of the warps meet in shared
//      memory; split_k > 1 additionally uses the same last-arriver fix-up as the generic kernel.
//
// The dot product is permutation-invariant, so the order in which codes meet MMA k-slots is chosen to
// suit the unpack: activations are staged once per CTA in that same order ("x fragments").
#include <algorithm>

#include "cb_common.cuh"

namespace cb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kRowsPerPass = 32;          // two 16-row MMA tiles
constexpr int kMaxBuf = 3;
constexpr int kSpinLimit = 1 << 22;       // bounded mbarrier wait (~ a second), then give up and flag
constexpr size_t kSmemCap = 220 * 1024;

__device__ int g_stream_status;           // 0 = ok; else the pass whose copy never landed, plus one

struct StreamParams {
    GemvParams g;
    int nslabs;            // CTAs per K-partition
    int nbuf;              // ring depth
    int pitch;             // shared-memory bytes per staged row (row bytes + bank-spreading pad)
    int xb_stride;         // bytes between batch rows of the x fragments
    int bpad;              // batch rows staged (>= B)
    unsigned off_x, off_xsum, off_red, off_ring, off_bar;   // shared-memory carve-up
};

// ---- small PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
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
__device__ __forceinline__ uint32_t h2add(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t a0, const uint32_t a1, const uint32_t a2,
                                         const uint32_t a3, const uint32_t b0, const uint32_t b1, const float (&c)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

constexpr uint32_t kMagic = 0x64006400u;      // half2(1024, 1024)
constexpr uint32_t kNeg1024 = 0xE400E400u;

// The 32 codes of one chunk -> 16 half2 registers of exact integer values.  e[m] holds the code pair
// pair_lo<BITS>(m), pair_lo<BITS>(m) + pair_gap<BITS>() (low half, high half).
template <int BITS> struct Unpack;

template <> struct Unpack<4> {
    // word i: e[4i+j] = (code 8i+j, code 8i+j+4)
    __device__ static __forceinline__ int pair_lo(int m) { return 8 * (m >> 2) + (m & 3); }
    __device__ static __forceinline__ int pair_gap() { return 4; }
    __device__ static __forceinline__ void run(const uint32_t (&w)[4], uint32_t (&e)[16]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t lo = w[i], hi = w[i] >> 8;
            e[4 * i + 0] = h2add(lop3_and_or(lo, 0x000F000Fu, kMagic), kNeg1024);
            e[4 * i + 1] = h2fma(lop3_and_or(lo, 0x00F000F0u, kMagic), 0x2C002C00u, 0xD400D400u);   // /16, -64
            e[4 * i + 2] = h2add(lop3_and_or(hi, 0x000F000Fu, kMagic), kNeg1024);
            e[4 * i + 3] = h2fma(lop3_and_or(hi, 0x00F000F0u, kMagic), 0x2C002C00u, 0xD400D400u);
        }
    }
};

template <> struct Unpack<2> {
    // word i: e[8i+j] = (code 16i+j, code 16i+j+8)
    __device__ static __forceinline__ int pair_lo(int m) { return 16 * (m >> 3) + (m & 7); }
    __device__ static __forceinline__ int pair_gap() { return 8; }
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t (&e)[16]) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t lo = w[i], hi = w[i] >> 10;
            e[8 * i + 0] = h2add(lop3_and_or(lo, 0x00030003u, kMagic), kNeg1024);
            e[8 * i + 1] = h2fma(lop3_and_or(lo, 0x000C000Cu, kMagic), 0x34003400u, 0xDC00DC00u);   // /4,   -256
            e[8 * i + 2] = h2fma(lop3_and_or(lo, 0x00300030u, kMagic), 0x2C002C00u, 0xD400D400u);   // /16,  -64
            e[8 * i + 3] = h2fma(lop3_and_or(lo, 0x00C000C0u, kMagic), 0x24002400u, 0xCC00CC00u);   // /64,  -16
            e[8 * i + 4] = h2fma(lop3_and_or(lo, 0x03000300u, kMagic), 0x1C001C00u, 0xC400C400u);   // /256, -4
            e[8 * i + 5] = h2add(lop3_and_or(hi, 0x00030003u, kMagic), kNeg1024);
            e[8 * i + 6] = h2fma(lop3_and_or(hi, 0x000C000Cu, kMagic), 0x34003400u, 0xDC00DC00u);
            e[8 * i + 7] = h2fma(lop3_and_or(hi, 0x00300030u, kMagic), 0x2C002C00u, 0xD400D400u);
        }
    }
};

template <> struct Unpack<3> {
    // e[j] = (code j, code j+16): the chunk is a 96-bit stream; code j sits at bit 3j, code j+16 at bit
    // 3j+48.  Windows of 15 bits (5 codes) of both halves are brought side by side into one register.
    __device__ static __forceinline__ int pair_lo(int m) { return m; }
    __device__ static __forceinline__ int pair_gap() { return 16; }
    __device__ static __forceinline__ void five(uint32_t p, uint32_t* e) {
        const uint32_t q = p >> 9;
        e[0] = h2add(lop3_and_or(p, 0x00070007u, kMagic), kNeg1024);
        e[1] = h2fma(lop3_and_or(p, 0x00380038u, kMagic), 0x30003000u, 0xD800D800u);   // /8,  -128
        e[2] = h2fma(lop3_and_or(p, 0x01C001C0u, kMagic), 0x24002400u, 0xCC00CC00u);   // /64, -16
        e[3] = h2add(lop3_and_or(q, 0x00070007u, kMagic), kNeg1024);
        e[4] = h2fma(lop3_and_or(q, 0x00380038u, kMagic), 0x30003000u, 0xD800D800u);
    }
    __device__ static __forceinline__ void run(const uint32_t (&w)[3], uint32_t (&e)[16]) {
        // stream bits [s, s+16) of the first half next to bits [48+s, 48+s+16) of the second half
        const uint32_t l1 = __funnelshift_r(w[0], w[1], 15), l2 = __funnelshift_r(w[0], w[1], 30);
        const uint32_t u0 = __funnelshift_r(w[1], w[2], 16), u1 = __funnelshift_r(w[1], w[2], 31), u2 = w[2] >> 14;
        five(__byte_perm(w[0], u0, 0x5410), e);
        five(__byte_perm(l1, u1, 0x5410), e + 5);
        five(__byte_perm(l2, u2, 0x5410), e + 10);
        const uint32_t last = __byte_perm(w[1] >> 13, w[2] >> 29, 0x5410);               // codes 15 and 31
        e[15] = h2add(lop3_and_or(last, 0x00070007u, kMagic), kNeg1024);
    }
};

template <int BITS> __device__ __forceinline__ void lds_chunk(uint32_t addr, uint32_t (&w)[BITS]) {
    if constexpr (BITS == 4)
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
    else if constexpr (BITS == 2)
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(addr));
    else {
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[0]) : "r"(addr));
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[1]) : "r"(addr + 4));
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[2]) : "r"(addr + 8));
    }
}

// Even split of n items into parts: start of part i.
__device__ __host__ __forceinline__ int part_begin(int n, int parts, int i) { return (int)(((long long)n * i) / parts); }

template <int BITS>
__global__ void __launch_bounds__(kThreads, 1)
gemv_stream_kernel(const __half* __restrict__ x, const StreamParams S) {
    extern __shared__ __align__(128) unsigned char smem[];
    const GemvParams& P = S.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr int kChunkBytes = 4 * BITS;            // one 32-code chunk
    constexpr int kGroupBytes = 4 * kChunkBytes;     // one 128-code group

    // ---- this CTA's share: K-partition `split`, row slab `slab`
    const int split = blockIdx.x % P.split_k, slab = blockIdx.x / P.split_k;
    const int g_begin = part_begin(P.groups, P.split_k, split), g_end = part_begin(P.groups, P.split_k, split + 1);
    const int ng = g_end - g_begin;
    const int vpairs = (P.V + 1) >> 1;
    const int row_begin = 2 * part_begin(vpairs, S.nslabs, slab);
    const int row_end = min(P.V, 2 * part_begin(vpairs, S.nslabs, slab + 1));
    const int npass = (row_end - row_begin + kRowsPerPass - 1) / kRowsPerPass;
    const uint32_t row_bytes = (uint32_t)ng * kGroupBytes;

    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_ring = s_base + S.off_ring, s_bar = s_base + S.off_bar, s_x = s_base + S.off_x;
    float* xsum = reinterpret_cast<float*>(smem + S.off_xsum);       // [ng][8]
    float* red = reinterpret_cast<float*>(smem + S.off_red);         // [2][warps][2 tiles][32 lanes][4]

    if (tid == 0) {
        for (int b = 0; b < S.nbuf; ++b) mbar_init(s_bar + 8 * b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // Issue the row copies of pass `p` into ring slot p % nbuf (warp 0, one row per lane).
    auto issue_pass = [&](int p) {
        const int buf = p % S.nbuf;
        const int row0 = row_begin + p * kRowsPerPass;
        const int nrows = min(kRowsPerPass, row_end - row0);
        const uint32_t bar = s_bar + 8 * buf;
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)nrows * row_bytes);
        __syncwarp();
        if (lane < nrows) {
            int proj, lr;
            map_row(P, row0 + lane, proj, lr);
            const unsigned char* src = reinterpret_cast<const unsigned char*>(P.p[proj].w) +
                                       ((size_t)lr * P.wpr * 4 + (size_t)g_begin * kGroupBytes);
            bulk_g2s(s_ring + (uint32_t)buf * (kRowsPerPass * S.pitch) + (uint32_t)lane * S.pitch, src, row_bytes, bar);
        }
    };
    if (warp == 0) {
        for (int p = 0; p < min(npass, S.nbuf); ++p) issue_pass(p);
    }
    // Let the next kernel of the stream start its own weight copies, then wait until everything the
    // previous kernel wrote (our activations, the scratch) is visible.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- stage activations as MMA B fragments: xfrag[b][group][i][t] = 16 bytes = e-order pairs 4i..4i+3
    // of chunk t of the group; xsum[group][b] = sum of the 128 activations.
    const int nitems = S.bpad * ng * 4;
    for (int base = 0; base < nitems; base += kThreads) {      // whole warps stay in the loop: it shuffles
        const int item = base + tid;
        const bool live = item < nitems;
        const int c = item & 3, gl = live ? (item >> 2) % ng : 0, b = live ? (item >> 2) / ng : 0;
        float sum = 0.f;
        uint32_t out[16];
#pragma unroll
        for (int m = 0; m < 16; ++m) out[m] = 0u;
        if (live && b < P.B) {
            const __half* src = x + (size_t)b * P.K + (size_t)(g_begin + gl) * 128 + c * 32;
            __half v[32];
            const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
            for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(v)[i] = __ldg(s4 + i);
#pragma unroll
            for (int j = 0; j < 32; ++j) sum += __half2float(v[j]);
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                const int lo = Unpack<BITS>::pair_lo(m);
                const __half2 pr = __halves2half2(v[lo], v[lo + Unpack<BITS>::pair_gap()]);
                out[m] = *reinterpret_cast<const uint32_t*>(&pr);
            }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (live) {
            unsigned char* dst = smem + S.off_x + (size_t)b * S.xb_stride + (size_t)gl * 256;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                *reinterpret_cast<uint4*>(dst + (i * 4 + c) * 16) =
                    make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
            if (c == 0) xsum[gl * 8 + b] = sum;
        }
    }
    // zero the sums of batch rows that do not exist (the epilogue math reads all eight)
    for (int i = tid; i < ng * 8; i += kThreads)
        if ((i & 7) >= S.bpad) xsum[i] = 0.f;
    __syncthreads();

    // ---- this warp's groups inside the K-partition
    const int wg_begin = part_begin(ng, kWarps, warp), wg_end = part_begin(ng, kWarps, warp + 1);
    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
    const bool has_x = g < S.bpad;
    int failed = 0;

    for (int p = 0; p < npass; ++p) {
        const int buf = p % S.nbuf;
        const int row0 = row_begin + p * kRowsPerPass;
        const uint32_t parity = (uint32_t)((p / S.nbuf) & 1);
        // scale/zero rows of this thread: rows g and g+8 of both tiles
        const __half* sp[4];
        const __half* zp[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int v = row0 + (r >> 1) * 16 + (r & 1) * 8 + g;
            int proj = 0, lr = 0;
            if (v < row_end) map_row(P, v, proj, lr);
            const bool ok = v < row_end;
            sp[r] = ok ? reinterpret_cast<const __half*>(P.p[proj].s) + (size_t)lr * P.groups + g_begin : nullptr;
            zp[r] = ok ? reinterpret_cast<const __half*>(P.p[proj].z) + (size_t)lr * P.groups + g_begin : nullptr;
        }
        float acc[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

        // first group's metadata goes out before we block on the weights
        float sc[4], sz[4];
        auto load_meta = [&](int gl) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                float s = 0.f, z = 0.f;
                if (sp[r] != nullptr && gl < wg_end) { s = __half2float(__ldg(sp[r] + gl)); z = __half2float(__ldg(zp[r] + gl)); }
                sc[r] = s; sz[r] = -s * z;
            }
        };
        load_meta(wg_begin);

        {   // bounded wait for this pass's rows
            int spins = 0;
            const uint32_t bar = s_bar + 8 * buf;
            while (!mbar_try_wait(bar, parity)) {
                if (++spins > kSpinLimit) { failed = p + 1; break; }
            }
        }
        const int ntile = (min(kRowsPerPass, row_end - row0) + 15) >> 4;
        const uint32_t rbase = s_ring + (uint32_t)buf * (kRowsPerPass * S.pitch);

        for (int gl = wg_begin; gl < wg_end; ++gl) {
            float cs[4], cz[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) { cs[r] = sc[r]; cz[r] = sz[r]; }
            if (gl + 1 < wg_end) load_meta(gl + 1);
            // activations of this group for batch row g
            uint32_t xf[16];
            if (has_x) {
                const uint32_t xa = s_x + (uint32_t)g * S.xb_stride + (uint32_t)gl * 256 + (uint32_t)t * 16;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(xf[4 * i]), "=r"(xf[4 * i + 1]), "=r"(xf[4 * i + 2]), "=r"(xf[4 * i + 3]) : "r"(xa + i * 64));
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) xf[i] = 0u;
            }
            const float2 xs = *reinterpret_cast<const float2*>(&xsum[gl * 8 + 2 * t]);
#pragma unroll
            for (int tile = 0; tile < 2; ++tile) {
                if (tile < ntile) {
                    uint32_t wa[BITS], wb[BITS], ea[16], eb[16];
                    const uint32_t a_addr = rbase + (uint32_t)(tile * 16 + g) * S.pitch + (uint32_t)gl * kGroupBytes + (uint32_t)t * kChunkBytes;
                    lds_chunk<BITS>(a_addr, wa);
                    lds_chunk<BITS>(a_addr + 8u * S.pitch, wb);
                    Unpack<BITS>::run(wa, ea);
                    Unpack<BITS>::run(wb, eb);
                    float d[4];
                    mma16816(d, ea[0], eb[0], ea[1], eb[1], xf[0], xf[1], zero4);
#pragma unroll
                    for (int m = 1; m < 8; ++m) mma16816(d, ea[2 * m], eb[2 * m], ea[2 * m + 1], eb[2 * m + 1], xf[2 * m], xf[2 * m + 1], d);
                    // acc += s*D - (s*z)*sum(x): rows g (d0,d1) and g+8 (d2,d3), batch columns 2t, 2t+1
                    acc[tile][0] = fmaf(cs[2 * tile], d[0], fmaf(cz[2 * tile], xs.x, acc[tile][0]));
                    acc[tile][1] = fmaf(cs[2 * tile], d[1], fmaf(cz[2 * tile], xs.y, acc[tile][1]));
                    acc[tile][2] = fmaf(cs[2 * tile + 1], d[2], fmaf(cz[2 * tile + 1], xs.x, acc[tile][2]));
                    acc[tile][3] = fmaf(cs[2 * tile + 1], d[3], fmaf(cz[2 * tile + 1], xs.y, acc[tile][3]));
                }
            }
        }

        // ---- meet the other warps (they covered other groups of the same rows)
        float* myred = red + (size_t)(p & 1) * (kWarps * 2 * 32 * 4);
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
            *reinterpret_cast<float4*>(&myred[((warp * 2 + tile) * 32 + lane) * 4]) =
                make_float4(acc[tile][0], acc[tile][1], acc[tile][2], acc[tile][3]);
        __syncthreads();
        // the ring slot is free again: refill it with pass p + nbuf
        if (warp == 0 && p + S.nbuf < npass) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_pass(p + S.nbuf);
        }
        {
            // thread -> (tile, row in tile, batch column)
            const int tile = tid >> 7, r = (tid >> 3) & 15, b = tid & 7;
            const int v = row0 + tile * 16 + r;
            const int fl = (r & 7) * 4 + (b >> 1), fe = (r >> 3) * 2 + (b & 1);
            const int pl = ((r ^ 1) & 7) * 4 + (b >> 1);
            float mine = 0.f, partner = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                mine += myred[((w * 2 + tile) * 32 + fl) * 4 + fe];
                partner += myred[((w * 2 + tile) * 32 + pl) * 4 + fe];
            }
            if (v < row_end && b < P.B && !failed) {
                if (P.split_k == 1) epilogue<__half>(P, b, v, mine, partner);
                else P.partial[((size_t)split * P.B + b) * P.V + v] = mine;
            }
        }
    }
    if (failed) atomicExch(&g_stream_status, failed);

    if (P.split_k > 1) {
        // Last CTA to arrive for this row slab adds the partial planes in split order and finishes
        // (counter reset by that CTA, so the scratch counters stay zero between calls).
        __shared__ int s_last;
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = (atomicAdd(P.counters + slab, 1) == P.split_k - 1) ? 1 : 0;
        __syncthreads();
        if (s_last) {
            __threadfence();
            const int nrow = row_end - row_begin;
            for (int e = tid; e < nrow * P.B; e += kThreads) {
                const int v = row_begin + e % nrow, b = e / nrow;
                float m = 0.f, pt = 0.f;
                const bool has_partner = (v ^ 1) < P.V;
                for (int s = 0; s < P.split_k; ++s) {
                    const float* ps = P.partial + ((size_t)s * P.B + b) * P.V;
                    m += __ldcg(ps + v);
                    if (has_partner) pt += __ldcg(ps + (v ^ 1));
                }
                epilogue<__half>(P, b, v, m, pt);
            }
            if (tid == 0) P.counters[slab] = 0;
        }
    }
}

template <int BITS>
int launch_t(const void* x, GemvParams P, int64_t rho, bool pdl, void* scratch, size_t scratch_bytes,
             cudaStream_t stream) {
    const int sms = sm_count_current();
    if (sms <= 0) return CB_ERR_CUDA;
    StreamParams S{};
    // K-partitions: the caller's split_k in units of groups, raised if the x fragments of one
    // partition would not fit beside the weight ring.
    int split = std::max(1, std::min(P.split_k, P.groups));
    const int bpad = P.B <= 1 ? 1 : (P.B <= 2 ? 2 : (P.B <= 4 ? 4 : 8));
    const int group_bytes = 16 * BITS;
    auto layout = [&](int sp, int nbuf, StreamParams& out) -> size_t {
        const int ng = (P.groups + sp - 1) / sp;                      // largest partition
        int pitch = ng * group_bytes;
        pitch += ((group_bytes - pitch) % 128 + 128) % 128;           // pitch == group_bytes (mod 128): conflict-free fragment reads
        int xb = ng * 256;
        xb += ((64 - xb) % 128 + 128) % 128;                          // batch rows 64 bytes apart (mod 128)
        size_t off = 0;
        out.off_bar = (unsigned)off; off += 64;
        out.off_xsum = (unsigned)off; off += (size_t)ng * 8 * sizeof(float);
        off = (off + 127) & ~(size_t)127;
        out.off_red = (unsigned)off; off += (size_t)2 * kWarps * 2 * 32 * 4 * sizeof(float);
        out.off_x = (unsigned)off; off += (size_t)bpad * xb;
        off = (off + 127) & ~(size_t)127;
        out.off_ring = (unsigned)off; off += (size_t)nbuf * kRowsPerPass * pitch;
        out.pitch = pitch; out.xb_stride = xb; out.nbuf = nbuf; out.bpad = bpad;
        return off;
    };
    while (layout(split, 1, S) > kSmemCap && split < P.groups) ++split;
    if (layout(split, 1, S) > kSmemCap) return -1;
    // scratch: [65536 counters | split x B x V partial sums]; without enough of it this path is not taken
    constexpr size_t kCounterBytes = 65536 * sizeof(int);
    if (split > 1) {
        const size_t need = kCounterBytes + (size_t)split * P.B * P.V * sizeof(float);
        if (scratch == nullptr || scratch_bytes < need || reinterpret_cast<uintptr_t>(scratch) % 16 != 0) return -1;
        P.counters = reinterpret_cast<int*>(scratch);
        P.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + kCounterBytes);
    }
    const int ctas = rho <= 0 ? 2 * sms : (int)std::min<int64_t>(rho, 4) * sms;   // rho 0: no persistence wanted -> small slabs
    const int vpairs = (P.V + 1) / 2;
    int nslabs = std::max(1, std::min(ctas / split, (vpairs + 7) / 8));           // at least 16 rows per slab when possible
    nslabs = std::min(nslabs, vpairs);
    if (split > 1 && nslabs > 65536) return -1;
    const int rows_per_slab = 2 * ((vpairs + nslabs - 1) / nslabs);
    const int npass = (rows_per_slab + kRowsPerPass - 1) / kRowsPerPass;
    int nbuf = std::min(npass, kMaxBuf);
    while (nbuf > 1 && layout(split, nbuf, S) > kSmemCap) --nbuf;
    const size_t smem = layout(split, nbuf, S);
    P.split_k = split;
    S.g = P;
    S.nslabs = nslabs;

    static bool attr_done[64] = {};     // per device: the opt-in to large dynamic shared memory
    auto kern = gemv_stream_kernel<BITS>;
    int dev = 0;
    CB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        CB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemCap));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(nslabs * split));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    CB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, reinterpret_cast<const __half*>(x), S));
    return CB_OK;
}

}  // namespace

// Returns CB_OK after launching, a CB_ERR_* code on a CUDA error, or -1 when this problem is outside
// the kernel's domain (the caller then uses the generic kernel).
int launch_gemv_stream(int bits, int dtype, const void* x, const GemvParams& P, int64_t rho, bool pdl,
                       void* scratch, size_t scratch_bytes, cudaStream_t stream) {
    if (dtype != CB_F16 || P.group_size != 128 || P.K % 128 != 0 || P.B > kMaxBatchBlock || P.B < 1) return -1;
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0) return -1;
    for (int i = 0; i < 3; ++i)
        if (reinterpret_cast<uintptr_t>(P.p[i].w) % 16 != 0) return -1;
    if ((P.mode != CB_MODE_GEMV) && (P.V & 1)) return -1;
    switch (bits) {
        case 2: return launch_t<2>(x, P, rho, pdl, scratch, scratch_bytes, stream);
        case 3: return launch_t<3>(x, P, rho, pdl, scratch, scratch_bytes, stream);
        default: return launch_t<4>(x, P, rho, pdl, scratch, scratch_bytes, stream);
    }
}

int stream_status_read_and_clear(int* out) {
    int v = 0, zero = 0;
    CB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int)));
    CB_CUDA_TRY(cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int)));
    *out = v;
    return CB_OK;
}

int occupancy_gemv_stream(int bits) {
    (void)bits;
    return 1;   // one persistent CTA per SM by construction (shared-memory ring)
}

}  // namespace cb
