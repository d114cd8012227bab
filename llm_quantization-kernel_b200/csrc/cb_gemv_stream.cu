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
#include "cb_frag.cuh"

namespace cb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kMaxRowsPerPass = 32;       // a pass is one or two 16-row MMA tiles (StreamParams::rpp)
constexpr int kMaxBuf = 6;
constexpr int kSpinLimit = 1 << 22;       // bounded mbarrier wait (~ a second), then give up and flag
constexpr size_t kSmemCap = 220 * 1024;       // one CTA per SM
constexpr size_t kSmemCapTwo = 112 * 1024;    // two CTAs per SM

__device__ int g_stream_status;
#ifdef CB_STREAM_TIMING
// Diagnostic build only: per-CTA nanosecond timestamps of the kernel's phases.
__device__ unsigned long long g_stream_times[1024][8];
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define CB_STAMP(i) do { if (threadIdx.x == 0 && blockIdx.x < 1024) { g_stream_times[blockIdx.x][i] = now_ns(); \
    if ((i) == 0) g_stream_times[blockIdx.x][7] = (unsigned long long)clock64(); \
    if ((i) == 6) g_stream_times[blockIdx.x][7] = (unsigned long long)clock64() - g_stream_times[blockIdx.x][7]; } } while (0)
#else
#define CB_STAMP(i) do { } while (0)
#endif           // 0 = ok; else the pass whose copy never landed, plus one

#ifdef CB_STREAM_DEBUG
#define CB_DBG(bit) (S.dbg & (bit))
#else
#define CB_DBG(bit) 0
#endif

struct StreamParams {
    GemvParams g;
    int nslabs;            // CTAs per K-partition
    int nbuf;              // ring depth
    int rpp;               // rows per pass: 32 or 16
    int dbg;               // diagnostic builds only: parts of the kernel to leave out
    int pitch;             // shared-memory bytes per staged row (row bytes + bank-spreading pad)
    int meta_stride;       // shared-memory bytes per staged row of scales (and of zeros)
    int slot_bytes;        // one ring slot: rpp weight rows, rpp scale rows, rpp zero rows
    int xb_stride;         // shared-memory bytes between batch rows of the staged activations
    int pair_q, pair_r;    // row pairs per slab: quotient and remainder of (V/2) / nslabs
    int grp_q, grp_r;      // group PAIRS per K-partition: quotient and remainder of (groups/2) / split_k
    unsigned off_x, off_red, off_ring, off_bar;   // shared-memory carve-up
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
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
// The mbarrier receives one arrival once all cp.async issued so far by this thread have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// One chunk (BITS words) from shared memory with the widest load its alignment allows.
template <int BITS> __device__ __forceinline__ void lds_chunk(const unsigned char* p, uint32_t (&w)[BITS]) {
    if constexpr (BITS == 4) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else if constexpr (BITS == 2) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        w[0] = v.x; w[1] = v.y;
    } else {
        const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
        w[0] = q[0]; w[1] = q[1]; w[2] = q[2];
    }
}

template <int BITS, bool BF>
__global__ void __launch_bounds__(kThreads, 2)
gemv_stream_kernel(const __half* __restrict__ x, const StreamParams S) {
    // BF: activations, scales, zeros and outputs are bfloat16 (the pointer types below only stand for "16-bit elements")
    using U = std::conditional_t<BF, UnpackB<BITS>, Unpack<BITS>>;
    using OutT = std::conditional_t<BF, __nv_bfloat16, __half>;
    extern __shared__ __align__(128) unsigned char smem[];
    // The next kernel of the stream may start right away: it only prefetches its own weights until
    // this grid has completed.
    asm volatile("griddepcontrol.launch_dependents;");
    CB_STAMP(0);
    const GemvParams& P = S.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr int kChunkBytes = 4 * BITS;            // one 32-code chunk
    constexpr int kGroupBytes = 4 * kChunkBytes;     // one 128-code group

    // ---- this CTA's share: K-partition `split`, row slab `slab`
    int split = 0, slab = blockIdx.x;
    if (P.split_k > 1) { split = blockIdx.x % P.split_k; slab = blockIdx.x / P.split_k; }
    const int g_begin = 2 * split_begin(split, S.grp_q, S.grp_r);
    const int ng = 2 * split_begin(split + 1, S.grp_q, S.grp_r) - g_begin;
    const int row_begin = 2 * split_begin(slab, S.pair_q, S.pair_r);
    const int row_end = min(P.V, 2 * split_begin(slab + 1, S.pair_q, S.pair_r));
    const int rpp = S.rpp;
    const int npass = (row_end - row_begin + rpp - 1) / rpp;
    const uint32_t row_bytes = (uint32_t)ng * kGroupBytes;

    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_ring = s_base + S.off_ring, s_bar = s_base + S.off_bar;
    float* red = reinterpret_cast<float*>(smem + S.off_red);         // [2][warps][2 tiles][32 lanes][4]

    if (tid == 0) {
        for (int b = 0; b < S.nbuf; ++b) mbar_init(s_bar + 8 * b, 33);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // Issue the copies of pass `p` into ring slot p % nbuf (warp 0, one row per lane): the packed row
    // with one bulk copy, its scales and zeros with 4-byte cp.async.  The slot's mbarrier completes
    // after the expect-tx arrival, the bulk bytes, and one arrival per lane once its cp.async landed.
    auto issue_pass = [&](int p) {
        const int buf = p % S.nbuf;
        const int row0 = row_begin + p * rpp;
        const int nrows = min(rpp, row_end - row0);
        const uint32_t slot = s_ring + (uint32_t)buf * S.slot_bytes;
        const uint32_t bar = s_bar + 8 * buf;
        if (lane == 0) mbar_expect_tx(bar, CB_DBG(4) ? 0u : (uint32_t)nrows * row_bytes);
        __syncwarp();
        if (lane < nrows) {
            int proj, lr;
            map_row(P, row0 + lane, proj, lr);
            const unsigned char* src = reinterpret_cast<const unsigned char*>(P.p[proj].w) +
                                       ((size_t)lr * P.wpr * 4 + (size_t)g_begin * kGroupBytes);
            if (!CB_DBG(4)) bulk_g2s(slot + (uint32_t)lane * S.pitch, src, row_bytes, bar);
            const __half* ssrc = reinterpret_cast<const __half*>(P.p[proj].s) + (size_t)lr * P.groups + g_begin;
            const __half* zsrc = reinterpret_cast<const __half*>(P.p[proj].z) + (size_t)lr * P.groups + g_begin;
            const uint32_t sdst = slot + rpp * S.pitch + (uint32_t)lane * S.meta_stride;
            const uint32_t zdst = sdst + rpp * S.meta_stride;
            for (int j = 0; j < (CB_DBG(1) ? 0 : ng); j += 2) {
                cp_async4(sdst + 2 * j, ssrc + j);
                cp_async4(zdst + 2 * j, zsrc + j);
            }
        }
        cp_async_arrive_noinc(bar);
    };
    if (warp == 0) {
        for (int p = 0; p < min(npass, S.nbuf); ++p) issue_pass(p);
    }
    CB_STAMP(1);

    // ---- this warp's groups inside the K-partition
    const int wg_begin = (ng * warp) >> 3, wg_end = (ng * (warp + 1)) >> 3;

    // Wait until everything the previous kernel wrote (our activations, the scratch) is visible.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const unsigned int peer_epoch = peer_wait(P);      // sharded stacks: the peers' slices of our activations have landed
    CB_STAMP(2);

    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
    // Lane (g, t) supplies the MMA B fragments of batch row g: the 32 activations of chunk t of each
    // group, read straight from global memory one group ahead of their use (the vector is small and
    // stays in L1/L2; staging it in shared memory would cost a CTA-wide barrier).
    const bool has_x = g < P.B;
    const __half* xrow = x + (size_t)(has_x ? g : 0) * P.K + (size_t)g_begin * 128 + t * 32;
    auto load_x = [&](int gl, uint32_t (&r)[16]) {
        if (has_x && gl < wg_end) {
            const uint4* xp = reinterpret_cast<const uint4*>(xrow + (size_t)gl * 128);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = __ldg(xp + i);
                r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = 0u;
        }
    };
    uint32_t xnext[16];
    load_x(wg_begin, xnext);
    int failed = 0;
    CB_STAMP(3);

    for (int p = 0; p < npass; ++p) {
        const int buf = p % S.nbuf;
        const int row0 = row_begin + p * rpp;
        const uint32_t parity = (uint32_t)((p / S.nbuf) & 1);
        const int ntile = (min(rpp, row_end - row0) + 15) >> 4;
        const unsigned char* rbase = smem + S.off_ring + (size_t)buf * S.slot_bytes;
        float* myred = red + (size_t)(p & 1) * (kWarps * 2 * 32 * 4);
        {   // bounded wait for this pass's rows
            int spins = 0;
            const uint32_t bar = s_bar + 8 * buf;
            while (!mbar_try_wait(bar, parity)) {
                if (++spins > kSpinLimit) { failed = p + 1; break; }
            }
        }
        if (p == 0) CB_STAMP(4);
        float acc[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

        for (int gl = wg_begin; gl < (CB_DBG(2) ? wg_begin : wg_end); ++gl) {
            // activations of this group, re-paired to match the unpack order; the next group's are requested now
            uint32_t xf[16];
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                const int lo = U::pair_lo(m), hi = lo + U::pair_gap();
                xf[m] = __byte_perm(xnext[lo >> 1], xnext[hi >> 1], (lo & 1) ? 0x7632 : 0x5410);
            }
            if (!CB_DBG(8)) load_x(gl + 1 < wg_end ? gl + 1 : wg_begin, xnext);      // wraps to the first group for the next pass
#pragma unroll
            for (int tile = 0; tile < 2; ++tile) {
                if (tile < ntile) {
                    const unsigned char* arow = rbase + (size_t)(tile * 16 + g) * S.pitch + (size_t)gl * kGroupBytes + (size_t)t * kChunkBytes;
                    const __half* s0 = reinterpret_cast<const __half*>(rbase + rpp * S.pitch + (size_t)(tile * 16 + g) * S.meta_stride);
                    const __half* s1 = s0 + 4 * S.meta_stride;                       // 8 rows further (stride is in bytes, pointer in halves)
                    const __half* z0 = s0 + (rpp / 2) * S.meta_stride;               // the zeros follow the scale rows
                    const __half* z1 = z0 + 4 * S.meta_stride;
                    // rows past the end of the slab were never copied: give them scale 0 and a finite zero point
                    const bool ok0 = row0 + tile * 16 + g < row_end, ok1 = row0 + tile * 16 + g + 8 < row_end;
                    const float cs0 = ok0 ? to_f32(reinterpret_cast<const OutT*>(s0)[gl]) : 0.f, cs1 = ok1 ? to_f32(reinterpret_cast<const OutT*>(s1)[gl]) : 0.f;
                    const uint32_t zr0 = ok0 ? (uint32_t)reinterpret_cast<const unsigned short*>(z0)[gl] : 0u;
                    const uint32_t zr1 = ok1 ? (uint32_t)reinterpret_cast<const unsigned short*>(z1)[gl] : 0u;
                    uint32_t ka[U::kConsts], kb[U::kConsts];
                    U::consts(zr0 | (zr0 << 16), ka);
                    U::consts(zr1 | (zr1 << 16), kb);
                    uint32_t wa[BITS], wb[BITS], ea[16], eb[16];
                    lds_chunk<BITS>(arow, wa);
                    lds_chunk<BITS>(arow + 8 * (size_t)S.pitch, wb);
                    if (CB_DBG(32)) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) { ea[i] = wa[i % BITS] + ka[0]; eb[i] = wb[i % BITS] + kb[0]; }
                    } else {
                    U::run(wa, ka, ea);
                    U::run(wb, kb, eb);
                    }
                    // Four independent accumulation chains of depth two: on this GPU a dependent mma.sync
                    // issues ~110 cycles after its predecessor, so the eight k-steps must not form one chain.
                    float d0[4], d1[4], d2[4], d3[4];
                    if (CB_DBG(16)) {
                        uint32_t h = 0;
#pragma unroll
                        for (int i = 0; i < 16; ++i) h ^= ea[i] ^ eb[i] ^ xf[i];
#pragma unroll
                        for (int j = 0; j < 4; ++j) { d0[j] = __uint_as_float(h & 0x3fffffff); d1[j] = d2[j] = d3[j] = 0.f; }
                    } else {
                    auto mma = [](float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                                  const float (&c)[4]) {
                        if constexpr (BF) mma16816_bf16(d, a0, a1, a2, a3, b0, b1, c);
                        else mma16816(d, a0, a1, a2, a3, b0, b1, c);
                    };
                    mma(d0, ea[0], eb[0], ea[1], eb[1], xf[0], xf[1], zero4);
                    mma(d1, ea[2], eb[2], ea[3], eb[3], xf[2], xf[3], zero4);
                    mma(d2, ea[4], eb[4], ea[5], eb[5], xf[4], xf[5], zero4);
                    mma(d3, ea[6], eb[6], ea[7], eb[7], xf[6], xf[7], zero4);
                    mma(d0, ea[8], eb[8], ea[9], eb[9], xf[8], xf[9], d0);
                    mma(d1, ea[10], eb[10], ea[11], eb[11], xf[10], xf[11], d1);
                    mma(d2, ea[12], eb[12], ea[13], eb[13], xf[12], xf[13], d2);
                    mma(d3, ea[14], eb[14], ea[15], eb[15], xf[14], xf[15], d3);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) { d0[j] = (d0[j] + d1[j]) + (d2[j] + d3[j]); d1[j] = 0.f; }
                    // acc += s * sum((q - z) x): rows g (d[0], d[1]) and g+8 (d[2], d[3]), batch columns 2t, 2t+1
                    acc[tile][0] = fmaf(cs0, d0[0] + d1[0], acc[tile][0]);
                    acc[tile][1] = fmaf(cs0, d0[1] + d1[1], acc[tile][1]);
                    acc[tile][2] = fmaf(cs1, d0[2] + d1[2], acc[tile][2]);
                    acc[tile][3] = fmaf(cs1, d0[3] + d1[3], acc[tile][3]);
                }
            }
        }
        // ---- hand the partial sums to the reduction (other warps covered other groups)
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
            *reinterpret_cast<float4*>(&myred[((warp * 2 + tile) * 32 + lane) * 4]) =
                make_float4(acc[tile][0], acc[tile][1], acc[tile][2], acc[tile][3]);
        if (p == 0) CB_STAMP(5);
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
            if (tile < ntile && v < row_end && b < P.B && !failed) {
                if (P.split_k == 1) epilogue<OutT>(P, b, v, mine, partner);
                else P.partial[((size_t)split * P.B + b) * P.V + v] = mine;
            }
        }
    }
    CB_STAMP(6);
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
                epilogue<OutT>(P, b, v, m, pt);
            }
            if (tid == 0) P.counters[slab] = 0;
        }
    }
    peer_signal(P, peer_epoch);
}

template <int BITS, bool BF>
int launch_t(const void* x, GemvParams P, int64_t rho, bool pdl, void* scratch, size_t scratch_bytes,
             cudaStream_t stream) {
    const int sms = sm_count_current();
    if (sms <= 0) return CB_ERR_CUDA;
    StreamParams S{};
    // K-partitions are whole PAIRS of groups (4-byte granularity of the metadata copies); the caller's
    // split_k is raised if the activations of one partition would not fit beside the weight ring.
    const int gpairs = P.groups / 2;
    int split = std::max(1, std::min(P.split_k, gpairs));
    const int group_bytes = 16 * BITS;
    auto layout = [&](int sp, int nbuf, int rpp, StreamParams& out) -> size_t {
        const int ng = 2 * ((gpairs + sp - 1) / sp);                  // largest partition
        int meta = ng * 2;
        meta += ((4 - meta) % 128 + 128) % 128;                        // rows 4 bytes apart (mod 128): conflict-free 2-byte reads
        int pitch = ng * group_bytes;
        pitch += ((group_bytes - pitch) % 128 + 128) % 128;           // pitch == group_bytes (mod 128): conflict-free fragment reads
        int xb = ng * 256;
        xb += ((64 - xb) % 128 + 128) % 128;                          // batch rows 64 bytes apart (mod 128)
        size_t off = 0;
        out.off_bar = (unsigned)off; off += 64;                      // one mbarrier per ring slot, at most 8 slots
        off = (off + 127) & ~(size_t)127;
        out.off_red = (unsigned)off; off += (size_t)2 * kWarps * 2 * 32 * 4 * sizeof(float);
        out.off_x = 0;
        off = (off + 127) & ~(size_t)127;
        out.slot_bytes = rpp * (pitch + 2 * meta);
        out.off_ring = (unsigned)off; off += (size_t)nbuf * out.slot_bytes;
        out.pitch = pitch; out.meta_stride = meta; out.xb_stride = xb; out.nbuf = nbuf; out.rpp = rpp;
        return off;
    };
    const int vpairs = (P.V + 1) / 2;
    // Slabs, passes and ring depth of a candidate (CTAs, split, rows per pass) under a shared-memory cap.
    struct Plan { int split, rpp, nbuf, nslabs, npass; bool ok; };
    auto plan = [&](int ctas, int sp, int rpp, size_t cap) -> Plan {
        Plan pl{sp, rpp, 0, 0, 0, false};
        StreamParams tmp{};
        if (layout(sp, 1, rpp, tmp) > cap) return pl;
        int nslabs = std::max(1, std::min(ctas / sp, (vpairs + 7) / 8));          // at least 16 rows per slab when possible
        nslabs = std::min(nslabs, vpairs);
        const int rows_per_slab = 2 * ((vpairs + nslabs - 1) / nslabs);
        pl.nslabs = nslabs;
        pl.npass = (rows_per_slab + rpp - 1) / rpp;
        pl.nbuf = std::min(pl.npass, kMaxBuf);
        while (pl.nbuf > 1 && layout(sp, pl.nbuf, rpp, tmp) > cap) --pl.nbuf;
        pl.ok = true;
        return pl;
    };
    // (1) One CTA per SM covers its rows in a single 32-row pass: do that, and leave the SM's second CTA slot to
    //     the next launch of the stream, whose prologue and first copies then overlap this launch's arithmetic.
    // (2) Otherwise prefer a ring that keeps copies in flight during the arithmetic (two slots or more): two CTAs
    //     per SM (twice the warps to hide latency) with 32- or 16-row passes, else one CTA per SM likewise.
    // (3) Otherwise one CTA per SM with a single slot, the K split raised until a slot fits.
    const int per_sm = rho <= 0 ? 2 : (int)std::min<int64_t>(std::max<int64_t>(rho, 2), 4);
    Plan pick{};
    {
        const Plan c = plan(sms, split, 32, kSmemCap);
        if (rho > 0 && rho <= 2 && c.ok && c.npass == 1) pick = c;
    }
    if (!pick.ok) {
        const struct { int ctas; size_t cap; } tries[2] = {{per_sm * sms, kSmemCapTwo}, {sms, kSmemCap}};
        for (int i = 0; i < 2 && !pick.ok; ++i)
            for (int rpp : {32, 16}) {
                const Plan c = plan(tries[i].ctas, split, rpp, tries[i].cap);
                if (c.ok && c.nbuf >= std::min(2, c.npass)) { pick = c; break; }
            }
    }
    if (!pick.ok) {
        int sp = split;
        while (!plan(sms, sp, 32, kSmemCap).ok && sp < gpairs) ++sp;
        pick = plan(sms, sp, 32, kSmemCap);
        if (!pick.ok) return -1;
    }
    split = pick.split;
    const int nslabs = pick.nslabs;
    if (split > 1 && nslabs > 65536) return -1;
    // scratch: [65536 counters | split x B x V partial sums]; without enough of it this path is not taken
    constexpr size_t kCounterBytes = 65536 * sizeof(int);
    if (split > 1) {
        const size_t need = kCounterBytes + (size_t)split * P.B * P.V * sizeof(float);
        if (scratch == nullptr || scratch_bytes < need || reinterpret_cast<uintptr_t>(scratch) % 16 != 0) return -1;
        P.counters = reinterpret_cast<int*>(scratch);
        P.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + kCounterBytes);
    }
    const size_t smem = layout(split, pick.nbuf, pick.rpp, S);
    P.split_k = split;
#ifdef CB_STREAM_DEBUG
    { const char* e = getenv("CB_GEMV_DEBUG"); S.dbg = e ? atoi(e) : 0; }
#endif
    S.g = P;
    S.nslabs = nslabs;
    S.pair_q = vpairs / nslabs; S.pair_r = vpairs % nslabs;
    S.grp_q = gpairs / split; S.grp_r = gpairs % split;

    static bool attr_done[64] = {};     // per device: the opt-in to large dynamic shared memory
    auto kern = gemv_stream_kernel<BITS, BF>;
    int dev = 0;
    CB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        CB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemCap));
        // every decode kernel asks for the same shared-memory carve-out, so that consecutive launches of a stream
        // never make an SM drain to re-partition its L1 / shared memory
        CB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
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
    if ((dtype != CB_F16 && dtype != CB_BF16) || P.group_size != 128 || P.K % 256 != 0 || P.B > kMaxBatchBlock || P.B < 1) return -1;
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0) return -1;
    for (int i = 0; i < 3; ++i)
        if (reinterpret_cast<uintptr_t>(P.p[i].w) % 16 != 0) return -1;
    if ((P.mode != CB_MODE_GEMV) && (P.V & 1)) return -1;
    switch (bits) {
        case 2: return dtype == CB_BF16 ? launch_t<2, true>(x, P, rho, pdl, scratch, scratch_bytes, stream)
                                        : launch_t<2, false>(x, P, rho, pdl, scratch, scratch_bytes, stream);
        case 3: return dtype == CB_BF16 ? launch_t<3, true>(x, P, rho, pdl, scratch, scratch_bytes, stream)
                                        : launch_t<3, false>(x, P, rho, pdl, scratch, scratch_bytes, stream);
        default: return dtype == CB_BF16 ? launch_t<4, true>(x, P, rho, pdl, scratch, scratch_bytes, stream)
                                         : launch_t<4, false>(x, P, rho, pdl, scratch, scratch_bytes, stream);
    }
}

int stream_status_read_and_clear(int* out) {
    int v = 0, zero = 0;
    CB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int)));
    CB_CUDA_TRY(cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int)));
    *out = v;
    return CB_OK;
}

#ifdef CB_STREAM_TIMING
}  // namespace cb
extern "C" int cb_debug_stream_times(unsigned long long* host, int ctas) {
    return (int)cudaMemcpyFromSymbol(host, cb::g_stream_times, sizeof(unsigned long long) * 8 * ctas);
}
namespace cb {
#endif

int occupancy_gemv_stream(int bits) {
    (void)bits;
    return 1;   // one persistent CTA per SM by construction (shared-memory ring)
}

}  // namespace cb
