// Ring decode GEMV for sm_100a: the memory-bound fast path (fp16 / bf16, group size 128, K a multiple of 256,
// batch <= 8, all three modes).
//
// Why it looks the way it does.  A 4096x4096 W4 matrix is 8.9 MB: at B200's HBM rate that is ~1.4 us of traffic,
// the same order as one DRAM round trip and as the hand-over between two kernels of a stream, so (1) every byte a
// CTA needs must be in flight at once, (2) the per-code ALU work must stay near one instruction per code PAIR, and
// (3) the stretch between "the activations exist" and "the outputs are stored" must be as short as possible.
//
//  (1) Each CTA owns a contiguous slab of virtual output rows and one of split_k K-partitions.  Rows of a slab are
//      fetched up to 32 at a time ("a pass") with one cp.async.bulk per row into a shared-memory ring guarded by
//      mbarriers; scales and zeros follow as 4-byte cp.async issued by all threads.  Where the matrix allows it every
//      CTA has a single pass and one, two or three CTAs share an SM (plan_stream).  The copies of the first passes
//      are issued before anything else, also before the kernel waits for its predecessor in the stream, so they
//      overlap the previous kernel.  Packed weights are assumed constant for the duration of the call.
//  (2) The 8 warps split the K-partition by quantisation group.  A packed word becomes MMA A operands with one
//      AND per code pair and nothing else (cb_frag.cuh, Frag<>): in fp16 the masked field is read as a subnormal
//      number, code * 2^(p-24) for a field at bit p, and the activations that meet it are multiplied by 2^-p when
//      they are staged, once per CTA, in the order the unpack produces codes.  mma.sync m16n8k16 (16 weight rows x
//      16 codes, up to 8 batch rows as the B operand, fp32 accumulation) then gives 2^-24 * sum(q x) per group; the
//      scale enters as one FMA per group, acc += s * sum(q x), and the zero-point terms  s * z * sum(x)  of a pass are
//      added up once per pass with lane = row and subtracted in the final reduction:
//      y = sum over groups of  s * (sum(q x) - z sum(x))   (Crispybits/Kernel/csrc/packed_gemv.cu:131-135).  The group
//      sums of x come from eight more MMAs per 8 (group, batch row) pairs with an all-ones A operand.  bf16 has too few mantissa
//      bits and too small an exponent range for the subnormal form: there (field | 0x4300) = 128 + code is used and
//      the 128 * sum(x') it adds is subtracted with the zero-point term.
//  (3) Hand-over.  A launch is a programmatic dependent launch: it may start (and prefetch weights) while its
//      predecessor in the stream runs, and it waits for the predecessor's completion (griddepcontrol.wait) before it
//      reads x or writes anything.  That completion event arrives ~1.5 us after the predecessor's last store on this
//      GPU, which is as long as a 4096x4096 matrix takes to stream.  Inside stream capture the host can do better for
//      launches that do not depend on one another: consecutive launches of this kernel on one capturing stream form a
//      CHAIN (a launch whose only capture dependency is the previous launch of this kernel, checked with
//      cudaStreamGetCaptureInfo; anything else in between starts a new chain).  The host knows the operands of every
//      launch of a chain, so a launch is one of two kinds:
//        - ORDERED (the first of a chain, and every launch whose x / out / scratch byte ranges overlap those of a launch
//          that may still be running): it waits for its predecessor's completion first and lets its own successor start
//          only after that wait, so a successor that starts knows that everything before the ordered launch is done;
//        - FREE (no overlap with any launch since the last ordered one): it does not wait at all and overlaps its
//          predecessors; only its first CTA waits for the predecessor's completion before it EXITS, so grids still
//          complete in launch order and whatever follows the chain sees all of it.
//      No device-side state is involved.  Outside capture every launch waits at once and triggers at once, as a plain
//      programmatic dependent launch does.  Free single-pass launches run a build of the kernel capped at 80 registers,
//      so that three launches of a chain fit an SM: independent launches then complete every (CTA lifetime) / 3.
//      In a column-parallel stack with the numbered hand-shake (PeerSync::on == 2) a launch is free in this sense too:
//      its dependency is the ranks' flags, which it polls before it reads x.
//
// The dot product is permutation-invariant, so the order in which codes meet MMA k-slots is chosen to suit the unpack.
#include <algorithm>
#include <map>
#include <mutex>

#include "cb_common.cuh"
#include "cb_frag.cuh"

namespace cb {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = 32 * kWarps;
constexpr int kRowLanes = kThreads / 32;        // threads that share one row of a pass when copies are issued and results reduced
constexpr int kMaxBuf = 6;
constexpr int kSpinLimit = 1 << 22;           // bounded mbarrier wait (~ a second), then give up and flag
constexpr size_t kSmemCap = 226 * 1024;       // one CTA per SM
constexpr size_t kSmemCapTwo = 112 * 1024;    // two CTAs per SM
constexpr size_t kSmemCapThree = 75 * 1024;   // three CTAs per SM (228 KB per SM, 1 KB reserved per CTA)

__device__ int g_stream_status;               // 0 = ok; k > 0: the copy of pass k-1 never landed

// How a launch relates to its predecessor in the stream (see the head of this file).
constexpr int kLaunchPlain = 0;      // wait at once, trigger at once (outside stream capture)
constexpr int kLaunchOrdered = 1;    // wait, then trigger (captured chain: this launch depends on earlier ones)
constexpr int kLaunchFree = 2;       // trigger at once, never wait before working; the first CTA waits before it exits

struct StreamParams {
    GemvParams g;
    int nslabs;            // CTAs per K-partition
    int nbuf;              // ring depth
    int rpp;               // rows per pass: 16 to 32, even
    int pitch;             // shared-memory bytes per staged row (row bytes + bank-spreading pad)
    int meta_stride;       // shared-memory bytes per staged row of scales (and of zeros)
    int slot_bytes;        // one ring slot: rpp weight rows, rpp scale rows, rpp zero rows
    int row_gran;          // slabs begin at multiples of this many virtual rows
    int pair_q, pair_r;    // row units per slab: quotient and remainder of ceil(V / row_gran) / nslabs
    int grp_q, grp_r;      // group PAIRS per K-partition: quotient and remainder of (groups/2) / split_k
    unsigned off_red, off_xs, off_xsum, off_ring, off_bar;   // shared-memory carve-up
    int launch_kind;       // kLaunchPlain / kLaunchOrdered / kLaunchFree
    int x_plane;           // bytes of one plane of staged activations: 16 * (groups of the largest partition) * B * 4
    int red_bufs;          // copies of the reduction buffer: 2 (alternating with the pass) or 1 (a single pass)
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
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
// The mbarrier receives one arrival once all cp.async issued so far by this thread have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// Shared-memory loads through 32-bit shared-window addresses (no generic-pointer arithmetic in the inner loop).
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ unsigned short lds16(uint32_t a) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t a, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// One chunk (BITS words) from shared memory with the widest load its alignment allows.
template <int BITS> __device__ __forceinline__ void lds_chunk(uint32_t a, uint32_t (&w)[BITS]) {
    if constexpr (BITS == 4) {
        const uint4 v = lds128(a);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else if constexpr (BITS == 2) {
        const uint2 v = lds64(a);
        w[0] = v.x; w[1] = v.y;
    } else {
        w[0] = lds32(a); w[1] = lds32(a + 4); w[2] = lds32(a + 8);
    }
}
template <bool BF> __device__ __forceinline__ float meta_f32(unsigned short bits) {
    if constexpr (BF) return __uint_as_float((uint32_t)bits << 16);
    else return __half2float(__ushort_as_half(bits));
}

// Staged activations: a block = the 64 bytes one (group, batch row, chunk) contributes, stored as four 16-byte pieces
// in four planes (piece i of block j at i * plane + 16 * j): the lanes of a warp read and write consecutive 16-byte
// pieces of one plane, which is conflict-free without padding.

// MINB = CTAs per SM the register allocation allows: 2 (up to 128 registers), or 3 (80 registers; a few spilled words)
// for single-pass launches small enough that THREE consecutive launches of a stream fit an SM together.
template <int BITS, int KIND, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
gemv_stream_kernel(const unsigned char* x, const StreamParams S) {
    // x is read with L2-coherent loads only (ld.global.cg): it is written while this grid is already resident, by the
    // previous kernel of the stream or, in a column-parallel stack, by peer GPUs.
    using F = Frag<BITS, KIND>;
    constexpr bool BF = F::kBf;      // activations, scales, zeros and outputs are bfloat16
    using OutT = std::conditional_t<BF, __nv_bfloat16, __half>;
    extern __shared__ __align__(128) unsigned char smem[];
    // The next kernel of the stream may start right away: it only prefetches its own weights until this grid lets it
    // go on.  An ordered launch of a captured chain holds its successor back until its own wait is over (below).
    if (S.launch_kind != kLaunchOrdered) asm volatile("griddepcontrol.launch_dependents;");
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
    const int row_begin = S.row_gran * split_begin(slab, S.pair_q, S.pair_r);
    const int row_end = min(P.V, S.row_gran * split_begin(slab + 1, S.pair_q, S.pair_r));
    const int rpp = S.rpp;
    const int npass = (row_end - row_begin + rpp - 1) / rpp;
    const uint32_t row_bytes = (uint32_t)ng * kGroupBytes;

    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_ring = s_base + S.off_ring, s_bar = s_base + S.off_bar, s_xs = s_base + S.off_xs;
    const uint32_t s_zero = s_base + S.off_bar + 64;      // 64 zero bytes: what lanes without a batch row load as activations
    // per pass parity: partial sums [warps][2 tiles][8 row pairs][tcols lanes][4], then zero-point terms [warps][32 rows][B]
    float* red = reinterpret_cast<float*>(smem + S.off_red);
    const int tcols = (P.B + 1) >> 1;                 // lanes t < tcols hold batch columns below B
    const int acc_floats = kWarps * 2 * 8 * tcols * 4;
    const int red_floats = acc_floats + kWarps * 32 * P.B;

    if (tid == 0) {
        for (int b = 0; b < S.nbuf; ++b) mbar_init(s_bar + 8 * b, kThreads + 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 16) reinterpret_cast<uint32_t*>(smem + S.off_bar + 64)[tid] = 0u;
    __syncthreads();

    // Issue the copies of pass `p` into ring slot p % nbuf.  Thread = (row of the pass, one eighth of the row's group
    // pairs).  The first thread of a row issues one bulk copy for the packed row (four rows per warp: bulk copies of
    // one warp are issued one after the other); every thread copies its share of the row's scales and zeros, 4 bytes
    // (two groups) per cp.async.  The slot's mbarrier completes after the expect-tx arrival, the bulk bytes, and one
    // arrival per thread once its cp.async have landed.
    auto issue_pass = [&](int p, int buf) {
        const int row0 = row_begin + p * rpp;
        const int nrows = min(rpp, row_end - row0);
        const uint32_t slot = s_ring + (uint32_t)buf * S.slot_bytes;
        const uint32_t bar = s_bar + 8 * buf;
        if (tid == 0) mbar_expect_tx(bar, (uint32_t)nrows * row_bytes);
        const int r = tid / kRowLanes;
        if (r < nrows) {
            int proj, lr;
            map_row(P, row0 + r, proj, lr);
            if ((tid % kRowLanes) == 0) {
                const unsigned char* src = reinterpret_cast<const unsigned char*>(P.p[proj].w) +
                                           ((size_t)lr * P.wpr * 4 + (size_t)g_begin * kGroupBytes);
                bulk_g2s(slot + (uint32_t)r * S.pitch, src, row_bytes, bar);
            }
            const __half* ssrc = reinterpret_cast<const __half*>(P.p[proj].s) + (size_t)lr * P.groups + g_begin;
            const __half* zsrc = reinterpret_cast<const __half*>(P.p[proj].z) + (size_t)lr * P.groups + g_begin;
            const uint32_t sdst = slot + rpp * S.pitch + (uint32_t)r * S.meta_stride;
            const uint32_t zdst = sdst + rpp * S.meta_stride;
            for (int j = 2 * (tid % kRowLanes); j < ng; j += 2 * kRowLanes) {
                cp_async4(sdst + 2 * j, ssrc + j);
                cp_async4(zdst + 2 * j, zsrc + j);
            }
        }
        cp_async_arrive_noinc(bar);
    };
    for (int p = 0; p < min(npass, S.nbuf); ++p) issue_pass(p, p);
    // Touch the activations' pages now (the values may be stale and are not used): address translation and the
    // request path are then warm when the real loads follow the hand-over.
    if (lane == 0) {
        unsigned int sink;
        asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(sink) : "l"(x + 2 * (size_t)(warp % P.B) * P.K + 256 * (size_t)(g_begin + (ng * warp) / kWarps)));
    }

    // ---- this warp's groups inside the K-partition
    const int wg_begin = (ng * warp) / kWarps, wg_end = (ng * (warp + 1)) / kWarps;
    int failed = 0;

    // ---- hand-over: after this block everything this launch depends on (its activations, earlier readers and writers of
    //      its outputs, the scratch) is complete and visible.  A free launch depends on nothing that may still run.
    if (S.launch_kind != kLaunchFree) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (S.launch_kind == kLaunchOrdered) asm volatile("griddepcontrol.launch_dependents;");
    }
    const unsigned int peer_epoch = peer_wait(P);      // sharded stacks: the peers' slices of our activations have landed

    // ---- activations of this warp's groups -> shared memory in MMA B-fragment order, scaled by 2^-shift; group sums.
    // One task = the 32 activations that one (batch row b, group, chunk t) contributes: a lane loads them, re-pairs
    // them to the unpack order and stores the 16 registers that lane (g = b, t) of the main loop will load back.
    // The four lanes of a quad hold the four chunks of one (group, batch row), i.e. one column of an MMA B operand:
    // eight MMAs with an all-ones A operand add the 128 values up in fp32 for the eight quads at once.
    float* xsum = reinterpret_cast<float*>(smem + S.off_xsum);         // [group][8]: sum(x) / unit, then [group][8]: base * sum(x')
    {
        const int ntask = (wg_end - wg_begin) * P.B * 4;
        for (int first = 0; first < ntask; first += 32) {
            const int id = first + lane;
            const bool on = id < ntask;
            const int q = id >> 2, tq = id & 3;
            const int ql = P.B == 1 ? q : q / P.B;
            const int gl = wg_begin + ql, b = q - ql * P.B;
            uint32_t raw[16];
            if (on) {
                const uint4* xp = reinterpret_cast<const uint4*>(x + 2 * ((size_t)b * P.K + (size_t)(g_begin + gl) * 128 + tq * 32));
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 v = __ldcg(xp + i);
                    raw[4 * i] = v.x; raw[4 * i + 1] = v.y; raw[4 * i + 2] = v.z; raw[4 * i + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) raw[i] = 0u;
            }
            // group sums first: the MMAs run while the activations are re-paired and stored
            const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
            float sa[4], sb[4], sc[4], sd[4];
            auto mma = [](float (&d)[4], uint32_t a, uint32_t b0, uint32_t b1, const float (&c)[4]) {
                if constexpr (BF) mma16816_bf16(d, a, a, a, a, b0, b1, c);
                else mma16816(d, a, a, a, a, b0, b1, c);
            };
            mma(sa, F::kOnes, raw[0], raw[1], zero4);
            mma(sb, F::kOnes, raw[2], raw[3], zero4);
            mma(sc, F::kOnes, raw[4], raw[5], zero4);
            mma(sd, F::kOnes, raw[6], raw[7], zero4);
            mma(sa, F::kOnes, raw[8], raw[9], sa);
            mma(sb, F::kOnes, raw[10], raw[11], sb);
            mma(sc, F::kOnes, raw[12], raw[13], sc);
            mma(sd, F::kOnes, raw[14], raw[15], sd);
            uint32_t xf[16];
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                const int lo = F::pair_lo(m), hi = F::pair_hi(m);          // same parity: one permute pairs them
                xf[m] = __byte_perm(raw[lo >> 1], raw[hi >> 1], (lo & 1) ? 0x7632 : 0x5410);
                if (F::scale2(m) != F::pow2neg2(0, 0)) xf[m] = F::mul2(xf[m], F::scale2(m));
            }
            if (on) {
                const uint32_t dst = s_xs + (uint32_t)(((gl * P.B + b) * 4 + tq) * 16);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    sts128(dst + (uint32_t)(i * S.x_plane), make_uint4(xf[4 * i], xf[4 * i + 1], xf[4 * i + 2], xf[4 * i + 3]));
            }
            float x0 = (sa[0] + sb[0]) + (sc[0] + sd[0]), x1 = (sa[1] + sb[1]) + (sc[1] + sd[1]);
            float c0 = 0.f, c1 = 0.f;
            if constexpr (F::kBase != 0.f) {
                mma(sa, F::kOnes, xf[0], xf[1], zero4);
                mma(sb, F::kOnes, xf[2], xf[3], zero4);
                mma(sc, F::kOnes, xf[4], xf[5], zero4);
                mma(sd, F::kOnes, xf[6], xf[7], zero4);
                mma(sa, F::kOnes, xf[8], xf[9], sa);
                mma(sb, F::kOnes, xf[10], xf[11], sb);
                mma(sc, F::kOnes, xf[12], xf[13], sc);
                mma(sd, F::kOnes, xf[14], xf[15], sd);
                c0 = F::kBase * ((sa[0] + sb[0]) + (sc[0] + sd[0]));
                c1 = F::kBase * ((sa[1] + sb[1]) + (sc[1] + sd[1]));
            }
            // lane l < 4 holds columns 2l and 2l+1, i.e. the quads 2l and 2l+1 of this round
            if (lane < 4) {
                const int q0 = (first >> 2) + 2 * lane;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int qq = q0 + j;
                    if (4 * qq < ntask) {
                        const int gq = P.B == 1 ? qq : qq / P.B;
                        const int at = (wg_begin + gq) * 8 + (qq - gq * P.B);
                        xsum[at] = (j ? x1 : x0) * (1.0f / F::kInvUnit);
                        if constexpr (F::kBase != 0.f) xsum[S.g.groups * 8 + at] = j ? c1 : c0;
                    }
                }
            }
        }
        __syncwarp();
    }

    // Lane (g, t) of the main loop supplies the MMA B fragments of batch row g: lanes without a batch row read zeros.
    const bool has_x = g < P.B;
    const uint32_t x_lane0 = has_x ? s_xs + (uint32_t)(((wg_begin * P.B + g) * 4 + t) * 16) : s_zero;
    const uint32_t x_step = has_x ? (uint32_t)(P.B * 4 * 16) : 0u;
    const uint32_t x_plane = has_x ? (uint32_t)S.x_plane : 16u;      // (the zero block is 64 bytes: its pieces sit side by side)
    const uint32_t p8 = 8u * S.pitch, m8 = 8u * S.meta_stride;
    const int ngw = wg_end - wg_begin;
    int buf = 0;
    uint32_t parity = 0u;              // ring slot of pass p and the phase of its mbarrier: p % nbuf, (p / nbuf) & 1
    for (int p = 0; p < npass; ++p) {
        const int row0 = row_begin + p * rpp;
        const int ntile = (min(rpp, row_end - row0) + 15) >> 4;
        const uint32_t slot = s_ring + (uint32_t)buf * S.slot_bytes;
        float* myred = red + (size_t)(p & (S.red_bufs - 1)) * red_floats;
        {   // bounded wait for this pass's rows
            int spins = 0;
            const uint32_t bar = s_bar + 8 * buf;
            while (!mbar_try_wait(bar, parity)) {
                if (++spins > kSpinLimit) { failed = p + 1; break; }
            }
        }
        float acc[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        // Rows past the end of the slab were never copied: their ring bytes are stale.  They only feed accumulator
        // rows that are never stored (rows are independent in the MMA), so nothing masks them here.
        uint32_t w_at = slot + (uint32_t)g * S.pitch + (uint32_t)(t * kChunkBytes + wg_begin * kGroupBytes);   // row g, this lane's chunk
        uint32_t m_at = slot + (uint32_t)rpp * S.pitch + (uint32_t)g * S.meta_stride + 2u * wg_begin;          // scale of row g
        uint32_t x_at = x_lane0;

        // One step = one group of this warp against TILES 16-row tiles of the pass: sum(q x) per (row, batch column),
        // times the scale.  Both tiles sit in one straight-line block so that the unpack of one overlaps the MMAs of
        // the other (a dependent mma.sync issues 110-150 cycles after its predecessor on this GPU; four independent
        // accumulation chains of depth two per tile).
        auto step = [&](auto tiles_tag, int tile0) {
            constexpr int TILES = decltype(tiles_tag)::value;
            const bool advance = TILES == 2 || tile0 == ntile - 1;
            uint32_t xf[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = lds128(x_at + i * x_plane);
                xf[4 * i] = v.x; xf[4 * i + 1] = v.y; xf[4 * i + 2] = v.z; xf[4 * i + 3] = v.w;
            }
            uint32_t wa[TILES][BITS], wb[TILES][BITS];
            float s0[TILES], s1[TILES];
#pragma unroll
            for (int tile = 0; tile < TILES; ++tile) {
                lds_chunk<BITS>(w_at + 2 * (tile + tile0) * p8, wa[tile]);
                lds_chunk<BITS>(w_at + (2 * (tile + tile0) + 1) * p8, wb[tile]);
                s0[tile] = meta_f32<BF>(lds16(m_at + 2 * (tile + tile0) * m8));
                s1[tile] = meta_f32<BF>(lds16(m_at + (2 * (tile + tile0) + 1) * m8));
            }
            float d[TILES][4][4];
            const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
            auto mma = [](float (&dd)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                          const float (&c)[4]) {
                if constexpr (BF) mma16816_bf16(dd, a0, a1, a2, a3, b0, b1, c);
                else mma16816(dd, a0, a1, a2, a3, b0, b1, c);
            };
#pragma unroll
            for (int tile = 0; tile < TILES; ++tile) {
                uint32_t ea[16], eb[16];
                F::run(wa[tile], ea);
                F::run(wb[tile], eb);
                mma(d[tile][0], ea[0], eb[0], ea[1], eb[1], xf[0], xf[1], zero4);
                mma(d[tile][1], ea[2], eb[2], ea[3], eb[3], xf[2], xf[3], zero4);
                mma(d[tile][2], ea[4], eb[4], ea[5], eb[5], xf[4], xf[5], zero4);
                mma(d[tile][3], ea[6], eb[6], ea[7], eb[7], xf[6], xf[7], zero4);
                mma(d[tile][0], ea[8], eb[8], ea[9], eb[9], xf[8], xf[9], d[tile][0]);
                mma(d[tile][1], ea[10], eb[10], ea[11], eb[11], xf[10], xf[11], d[tile][1]);
                mma(d[tile][2], ea[12], eb[12], ea[13], eb[13], xf[12], xf[13], d[tile][2]);
                mma(d[tile][3], ea[14], eb[14], ea[15], eb[15], xf[14], xf[15], d[tile][3]);
            }
#pragma unroll
            for (int tile = 0; tile < TILES; ++tile) {
                const float q0 = (d[tile][0][0] + d[tile][1][0]) + (d[tile][2][0] + d[tile][3][0]);
                const float q1 = (d[tile][0][1] + d[tile][1][1]) + (d[tile][2][1] + d[tile][3][1]);
                const float q2 = (d[tile][0][2] + d[tile][1][2]) + (d[tile][2][2] + d[tile][3][2]);
                const float q3 = (d[tile][0][3] + d[tile][1][3]) + (d[tile][2][3] + d[tile][3][3]);
                if (TILES == 2 ? tile == 0 : tile0 == 0) {
                    acc[0][0] = fmaf(s0[tile], q0, acc[0][0]); acc[0][1] = fmaf(s0[tile], q1, acc[0][1]);
                    acc[0][2] = fmaf(s1[tile], q2, acc[0][2]); acc[0][3] = fmaf(s1[tile], q3, acc[0][3]);
                } else {
                    acc[1][0] = fmaf(s0[tile], q0, acc[1][0]); acc[1][1] = fmaf(s0[tile], q1, acc[1][1]);
                    acc[1][2] = fmaf(s1[tile], q2, acc[1][2]); acc[1][3] = fmaf(s1[tile], q3, acc[1][3]);
                }
            }
            if (advance) {
                w_at += kGroupBytes;
                m_at += 2;
                x_at += x_step;
            }
        };
        if (ntile == 2) {
            for (int i = 0; i < ngw; ++i) step(std::integral_constant<int, 2>{}, 0);
        } else {
            for (int i = 0; i < ngw; ++i) {
                step(std::integral_constant<int, 1>{}, 0);
                if (ntile == 2) step(std::integral_constant<int, 1>{}, 1);
            }
        }
        // ---- zero-point (and operand-base) terms of this warp's groups: lane = row of the pass,
        //      sum over groups of  s * (z * sum(x) + base * sum(x'))  per batch row
        {
            // (a pass of 16 rows stages 16 rows of metadata: lanes past it compute a value nobody reads)
            uint32_t ms = slot + (uint32_t)rpp * S.pitch + (uint32_t)(lane < rpp ? lane : 0) * S.meta_stride + 2u * wg_begin;
            const uint32_t zoff = (uint32_t)rpp * S.meta_stride;
            float* cdst = myred + acc_floats + (warp * 32 + lane) * P.B;
            const float* xs0 = xsum + wg_begin * 8;
            if (P.B <= 2) {
                float c0 = 0.f, c1 = 0.f;
                for (int i = 0; i < ngw; ++i, ms += 2, xs0 += 8) {
                    const float sc = meta_f32<BF>(lds16(ms));
                    const float sz = sc * meta_f32<BF>(lds16(ms + zoff));
                    const float2 xz = *reinterpret_cast<const float2*>(xs0);
                    c0 = fmaf(sz, xz.x, c0);
                    c1 = fmaf(sz, xz.y, c1);
                    if constexpr (F::kBase != 0.f) {
                        const float2 xc = *reinterpret_cast<const float2*>(xs0 + S.g.groups * 8);
                        c0 = fmaf(sc, xc.x, c0);
                        c1 = fmaf(sc, xc.y, c1);
                    }
                }
                cdst[0] = c0;
                if (P.B == 2) cdst[1] = c1;
            } else {
                float c[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) c[j] = 0.f;
                for (int i = 0; i < ngw; ++i, ms += 2, xs0 += 8) {
                    const float sc = meta_f32<BF>(lds16(ms));
                    const float sz = sc * meta_f32<BF>(lds16(ms + zoff));
                    const float4 xa = *reinterpret_cast<const float4*>(xs0);
                    const float4 xb = *reinterpret_cast<const float4*>(xs0 + 4);
                    c[0] = fmaf(sz, xa.x, c[0]); c[1] = fmaf(sz, xa.y, c[1]); c[2] = fmaf(sz, xa.z, c[2]); c[3] = fmaf(sz, xa.w, c[3]);
                    c[4] = fmaf(sz, xb.x, c[4]); c[5] = fmaf(sz, xb.y, c[5]); c[6] = fmaf(sz, xb.z, c[6]); c[7] = fmaf(sz, xb.w, c[7]);
                    if constexpr (F::kBase != 0.f) {
                        const float4 ca = *reinterpret_cast<const float4*>(xs0 + S.g.groups * 8);
                        const float4 cb = *reinterpret_cast<const float4*>(xs0 + S.g.groups * 8 + 4);
                        c[0] = fmaf(sc, ca.x, c[0]); c[1] = fmaf(sc, ca.y, c[1]); c[2] = fmaf(sc, ca.z, c[2]); c[3] = fmaf(sc, ca.w, c[3]);
                        c[4] = fmaf(sc, cb.x, c[4]); c[5] = fmaf(sc, cb.y, c[5]); c[6] = fmaf(sc, cb.z, c[6]); c[7] = fmaf(sc, cb.w, c[7]);
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < P.B) cdst[j] = c[j];
            }
        }
        // ---- hand the partial sums to the reduction (other warps covered other groups): lanes whose batch columns exist
        if (t < tcols) {
#pragma unroll
            for (int tile = 0; tile < 2; ++tile)
                *reinterpret_cast<float4*>(&myred[(((warp * 2 + tile) * 8 + g) * tcols + t) * 4]) =
                    make_float4(acc[tile][0], acc[tile][1], acc[tile][2], acc[tile][3]);
        }
        __syncthreads();
        // the ring slot is free again: refill it with pass p + nbuf
        if (p + S.nbuf < npass) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_pass(p + S.nbuf, buf);
        }
        // ---- reduction over the warps and final step: warp -> batch row (rotating with the pass, so that the warps
        //      without one are already in the next pass), lane -> row of the pass
        const int b = (warp + kWarps - (p & (kWarps - 1))) & (kWarps - 1);
        if (b < P.B) {
            const int tile = lane >> 4, r = lane & 15;
            const int v = row0 + lane;
            // element of the partial-sum block of a (warp, tile): row pair r & 7, lane t = b / 2, value (r / 8) * 2 + (b & 1)
            const int wstride = 2 * 8 * tcols * 4;
            const float* ared = myred + ((tile * 8 + (r & 7)) * tcols + (b >> 1)) * 4 + (r >> 3) * 2 + (b & 1);
            const float* cred = myred + acc_floats + lane * P.B + b;
            float mine = 0.f, cm = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                mine += ared[w * wstride];
                cm += cred[w * 32 * P.B];
            }
            mine = (mine - cm) * F::kInvUnit;
            // the partner row (the up row of a gate row, the other half of a rotated pair) is the neighbouring row: the
            // neighbouring lane, since passes begin at even rows
            const float partner = __shfl_xor_sync(0xffffffffu, mine, 1);
            if (tile < ntile && v < row_end && !failed) {
                if (P.split_k == 1) epilogue<OutT>(P, b, v, mine, partner);
                else P.partial[((size_t)split * P.B + b) * P.V + v] = mine;
            }
        }
        if (++buf == S.nbuf) { buf = 0; parity ^= 1u; }
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
                epilogue<OutT>(P, b, v, m, pt);
            }
            if (tid == 0) P.counters[slab] = 0;
        }
    }
    // A free launch did not wait for its predecessor: its first CTA does so before it exits, so that this grid never
    // completes before the grid it was issued after.
    if (S.launch_kind == kLaunchFree && blockIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
    peer_signal(P, peer_epoch);
}

// ---- chains: which launches of a capture follow one another directly, and what they touch (host side) --------------
struct ChainKey {
    unsigned long long capture;
    cudaStream_t stream;
    bool operator<(const ChainKey& o) const { return capture != o.capture ? capture < o.capture : stream < o.stream; }
};
struct Range {
    uintptr_t lo, hi;
    bool overlaps(const Range& o) const { return lo < o.hi && o.lo < hi; }
};
struct LaunchRec {
    Range in;              // activations
    Range out[3];          // outputs
    int nout;
    bool scratch;          // Split-K partial sums and counters
    bool exclusive;        // rank hand-shake or peer stores: ordered after everything, and everything after it
};
constexpr int kMaxUnordered = 64;    // launches a chain may run without an ordered one in between
struct ChainState {
    cudaGraphNode_t last;              // the node of this library's latest launch on (capture, stream)
    int count;                         // launches since (and including) the last ordered one
    LaunchRec recs[kMaxUnordered];     // their operands: what a new launch must not overlap to run free
};
std::mutex g_chain_mutex;
std::map<ChainKey, ChainState> g_chains;
long long g_chain_counts[4] = {0, 0, 0, 0};    // chain heads, followers, followers that are ordered, followers that run free

// The stream's capture state: true and (id, the single node the next launch will depend on) when a capture is active.
bool capture_tail(cudaStream_t stream, unsigned long long* id, cudaGraphNode_t* tail) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    const cudaGraphNode_t* deps = nullptr;
    const cudaGraphEdgeData* edges = nullptr;
    size_t ndeps = 0;
    cudaGraph_t graph = nullptr;
    if (cudaStreamGetCaptureInfo_v3(stream, &st, id, &graph, &deps, &edges, &ndeps) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    if (st != cudaStreamCaptureStatusActive) return false;
    *tail = (ndeps == 1 && deps != nullptr) ? deps[0] : nullptr;
    return true;
}

// Does launch `a` read what launch `b` (issued earlier) wrote?
bool reads_from(const LaunchRec& a, const LaunchRec& b) {
    if (a.exclusive || b.exclusive || (a.scratch && b.scratch)) return true;
    for (int k = 0; k < b.nout; ++k)
        if (a.in.overlaps(b.out[k])) return true;
    return false;
}

// Does launch `a` have to be ordered after launch `b` (issued earlier)?
bool conflicts(const LaunchRec& a, const LaunchRec& b) {
    if (reads_from(a, b)) return true;                                                    // read after write
    for (int m = 0; m < a.nout; ++m) {
        if (a.out[m].overlaps(b.in)) return true;                                         // write after read
        for (int k = 0; k < b.nout; ++k)
            if (a.out[m].overlaps(b.out[k])) return true;                                 // write after write
    }
    return false;
}

// Shared-memory layout of one CTA for K split `sp`, ring depth `nbuf` and `rpp` rows per pass; returns its size.
// *overrun is set when a tile of the last ring slot would be read past the end of the allocation.
size_t stream_layout(int bits, int B, int groups, int sp, int nbuf, int rpp, int npass, StreamParams& out, bool* overrun) {
    const int gpairs = groups / 2;
    const int group_bytes = 16 * bits;
    const int ng = 2 * ((gpairs + sp - 1) / sp);                  // largest partition
    int meta = ng * 2;
    if ((meta / 4) % 2 == 0) meta += 4;                            // an odd number of banks from row to row: conflict-free 2-byte reads
    int pitch = ng * group_bytes;
    pitch += ((group_bytes - pitch) % 128 + 128) % 128;           // pitch == group_bytes (mod 128): conflict-free fragment reads
    size_t off = 0;
    out.off_bar = (unsigned)off; off += 128;                     // one mbarrier per ring slot (at most 8), then 64 zero bytes
    // The ring comes first.  A pass shorter than its tiles (16 rows each) still reads, and discards, the ring bytes of
    // the absent rows: past the last slot those reads land in the regions below, inside the allocation.
    out.slot_bytes = rpp * (pitch + 2 * meta);
    out.off_ring = (unsigned)off; off += (size_t)nbuf * out.slot_bytes;
    off = (off + 127) & ~(size_t)127;
    out.red_bufs = npass > 1 ? 2 : 1;                          // the reduction buffer alternates with the pass
    out.off_red = (unsigned)off; off += (size_t)out.red_bufs * (kWarps * 2 * 8 * ((B + 1) / 2) * 4 + kWarps * 32 * B) * sizeof(float);
    out.off_xsum = (unsigned)off; off += (size_t)2 * groups * 8 * sizeof(float);
    off = (off + 127) & ~(size_t)127;
    out.x_plane = ng * B * 4 * 16;
    out.off_xs = (unsigned)off; off += (size_t)4 * out.x_plane;   // staged activations of one partition
    out.pitch = pitch; out.meta_stride = meta; out.nbuf = nbuf; out.rpp = rpp;
    const size_t tile_rows = (size_t)((rpp + 15) / 16) * 16;
    const size_t reach = (size_t)out.off_ring + (size_t)(nbuf - 1) * out.slot_bytes + tile_rows * pitch;
    if (overrun) *overrun = reach > off;
    return off;
}

// The launch plan of the ring kernel: K split, row slabs, rows per pass, ring depth.  Pure host arithmetic.
struct StreamPlan { int split, rpp, nbuf, nslabs, npass; size_t smem; bool ok; bool three; };

bool plan_stream(int bits, int B, int V, int groups, int split_k, int64_t rho, int sms, StreamPlan* out) {
    // K-partitions are whole PAIRS of groups (4-byte granularity of the metadata copies); the caller's
    // split_k is raised if the activations of one partition would not fit beside the weight ring.
    const int gpairs = groups / 2;
    if (gpairs < 1 || V < 1 || sms < 1) return false;
    const int split = std::max(1, std::min(split_k, gpairs));
    // slabs are whole row PAIRS (the two operands of silu(gate)*up and of a rotation are neighbouring rows)
    const int gran = 2;
    const int vpairs = (V + gran - 1) / gran;
    // Slabs, passes and ring depth of a candidate (CTAs, split, rows per pass) under a shared-memory cap.
    auto plan = [&](int ctas, int sp, int rpp, size_t cap) -> StreamPlan {
        StreamPlan pl{sp, rpp, 0, 0, 0, 0, false};
        StreamParams tmp{};
        bool overrun = false;
        int nslabs = std::max(1, std::min(ctas / sp, (gran * vpairs + 15) / 16));          // at least 16 rows per slab when possible
        nslabs = std::min(nslabs, vpairs);
        const int rows_per_slab = gran * ((vpairs + nslabs - 1) / nslabs);
        // a slab shorter than a pass: the slot holds only the slab's rows (never fewer than 16: the scale reads of a
        // tile's absent rows then stay inside the slot's metadata)
        pl.rpp = std::max(16, std::min(rpp, rows_per_slab));
        pl.npass = (rows_per_slab + pl.rpp - 1) / pl.rpp;
        if (stream_layout(bits, B, groups, sp, 1, pl.rpp, pl.npass, tmp, &overrun) > cap || overrun) return pl;
        pl.nslabs = nslabs;
        pl.nbuf = std::min(pl.npass, kMaxBuf);
        while (pl.nbuf > 1 && (stream_layout(bits, B, groups, sp, pl.nbuf, pl.rpp, pl.npass, tmp, &overrun) > cap || overrun)) --pl.nbuf;
        pl.smem = stream_layout(bits, B, groups, sp, pl.nbuf, pl.rpp, pl.npass, tmp, &overrun);
        pl.ok = !overrun;
        return pl;
    };
    // The plan is chosen here; the caller's rho only reorders step (2) when it is negative (a tuning and test knob).
    // (1) If one CTA per SM covers its rows in a single pass of at most 32 rows inside half an SM's shared memory, do
    //     that and leave the SM's second CTA slot to the next launch of the stream, whose prologue and first copies
    //     then overlap this launch's arithmetic.
    // (2) Otherwise two CTAs per SM with half of its shared memory each, else one CTA per SM with all of it (measured:
    //     16 warps per SM hide the MMA latency that 8 do not; rho < 0 tries one CTA per SM first): 32-row passes (two 16-row tiles per step, eight accumulation chains per warp)
    //     with two ring slots or more; else, under two CTAs per SM, 32-row passes with one slot (the SM's other CTA
    //     computes while this one's slot refills: measured 8 % faster than the next choice, whose passes cost the
    //     same fixed work for half the rows); else 16-row passes with two slots or more.
    // (3) Otherwise one CTA per SM with a single slot, the K split raised until a slot fits.
    StreamPlan pick{};
    {
        const StreamPlan c = plan(sms, split, 32, kSmemCapTwo);
        if (c.ok && c.npass == 1) pick = c;
    }
    if (!pick.ok && rho >= 0) {
        // (1b) the same with two, then three CTAs per SM: every row of the matrix is in flight at once and no CTA loops.
        //      Three per SM need the 80-register build and a third of the shared memory each.
        const StreamPlan c2 = plan(2 * sms, split, 32, kSmemCapTwo);
        const StreamPlan c3 = plan(3 * sms, split, 32, kSmemCapThree);
        if (c2.ok && c2.npass == 1) pick = c2;
        else if (c3.ok && c3.npass == 1) { pick = c3; pick.three = true; }
    }
    if (!pick.ok) {
        const bool one_first = rho < 0;
        struct Try { int ctas; size_t cap; bool one_slot; };
        const Try one{sms, kSmemCap, false}, two{2 * sms, kSmemCapTwo, true};
        const Try tries[2] = {one_first ? one : two, one_first ? two : one};
        for (int i = 0; i < 2 && !pick.ok; ++i) {
            const StreamPlan c32 = plan(tries[i].ctas, split, 32, tries[i].cap);
            const StreamPlan c16 = plan(tries[i].ctas, split, 16, tries[i].cap);
            if (c32.ok && (c32.nbuf >= std::min(2, c32.npass) || tries[i].one_slot)) pick = c32;
            else if (c16.ok && c16.nbuf >= std::min(2, c16.npass)) pick = c16;
        }
    }
    if (!pick.ok) {
        int sp = split;
        while (!plan(sms, sp, 32, kSmemCap).ok && sp < gpairs) ++sp;
        pick = plan(sms, sp, 32, kSmemCap);
        if (!pick.ok) return false;
    }
    *out = pick;
    return true;
}

template <int BITS, int KIND>
int launch_t(const void* x, GemvParams P, int64_t rho, bool pdl, bool chains, void* scratch, size_t scratch_bytes,
             cudaStream_t stream) {
    const int sms = sm_count_current();
    if (sms <= 0) return CB_ERR_CUDA;
    StreamParams S{};
    StreamPlan pick{};
    if (!plan_stream(BITS, P.B, P.V, P.groups, P.split_k, rho, sms, &pick)) return -1;
    const int gran = 2;
    const int vpairs = (P.V + gran - 1) / gran;
    const int gpairs = P.groups / 2;
    int split = pick.split;
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
    const size_t smem = stream_layout(BITS, P.B, P.groups, split, pick.nbuf, pick.rpp, pick.npass, S, nullptr);
    P.split_k = split;
    S.g = P;
    S.nslabs = nslabs;
    S.row_gran = gran;
    S.pair_q = vpairs / nslabs; S.pair_r = vpairs % nslabs;
    S.grp_q = gpairs / split; S.grp_r = gpairs % split;
    const unsigned int grid = (unsigned)(nslabs * split);

    // Kind of this launch.  Inside stream capture: a follower if the capture's tail is this library's previous launch
    // on this stream, else the head of a new chain (ordered).  A follower runs free if its operands overlap those of
    // no launch since the chain's last ordered one, and that was at most kMaxUnordered - 1 launches ago.
    ChainKey key{0ull, stream};
    cudaGraphNode_t tail = nullptr;
    // A launch of a numbered hand-shake (sync.on == 2) takes no part in chains: its dependency is the ranks' flags.
    const bool numbered = P.sync.on == 2;
    const bool in_chain = !numbered && pdl && chains && capture_tail(stream, &key.capture, &tail);
    std::unique_lock<std::mutex> lock(g_chain_mutex, std::defer_lock);
    LaunchRec rec{};
    S.launch_kind = kLaunchPlain;
    bool follower = false;
    if (in_chain) {
        lock.lock();
        if (g_chains.size() > 4096) g_chains.clear();      // forgotten chains only mean that their next launch is a head
        auto it = g_chains.find(key);
        follower = it != g_chains.end() && tail != nullptr && it->second.last == tail;
        const size_t esz = 2;
        rec.in = Range{reinterpret_cast<uintptr_t>(x), reinterpret_cast<uintptr_t>(x) + (size_t)P.B * P.K * esz};
        rec.nout = P.mode == CB_MODE_QKV ? 3 : 1;
        for (int k = 0; k < rec.nout; ++k) {
            const uintptr_t o = reinterpret_cast<uintptr_t>(P.p[k].out);
            rec.out[k] = Range{o, o + (size_t)P.B * P.p[k].n * esz};
        }
        rec.scratch = split > 1;
        rec.exclusive = P.sync.on != 0 || P.n_peers > 0;
        bool free_run = follower && it->second.count < kMaxUnordered;
        if (free_run)
            for (int j = 0; j < it->second.count && free_run; ++j)
                if (conflicts(rec, it->second.recs[j])) free_run = false;
        S.launch_kind = free_run ? kLaunchFree : kLaunchOrdered;
        ++g_chain_counts[follower ? 1 : 0];
        if (follower) ++g_chain_counts[free_run ? 3 : 2];
    }
    // Numbered hand-shake: launch seq > 0 starts as soon as its predecessor lets it, never waits for that predecessor's
    // completion (it waits for the flags instead) and keeps the completion order like any free launch; launch 0 of a
    // step is an ordinary fully serialised launch, so that nothing of the step starts before the previous step's end.
    bool programmatic = pdl;
    if (numbered) {
        S.launch_kind = (P.sync.seq > 0u && pdl) ? kLaunchFree : kLaunchPlain;
        if (P.sync.seq == 0u) programmatic = false;
    }
    // Which build of the kernel.  A FREE single-pass launch of at most a third of an SM's shared memory runs the build
    // capped at 80 registers, so that three consecutive launches of the chain are resident per SM (measured at
    // 4096x4096, independent launches: W4 2.80 -> 2.57 us, W3 3.08 -> 2.91, W2 2.61 -> 2.23); so does a plan that puts
    // three CTAs of ONE launch on every SM (11008x4096 W4: 8.0 -> 7.1 us).  The capped build itself is 3-8 % slower, so
    // launches that wait for their predecessor anyway, and multi-pass launches, keep the other one.
    using Kern = void (*)(const unsigned char*, const StreamParams);
    Kern kern = gemv_stream_kernel<BITS, KIND, 2>;
    int which = 0;
    if ((S.launch_kind == kLaunchFree && !numbered && pick.npass == 1 && smem <= kSmemCapThree) || pick.three) {
        kern = gemv_stream_kernel<BITS, KIND, 3>;
        which = 1;
    }
    static bool attr_done_all[2][64] = {};     // per build and device: the opt-in to large dynamic shared memory
    bool* attr_done = attr_done_all[which];
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
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = programmatic ? 1 : 0;
    CB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, reinterpret_cast<const unsigned char*>(x), S));
    if (in_chain) {
        unsigned long long id = 0;
        cudaGraphNode_t node = nullptr;
        if (capture_tail(stream, &id, &node) && id == key.capture && node != nullptr) {
            ChainState& cs = g_chains[key];
            cs.last = node;
            if (S.launch_kind == kLaunchOrdered) cs.count = 0;      // everything before an ordered launch is done when its successors start
            cs.recs[cs.count++] = rec;
        } else {
            g_chains.erase(key);
        }
    }
    return CB_OK;
}

}  // namespace

// Returns CB_OK after launching, a CB_ERR_* code on a CUDA error, or -1 when this problem is outside
// the kernel's domain (the caller then uses the generic kernel).  `operands`: 0 = fp16 subnormal form, 1 = fp16
// with the 1024 offset (A/B checks); bf16 always uses its 128-offset form.
int launch_gemv_stream(int bits, int dtype, const void* x, const GemvParams& P, int64_t rho, bool pdl, bool chains,
                       int operands, void* scratch, size_t scratch_bytes, cudaStream_t stream) {
    if ((dtype != CB_F16 && dtype != CB_BF16) || P.group_size != 128 || P.K % 256 != 0 || P.B > kMaxBatchBlock || P.B < 1) return -1;
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0) return -1;
    for (int i = 0; i < 3; ++i)
        if (reinterpret_cast<uintptr_t>(P.p[i].w) % 16 != 0) return -1;
    if ((P.mode != CB_MODE_GEMV) && (P.V & 1)) return -1;
    const int kind = dtype == CB_BF16 ? kFragMagicB : (operands == 1 ? kFragMagicH : kFragSubnormal);
#define CB_STREAM_CASE(B_, K_) \
    if (bits == B_ && kind == K_) return launch_t<B_, K_>(x, P, rho, pdl, chains, scratch, scratch_bytes, stream);
    CB_STREAM_CASE(2, kFragSubnormal) CB_STREAM_CASE(3, kFragSubnormal) CB_STREAM_CASE(4, kFragSubnormal)
    CB_STREAM_CASE(2, kFragMagicH) CB_STREAM_CASE(3, kFragMagicH) CB_STREAM_CASE(4, kFragMagicH)
    CB_STREAM_CASE(2, kFragMagicB) CB_STREAM_CASE(3, kFragMagicB) CB_STREAM_CASE(4, kFragMagicB)
#undef CB_STREAM_CASE
    return -1;
}

// out7 = {grid, dynamic shared memory bytes, K split, rows per pass, ring slots, passes per CTA, row slabs}; false when the
// ring kernel does not take this problem.
bool stream_plan_query(int bits, int B, int V, int K, int split_k, int64_t rho, int sms, long long* out7) {
    if (K % 256 != 0 || B < 1 || B > kMaxBatchBlock || (bits != 2 && bits != 3 && bits != 4)) return false;
    StreamPlan pl{};
    if (!plan_stream(bits, B, V, K / 128, split_k, rho, sms, &pl)) return false;
    if (pl.split > 1 && pl.nslabs > 65536) return false;
    out7[0] = (long long)pl.nslabs * pl.split; out7[1] = (long long)pl.smem; out7[2] = pl.split; out7[3] = pl.rpp;
    out7[4] = pl.nbuf; out7[5] = pl.npass; out7[6] = pl.nslabs;
    return true;
}

void chain_stats(long long* out4) {
    std::lock_guard<std::mutex> lock(g_chain_mutex);
    for (int i = 0; i < 4; ++i) out4[i] = g_chain_counts[i];
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
