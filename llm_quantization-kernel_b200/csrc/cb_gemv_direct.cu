// Register-streaming fp16 decode GEMV for sm_100a (group size 128, K a multiple of 2048, batch <= 8, all
// three modes): packed words go from global memory straight into the registers that feed mma.sync.
//
// A CTA owns a contiguous range of 16-row tiles of the virtual output rows; its 8 warps split K into 8
// slices of whole group pairs and all work on the same tile.  Lane (g, t) of a warp is responsible for
// tile rows g and g + 8 and, of every quantisation group, for the 32 codes of chunk t -- exactly the
// codes whose unpacked fp16 values it must hold as the A fragment of mma.sync m16n8k16 (the dot product is
// permutation-invariant, so the order in which codes meet the MMA k-slots is chosen to suit the unpack).
// Per group pair a lane therefore loads its two rows' chunks with plain vector loads (the four t-lanes
// of a row read one contiguous 16*BITS-byte piece: whole 32-byte sectors, nothing fetched twice) and the
// rows' scales and zeros as half2.  Loads run two group pairs ahead of the arithmetic in a register
// double buffer, across tile boundaries, and the first two are issued before the programmatic-dependent-
// launch wait, so they overlap the tail of the previous kernel of the stream.  There is no shared-memory
// staging of weights, no mbarrier and no spin-wait anywhere in this kernel.
//
// Activations are staged once per CTA in shared memory, already in MMA B-fragment order ("x fragments"),
// and swizzled so that the 128-bit reads of a quarter-warp touch all banks once.  Unpacking, the per-group
// algebra  acc += s * sum((q - z) * x)  and the epilogues are those of the ring kernel
// (Crispybits/Kernel/csrc/packed_gemv.cu:131-135 and :54-81).  Warp partial sums meet in shared memory once
// per tile.
#include <algorithm>

#include "cb_common.cuh"
#include "cb_frag.cuh"

namespace cb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr size_t kSmemCapOne = 220 * 1024;   // one CTA per SM
constexpr size_t kSmemCapTwo = 110 * 1024;   // two CTAs per SM

struct DirectParams {
    GemvParams g;
    int tile_q, tile_r;    // 16-row tiles per CTA: quotient and remainder of tiles / CTAs
    int pair_q, pair_r;    // group pairs per warp: quotient and remainder of (groups / 2) / 8
    int nb;                // batch rows staged in shared memory (= B)
    unsigned off_red;      // shared-memory offset of the warp partial sums (the x fragments start at 0)
};

template <int N> __device__ __forceinline__ void ldg_words(const unsigned char* p, uint32_t (&w)[N]) {
    if constexpr (N == 4) {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "l"(p));
    } else if constexpr (N == 2) {
        asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "l"(p));
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i)
            asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(w[i]) : "l"(p + 4 * i));
    }
}

__device__ __forceinline__ uint32_t ldg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// What one lane holds of one (tile, group pair): chunk t of both groups for rows g and g + 8, and the
// two rows' scales and zeros of both groups.
template <int BITS> struct Stage {
    uint32_t w[2][2][BITS];   // [group of the pair][row g / g+8][words]
    uint32_t s[2], z[2];      // half2 (group 2p, group 2p+1) for row g and row g+8
};

template <int BITS>
__global__ void __launch_bounds__(kThreads, 2)
gemv_direct_kernel(const __half* __restrict__ x, const DirectParams S) {
    extern __shared__ __align__(128) unsigned char smem[];
    asm volatile("griddepcontrol.launch_dependents;");
    const GemvParams& P = S.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr int kChunkBytes = 4 * BITS;
    constexpr int kGroupBytes = 4 * kChunkBytes;

    const int tile_begin = split_begin(blockIdx.x, S.tile_q, S.tile_r);
    const int ntile = split_begin(blockIdx.x + 1, S.tile_q, S.tile_r) - tile_begin;
    const int pair_begin = split_begin(warp, S.pair_q, S.pair_r);
    const int npair = split_begin(warp + 1, S.pair_q, S.pair_r) - pair_begin;     // >= 1 by the launcher's rule
    const int nsteps = ntile * npair;
    float* red = reinterpret_cast<float*>(smem + S.off_red);                      // [2][warps][32 lanes][4]

    // ---- loads of step (tile, pair): issued `two steps ahead'
    int ld_tile = tile_begin, ld_pair = 0;          // the step the next load() fetches
    const unsigned char* wrow[2];
    const __half* srow[2];
    const __half* zrow[2];
    auto set_rows = [&](int tile) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int v = min(tile * 16 + g + 8 * h, P.V - 1);      // rows past the end re-read the last row; never stored
            int proj, r;
            map_row(P, v, proj, r);
            wrow[h] = reinterpret_cast<const unsigned char*>(P.p[proj].w) + (size_t)r * P.wpr * 4 + (size_t)t * kChunkBytes +
                      (size_t)(2 * pair_begin) * kGroupBytes;
            srow[h] = reinterpret_cast<const __half*>(P.p[proj].s) + (size_t)r * P.groups + 2 * pair_begin;
            zrow[h] = reinterpret_cast<const __half*>(P.p[proj].z) + (size_t)r * P.groups + 2 * pair_begin;
        }
    };
    set_rows(ld_tile);
    auto load = [&](Stage<BITS>& st) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            ldg_words<BITS>(wrow[h], st.w[0][h]);
            ldg_words<BITS>(wrow[h] + kGroupBytes, st.w[1][h]);
            st.s[h] = ldg_u32(srow[h]);
            st.z[h] = ldg_u32(zrow[h]);
            wrow[h] += 2 * kGroupBytes; srow[h] += 2; zrow[h] += 2;
        }
        if (++ld_pair == npair) {
            ld_pair = 0;
            ++ld_tile;
            set_rows(min(ld_tile, tile_begin + ntile - 1));
        }
    };
    Stage<BITS> sa, sb;
    load(sa);
    if (nsteps > 1) load(sb);

    // ---- activations -> shared memory, in B-fragment order.  Block (group, t, b) is 64 bytes: the 16 half2
    // registers of lane (b, t) for that group, its four 16-byte pieces rotated by t against bank conflicts.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const unsigned int peer_epoch = peer_wait(P);
    {
        const int nblocks = S.nb * (P.K >> 5);
        for (int bid = tid; bid < nblocks; bid += kThreads) {
            const int c = bid / S.nb, b = bid - c * S.nb;            // c = group * 4 + t
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)b * P.K + (size_t)c * 32);
            uint32_t raw[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = __ldcg(src + i);       // written by the previous kernel (or a peer): L2 is the point of coherence
                raw[4 * i] = v.x; raw[4 * i + 1] = v.y; raw[4 * i + 2] = v.z; raw[4 * i + 3] = v.w;
            }
            uint32_t xf[16];
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                const int lo = Unpack<BITS>::pair_lo(m), hi = lo + Unpack<BITS>::pair_gap();
                xf[m] = __byte_perm(raw[lo >> 1], raw[hi >> 1], (lo & 1) ? 0x7632 : 0x5410);
            }
            unsigned char* dst = smem + (size_t)bid * 64;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                *reinterpret_cast<uint4*>(dst + (((i + c) & 3) << 4)) = make_uint4(xf[4 * i], xf[4 * i + 1], xf[4 * i + 2], xf[4 * i + 3]);
        }
    }
    __syncthreads();

    const bool has_x = g < S.nb;
    const unsigned xgroup = 4u * S.nb * 64u;                                  // bytes of x fragments per group
    const unsigned char* xbase = smem + ((size_t)(2 * pair_begin * 4 + t) * S.nb + g) * 64;
    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int cur_tile = tile_begin, cur_pair = 0;

    auto compute = [&](const Stage<BITS>& st) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            uint32_t xf[16];
            if (has_x) {
                const unsigned char* xb = xbase + (size_t)(2 * cur_pair + q) * xgroup;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 v = *reinterpret_cast<const uint4*>(xb + (((i + t) & 3) << 4));
                    xf[4 * i] = v.x; xf[4 * i + 1] = v.y; xf[4 * i + 2] = v.z; xf[4 * i + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) xf[i] = 0u;
            }
            // this group's scale and zero of both rows: half q of the half2 registers
            const __half2 s0h = *reinterpret_cast<const __half2*>(&st.s[0]), s1h = *reinterpret_cast<const __half2*>(&st.s[1]);
            const float cs0 = q ? __high2float(s0h) : __low2float(s0h), cs1 = q ? __high2float(s1h) : __low2float(s1h);
            uint32_t ka[Unpack<BITS>::kConsts], kb[Unpack<BITS>::kConsts];
            Unpack<BITS>::consts(__byte_perm(st.z[0], st.z[0], q ? 0x3232 : 0x1010), ka);
            Unpack<BITS>::consts(__byte_perm(st.z[1], st.z[1], q ? 0x3232 : 0x1010), kb);
            uint32_t ea[16], eb[16];
            Unpack<BITS>::run(st.w[q][0], ka, ea);
            Unpack<BITS>::run(st.w[q][1], kb, eb);
            // four independent accumulation chains of depth two (a dependent mma.sync issues ~110 cycles later)
            float d0[4], d1[4], d2[4], d3[4];
            mma16816(d0, ea[0], eb[0], ea[1], eb[1], xf[0], xf[1], zero4);
            mma16816(d1, ea[2], eb[2], ea[3], eb[3], xf[2], xf[3], zero4);
            mma16816(d2, ea[4], eb[4], ea[5], eb[5], xf[4], xf[5], zero4);
            mma16816(d3, ea[6], eb[6], ea[7], eb[7], xf[6], xf[7], zero4);
            mma16816(d0, ea[8], eb[8], ea[9], eb[9], xf[8], xf[9], d0);
            mma16816(d1, ea[10], eb[10], ea[11], eb[11], xf[10], xf[11], d1);
            mma16816(d2, ea[12], eb[12], ea[13], eb[13], xf[12], xf[13], d2);
            mma16816(d3, ea[14], eb[14], ea[15], eb[15], xf[14], xf[15], d3);
            // acc += s * sum((q - z) x): rows g (d[0], d[1]) and g+8 (d[2], d[3]), batch columns 2t, 2t+1
            acc[0] = fmaf(cs0, (d0[0] + d1[0]) + (d2[0] + d3[0]), acc[0]);
            acc[1] = fmaf(cs0, (d0[1] + d1[1]) + (d2[1] + d3[1]), acc[1]);
            acc[2] = fmaf(cs1, (d0[2] + d1[2]) + (d2[2] + d3[2]), acc[2]);
            acc[3] = fmaf(cs1, (d0[3] + d1[3]) + (d2[3] + d3[3]), acc[3]);
        }
        if (++cur_pair == npair) {
            // ---- the tile is complete in this warp: meet the other K-slices in shared memory
            float* myred = red + (size_t)(cur_tile & 1) * (kWarps * 32 * 4);
            *reinterpret_cast<float4*>(&myred[(warp * 32 + lane) * 4]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            __syncthreads();
            if (tid < 128) {
                const int r = tid >> 3, b = tid & 7;             // thread -> (row in tile, batch column)
                const int v = cur_tile * 16 + r;
                const int fl = (r & 7) * 4 + (b >> 1), fe = (r >> 3) * 2 + (b & 1);
                const int pl = ((r ^ 1) & 7) * 4 + (b >> 1);
                float mine = 0.f, partner = 0.f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) {
                    mine += myred[(w * 32 + fl) * 4 + fe];
                    partner += myred[(w * 32 + pl) * 4 + fe];
                }
                if (v < P.V && b < P.B) epilogue<__half>(P, b, v, mine, partner);
            }
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            cur_pair = 0;
            ++cur_tile;
        }
    };

    for (int s = 0; s < nsteps; s += 2) {
        compute(sa);
        if (s + 2 < nsteps) load(sa);
        if (s + 1 < nsteps) {
            compute(sb);
            if (s + 3 < nsteps) load(sb);
        }
    }
    peer_signal(P, peer_epoch);
}

template <int BITS>
int launch_t(const void* x, GemvParams P, bool pdl, cudaStream_t stream) {
    const int sms = sm_count_current();
    if (sms <= 0) return CB_ERR_CUDA;
    DirectParams S{};
    const int gpairs = P.groups / 2;
    const size_t xbytes = (size_t)P.B * P.K * 2;
    const size_t red_off = (xbytes + 127) & ~(size_t)127;
    const size_t smem = red_off + (size_t)2 * kWarps * 32 * 4 * sizeof(float);
    if (smem > kSmemCapOne) return -1;
    const int per_sm = smem <= kSmemCapTwo ? 2 : 1;
    const int tiles = (P.V + 15) / 16;
    const int ctas = std::max(1, std::min(tiles, per_sm * sms));
    P.split_k = 1;                       // K is split inside the CTA; no partial planes
    P.partial = nullptr; P.counters = nullptr;
    S.g = P;
    S.tile_q = tiles / ctas; S.tile_r = tiles % ctas;
    S.pair_q = gpairs / kWarps; S.pair_r = gpairs % kWarps;
    S.nb = P.B;
    S.off_red = (unsigned)red_off;

    static bool attr_done[64] = {};     // per device: the opt-in to large dynamic shared memory
    auto kern = gemv_direct_kernel<BITS>;
    int dev = 0;
    CB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        CB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemCapOne));
        // every decode kernel asks for the same shared-memory carve-out, so that consecutive launches of a stream
        // never make an SM drain to re-partition its L1 / shared memory
        CB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)ctas);
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

// Returns CB_OK after launching, a CB_ERR_* code on a CUDA error, or -1 when this problem is outside the
// kernel's domain (the caller then tries the next kernel).
int launch_gemv_direct(int bits, int dtype, const void* x, const GemvParams& P, bool pdl, cudaStream_t stream) {
    if (dtype != CB_F16 || P.group_size != 128 || P.K % 256 != 0 || P.groups < 2 * kWarps || P.B > kMaxBatchBlock || P.B < 1)
        return -1;
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0) return -1;
    const int nproj = P.mode == CB_MODE_QKV ? 3 : (P.mode == CB_MODE_GATEUP ? 2 : 1);
    for (int i = 0; i < nproj; ++i) {
        if (reinterpret_cast<uintptr_t>(P.p[i].w) % 16 != 0) return -1;
        if (reinterpret_cast<uintptr_t>(P.p[i].s) % 4 != 0 || reinterpret_cast<uintptr_t>(P.p[i].z) % 4 != 0) return -1;
    }
    if ((P.mode != CB_MODE_GEMV) && (P.V & 1)) return -1;
    switch (bits) {
        case 2: return launch_t<2>(x, P, pdl, stream);
        case 3: return launch_t<3>(x, P, pdl, stream);
        default: return launch_t<4>(x, P, pdl, stream);
    }
}

}  // namespace cb
