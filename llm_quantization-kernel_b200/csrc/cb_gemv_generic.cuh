// Shape-generic decode GEMV (any K, any group size that is a multiple of 32, fp32/fp16/bf16,
// all three modes).  It is the path for everything the streamlined fp16 kernel does not cover.
//
// Work decomposition.  A work unit is (batch block of up to 8 rows) x (tile of 16 virtual output
// rows) x (one of split_k chunk ranges).  A CTA of 8 warps walks units blockIdx.x, +gridDim.x, ...;
// inside a unit each warp owns two neighbouring virtual rows (v, v^1 -- the pair that gate/up and
// RoPE combine), lanes stride over 32-code chunks, and every weight word is read once for all
// batch rows of the block.  Per chunk the arithmetic is the reference's
//     acc += scale * (sum_j x_j q_j - zero * sum_j x_j)         (Crispybits/Kernel/csrc/packed_gemv.cu:131-135)
// in fp32.  With split_k > 1 the partial sums go to scratch and the LAST CTA to arrive at a tile
// (per-tile counter, reset to zero by that CTA) adds them in split order and runs the epilogue, so
// there is no second launch and the result does not depend on arrival order.
#pragma once
#include <algorithm>

#include "cb_bitpack.cuh"
#include "cb_common.cuh"

namespace cb {

constexpr int kGenericThreads = 256;
static_assert(kGenericThreads / 32 * 2 == kTileN, "8 warps x 2 rows = one tile");

// 32 consecutive activations starting at k0 as fp32, zero beyond K.  `vec` says rows of x start
// 16-byte aligned, so whole chunks can use 128-bit loads.  x is read through L2 (ld.global.cg / volatile), never
// through the non-coherent path: in a column-parallel stack peers store it while this grid may already be resident.
template <typename T>
__device__ __forceinline__ void load_x32(const T* xb, int k0, int K, bool vec, float (&xv)[32]) {
    if (vec && k0 + 32 <= K) {
        const uint4* p = reinterpret_cast<const uint4*>(xb + k0);
        if constexpr (std::is_same<T, float>::value) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 v = __ldcg(p + i);
                xv[4 * i + 0] = __uint_as_float(v.x); xv[4 * i + 1] = __uint_as_float(v.y);
                xv[4 * i + 2] = __uint_as_float(v.z); xv[4 * i + 3] = __uint_as_float(v.w);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = __ldcg(p + i);
                const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    if constexpr (std::is_same<T, __half>::value) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[h]));
                        xv[8 * i + 2 * h] = f.x; xv[8 * i + 2 * h + 1] = f.y;
                    } else {
                        xv[8 * i + 2 * h] = __uint_as_float(u[h] << 16);
                        xv[8 * i + 2 * h + 1] = __uint_as_float(u[h] & 0xFFFF0000u);
                    }
                }
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int k = k0 + j;
            xv[j] = (k < K) ? to_f32(*const_cast<const volatile T*>(xb + k)) : 0.f;
        }
    }
}

template <typename T, int BITS, int NB>
__global__ void __launch_bounds__(kGenericThreads)
gemv_generic_kernel(const T* x, const GemvParams P, const int xvec) {
    __shared__ int s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    for (int u = blockIdx.x; u < P.units; u += gridDim.x) {
        const int split = u % P.split_k;
        const int tb = u / P.split_k;
        const int tile = tb % P.ntiles, bb = tb / P.ntiles;
        const int c0 = (int)(((long long)P.nchunks * split) / P.split_k);
        const int c1 = (int)(((long long)P.nchunks * (split + 1)) / P.split_k);
        const int b0 = bb * kMaxBatchBlock;
        const int v0 = tile * kTileN + warp * 2;

        const uint32_t* wrow[2] = {nullptr, nullptr};
        const T* srow[2] = {nullptr, nullptr};
        const T* zrow[2] = {nullptr, nullptr};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (v0 + r < P.V) {
                int proj, lr;
                map_row(P, v0 + r, proj, lr);
                wrow[r] = P.p[proj].w + (size_t)lr * P.wpr;
                srow[r] = reinterpret_cast<const T*>(P.p[proj].s) + (size_t)lr * P.groups;
                zrow[r] = reinterpret_cast<const T*>(P.p[proj].z) + (size_t)lr * P.groups;
            }
        }

        float acc[2][NB];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int i = 0; i < NB; ++i) acc[r][i] = 0.f;

        for (int c = c0 + lane; c < c1; c += 32) {
            float qf[2][32], sc[2], ze[2];
            const int g = (c * 32) / P.group_size;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                if (wrow[r] != nullptr) {
                    uint32_t w[BITS];
                    load_chunk<BITS>(wrow[r] + (size_t)c * BITS, w);
#pragma unroll
                    for (int j = 0; j < 32; ++j) qf[r][j] = small_uint_to_float(chunk_code<BITS>(w, j));
                    sc[r] = to_f32(srow[r][g]);
                    ze[r] = to_f32(zrow[r][g]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) qf[r][j] = 0.f;
                    sc[r] = 0.f; ze[r] = 0.f;
                }
            }
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int b = b0 + i;
                if (b < P.B) {
                    float xv[32];
                    load_x32<T>(x + (size_t)b * P.K, c * 32, P.K, xvec != 0, xv);
                    float xs = 0.f, d0 = 0.f, d1 = 0.f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        xs += xv[j];
                        d0 = fmaf(xv[j], qf[0][j], d0);
                        d1 = fmaf(xv[j], qf[1][j], d1);
                    }
                    acc[0][i] = fmaf(sc[0], d0 - ze[0] * xs, acc[0][i]);
                    acc[1][i] = fmaf(sc[1], d1 - ze[1] * xs, acc[1][i]);
                }
            }
        }

#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int i = 0; i < NB; ++i)
#pragma unroll
                for (int off = 16; off > 0; off >>= 1)
                    acc[r][i] += __shfl_xor_sync(0xffffffffu, acc[r][i], off);

        // lane L finishes (row v0 + (L & 1), batch b0 + (L >> 1))
        float mine = 0.f, partner = 0.f;
#pragma unroll
        for (int i = 0; i < NB; ++i)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                if (lane == 2 * i + r) { mine = acc[r][i]; partner = acc[r ^ 1][i]; }
            }
        const int v = v0 + (lane & 1), b = b0 + (lane >> 1);
        const bool active = lane < 2 * NB && v < P.V && b < P.B;

        if (P.split_k == 1) {
            if (active) epilogue<T>(P, b, v, mine, partner);
        } else {
            if (active) P.partial[((size_t)split * P.B + b) * P.V + v] = mine;
            __threadfence();
            __syncthreads();
            int* counter = P.counters + (bb * P.ntiles + tile);
            if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1) == P.split_k - 1) ? 1 : 0;
            __syncthreads();
            if (s_last) {
                __threadfence();
                for (int e = threadIdx.x; e < kTileN * NB; e += kGenericThreads) {
                    const int rv = tile * kTileN + (e % kTileN), rb = b0 + e / kTileN;
                    if (rv < P.V && rb < P.B) {
                        float m = 0.f, pt = 0.f;
                        const bool has_partner = (rv ^ 1) < P.V;
                        for (int s = 0; s < P.split_k; ++s) {
                            const float* ps = P.partial + ((size_t)s * P.B + rb) * P.V;
                            m += __ldcg(ps + rv);
                            if (has_partner) pt += __ldcg(ps + (rv ^ 1));
                        }
                        epilogue<T>(P, rb, rv, m, pt);
                    }
                }
                if (threadIdx.x == 0) *counter = 0;   // leave the scratch counters zero for the next call
            }
            __syncthreads();
        }
    }
}

template <typename T, int BITS>
int launch_gemv_generic_t(const void* x, const GemvParams& P, int64_t rho, cudaStream_t stream) {
    const int sms = sm_count_current();
    if (sms <= 0) return CB_ERR_CUDA;
    const int64_t want = rho <= 0 ? (int64_t)P.units : std::min<int64_t>(P.units, rho * (int64_t)sms);
    const int grid = (int)std::max<int64_t>(1, want);
    const int nb = std::min(P.B, kMaxBatchBlock);
    const int xvec = ((reinterpret_cast<uintptr_t>(x) % 16) == 0 && ((size_t)P.K * sizeof(T)) % 16 == 0) ? 1 : 0;
    const T* xp = reinterpret_cast<const T*>(x);
    if (nb >= 5)      gemv_generic_kernel<T, BITS, 8><<<grid, kGenericThreads, 0, stream>>>(xp, P, xvec);
    else if (nb >= 3) gemv_generic_kernel<T, BITS, 4><<<grid, kGenericThreads, 0, stream>>>(xp, P, xvec);
    else if (nb == 2) gemv_generic_kernel<T, BITS, 2><<<grid, kGenericThreads, 0, stream>>>(xp, P, xvec);
    else              gemv_generic_kernel<T, BITS, 1><<<grid, kGenericThreads, 0, stream>>>(xp, P, xvec);
    CB_CUDA_TRY(cudaGetLastError());
    return CB_OK;
}

template <int BITS>
int launch_gemv_generic(int dtype, const void* x, const GemvParams& P, int64_t rho, cudaStream_t stream) {
    if (dtype == CB_F16) return launch_gemv_generic_t<__half, BITS>(x, P, rho, stream);
    if (dtype == CB_BF16) return launch_gemv_generic_t<__nv_bfloat16, BITS>(x, P, rho, stream);
    return launch_gemv_generic_t<float, BITS>(x, P, rho, stream);
}

template <int BITS>
int occupancy_gemv_generic() {
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, gemv_generic_kernel<__half, BITS, 1>,
                                                      kGenericThreads, 0) != cudaSuccess)
        return -1;
    return blocks;
}

// one translation unit per bit-width (cb_gemv_generic_w{2,3,4}.cu) provides these
int launch_gemv_generic_w2(int dtype, const void* x, const GemvParams& P, int64_t rho, cudaStream_t stream);
int launch_gemv_generic_w3(int dtype, const void* x, const GemvParams& P, int64_t rho, cudaStream_t stream);
int launch_gemv_generic_w4(int dtype, const void* x, const GemvParams& P, int64_t rho, cudaStream_t stream);
int occupancy_gemv_generic_w2();
int occupancy_gemv_generic_w3();
int occupancy_gemv_generic_w4();

}  // namespace cb
