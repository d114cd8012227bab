// CUDA-core prefill GEMM  out[M,N] = act(x[M,K] * Wdq^T + bias)  with fp32 arithmetic.
//
// It serves use_tensor_cores = 0 (the reference's scalar path,
// Crispybits/Kernel/csrc/packed_gemm.cu:118-156), every fp32 call, and shapes the tcgen05 kernel does
// not take.  `round_w` reproduces the tensor-core numerics (dequantised weight rounded to the
// storage type, packed_gemm.cu:56,60) when this kernel stands in for that path.
//
// Tiling: a CTA of 256 threads owns a 64x64 output tile and walks K in 32-code chunks; the x tile
// and the dequantised weight tile sit in shared memory k-major, each thread accumulates a 4x4
// micro-tile.  Bit-width is a run-time argument here: this path is not the fast one.
#include "cb_bitpack.cuh"
#include "cb_common.cuh"

namespace cb {
namespace {
constexpr int kBM = 64, kBN = 64, kBK = 32, kPitch = 68, kThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads)
gemm_simt_kernel(const T* __restrict__ x, const uint32_t* __restrict__ packed, const T* __restrict__ scales,
                 const T* __restrict__ zeros, const T* __restrict__ bias, T* __restrict__ out,
                 int M, int N, int K, int bits, int wpr, int groups, int group_size, int act, int round_w) {
    __shared__ float xs[kBK][kPitch];
    __shared__ float ws[kBK][kPitch];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * kBN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const int nchunks = (K + 31) / 32;
    for (int c = 0; c < nchunks; ++c) {
        // x tile: 64 rows x 32 k, thread t loads k = t & 31 for rows (t >> 5) + 8*i
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int mm = (tid >> 5) + 8 * i, kk = tid & 31;
            const int gm = m0 + mm, gk = c * 32 + kk;
            xs[kk][mm] = (gm < M && gk < K) ? to_f32(x[(size_t)gm * K + gk]) : 0.f;
        }
        // weight tile: thread t dequantises 8 codes of row n0 + (t >> 2)
        {
            const int nn = tid >> 2, q0 = (tid & 3) * 8, gn = n0 + nn;
            float s = 0.f, z = 0.f;
            const uint32_t* row = nullptr;
            if (gn < N) {
                const int g = (c * 32) / group_size;
                s = to_f32(scales[(size_t)gn * groups + g]);
                z = to_f32(zeros[(size_t)gn * groups + g]);
                row = packed + (size_t)gn * wpr;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float w = 0.f;
                if (row != nullptr) {
                    w = ((float)row_code(row, c * 32 + q0 + j, bits) - z) * s;
                    if (round_w) w = to_f32(from_f32<T>(w));
                }
                ws[q0 + j][nn] = w;
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kBK; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&ws[kk][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) {
                float v = acc[i][j];
                if (bias) v += to_f32(bias[gn]);
                out[(size_t)gm * N + gn] = from_f32<T>(activate(v, act));
            }
        }
    }
}

template <typename T>
int launch_t(const void* x, int64_t M, const cb_weight* w, void* out, int64_t K, int bits, int64_t gs, int act,
             int round_w, cudaStream_t stream) {
    const int N = (int)w->n, wpr = (int)((K + 31) / 32) * bits, groups = (int)((K + gs - 1) / gs);
    dim3 grid((N + kBN - 1) / kBN, (unsigned)((M + kBM - 1) / kBM));
    gemm_simt_kernel<T><<<grid, kThreads, 0, stream>>>(
        reinterpret_cast<const T*>(x), reinterpret_cast<const uint32_t*>(w->packed),
        reinterpret_cast<const T*>(w->scales), reinterpret_cast<const T*>(w->zeros),
        reinterpret_cast<const T*>(w->bias), reinterpret_cast<T*>(out), (int)M, N, (int)K, bits, wpr, groups,
        (int)gs, act, round_w);
    CB_CUDA_TRY(cudaGetLastError());
    return CB_OK;
}
}  // namespace

int launch_gemm_simt(int dtype, const void* x, int64_t M, const cb_weight* w, void* out, int64_t K, int bits,
                     int64_t gs, int act, int round_w, cudaStream_t stream) {
    if (dtype == CB_F16) return launch_t<__half>(x, M, w, out, K, bits, gs, act, round_w, stream);
    if (dtype == CB_BF16) return launch_t<__nv_bfloat16>(x, M, w, out, K, bits, gs, act, round_w, stream);
    return launch_t<float>(x, M, w, out, K, bits, gs, act, 0, stream);
}

}  // namespace cb
