/*
 * CPU oracle for the packed W2/W3/W4 linear path, plain C.  TEST INFRASTRUCTURE ONLY.
 *
 * A restatement of the CrispyBits reference's algorithm for this path, used (a) to check the
 * CUDA kernels bit-for-bit on integer work and within tolerance on floating work, and (b) as
 * the multi-threaded CPU baseline that the benchmark times beside the GPU.  The shipped
 * library never links or calls it.
 *
 * Parity status: PINNED through tests/golden (outputs of the reference's own reference.py /
 * emulator.py) and the known-answer vectors of the reference's tests/test_packing.py.
 *
 * Citations are Crispybits/Kernel/<file>:<lines> of the reference.
 *
 * Floating inputs arrive as float32 values already representable in the storage dtype; the
 * caller rounds outputs to the storage dtype (the numpy wrapper does).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int cbo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Threads the parallel loops below use from now on (a launcher such as torchrun exports OMP_NUM_THREADS=1, which
 * would otherwise make the timed CPU baseline single-threaded). */
void cbo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Code k of a row: bits [k*bits, k*bits+bits) of the row's little-endian stream of 32-bit words
 * (crispybits_kernels/reference.py:58-67; csrc/bitpack.cuh:10-18). */
static inline uint32_t code_at(const uint32_t* row, int64_t k, int bits) {
    const int64_t pos = k * bits;
    const int64_t wi = pos >> 5;
    const int off = (int)(pos & 31);
    uint64_t v = row[wi] >> off;
    if (off + bits > 32) v |= (uint64_t)row[wi + 1] << (32 - off);
    return (uint32_t)(v & ((1u << bits) - 1u));
}

/* packed int32 [n, wpr] -> codes int32 [n, k] */
void cbo_unpack_codes(const int32_t* packed, int64_t n, int64_t wpr, int bits, int64_t k, int32_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
        const uint32_t* row = (const uint32_t*)packed + r * wpr;
        for (int64_t j = 0; j < k; ++j) out[r * k + j] = (int32_t)code_at(row, j, bits);
    }
}

/* codes int32 [n, k] -> packed int32 [n, ceil(k/32)*bits], rows zero-padded to whole 32-code
 * chunks (crispybits_kernels/reference.py:37-55). */
void cbo_pack_codes(const int32_t* q, int64_t n, int64_t k, int bits, int32_t* packed) {
    const int64_t wpr = ((k + 31) / 32) * bits;
    const uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
        uint32_t* row = (uint32_t*)packed + r * wpr;
        memset(row, 0, (size_t)wpr * 4);
        for (int64_t j = 0; j < k; ++j) {
            const uint64_t v = (uint64_t)((uint32_t)q[r * k + j] & mask);
            const int64_t pos = j * bits, wi = pos >> 5;
            const int off = (int)(pos & 31);
            row[wi] |= (uint32_t)(v << off);
            if (off + bits > 32) row[wi + 1] |= (uint32_t)(v >> (32 - off));
        }
    }
}

/* Group-wise asymmetric affine quantizer, float32 arithmetic, round-half-even
 * (crispybits_kernels/reference.py:10-27).  The ragged last group repeats the last column.
 * w [n,k] -> q int32 [n,k], scale/zero float32 [n, ceil(k/gs)]. */
void cbo_quantize_affine(const float* w, int64_t n, int64_t k, int bits, int64_t gs,
                         int32_t* q, float* scale, float* zero) {
    const int64_t G = (k + gs - 1) / gs;
    const float qmax = (float)((1 << bits) - 1);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
        const float* wr = w + r * k;
        for (int64_t g = 0; g < G; ++g) {
            const int64_t k0 = g * gs, k1 = (k0 + gs < k) ? k0 + gs : k;
            float mn = wr[k0], mx = wr[k0];
            for (int64_t j = k0; j < k1; ++j) { mn = fminf(mn, wr[j]); mx = fmaxf(mx, wr[j]); }
            float s = (mx - mn) / qmax;
            if (s < 1e-8f) s = 1e-8f;
            float z = rintf(-mn / s);
            z = fminf(fmaxf(z, 0.f), qmax);
            scale[r * G + g] = s;
            zero[r * G + g] = z;
            for (int64_t j = k0; j < k1; ++j) {
                float c = rintf(wr[j] / s) + z;
                c = fminf(fmaxf(c, 0.f), qmax);
                q[r * k + j] = (int32_t)c;
            }
        }
    }
}

/* Decode partial sums with the kernel's chunk algebra (csrc/packed_gemv.cu:113-137;
 * crispybits_kernels/emulator.py:48-67):
 *   part[s][b][v] = sum over chunks c in split s of  scale[v,g(c)] * (sum_j x_j q_j - zero[v,g(c)] * sum_j x_j)
 * with g(c) = 32c / gs, split s covering chunks [C*s/P, C*(s+1)/P), float32 throughout.
 * x [B,K] float32, packed [V, C*bits], scales/zeros float32 [V, G].  part [P,B,V]. */
void cbo_gemv_partials(const float* x, int64_t B, const int32_t* packed, const float* scales,
                       const float* zeros, int64_t V, int64_t K, int bits, int64_t gs, int64_t P,
                       float* part) {
    const int64_t C = (K + 31) / 32, wpr = C * bits, G = (K + gs - 1) / gs;
    if (P < 1) P = 1;
    if (P > C) P = C;
    /* x padded to whole chunks, and per-chunk sums, shared by all rows */
    float* xp = (float*)calloc((size_t)(B * C * 32), sizeof(float));
    float* xs = (float*)calloc((size_t)(B * C), sizeof(float));
    for (int64_t b = 0; b < B; ++b) {
        memcpy(xp + b * C * 32, x + b * K, (size_t)K * sizeof(float));
        for (int64_t c = 0; c < C; ++c) {
            float s = 0.f;
            for (int j = 0; j < 32; ++j) s += xp[(b * C + c) * 32 + j];
            xs[b * C + c] = s;
        }
    }
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < V; ++v) {
        const uint32_t* row = (const uint32_t*)packed + v * wpr;
        float qf[32];
        for (int64_t s = 0; s < P; ++s) {
            const int64_t c0 = (C * s) / P, c1 = (C * (s + 1)) / P;
            for (int64_t b = 0; b < B; ++b) part[(s * B + b) * V + v] = 0.f;
            for (int64_t c = c0; c < c1; ++c) {
                for (int j = 0; j < 32; ++j) qf[j] = (float)code_at(row, c * 32 + j, bits);
                const int64_t g = (c * 32) / gs;
                const float sc = scales[v * G + g], ze = zeros[v * G + g];
                for (int64_t b = 0; b < B; ++b) {
                    const float* xb = xp + (b * C + c) * 32;
                    float d = 0.f;
                    for (int j = 0; j < 32; ++j) d = fmaf(xb[j], qf[j], d);
                    part[(s * B + b) * V + v] += sc * (d - ze * xs[b * C + c]);
                }
            }
        }
    }
    free(xp);
    free(xs);
}

/* y[b][v] = sum_s part[s][b][v]  (the Split-K reducer, csrc/packed_gemv.cu:166-180) */
void cbo_gemv(const float* x, int64_t B, const int32_t* packed, const float* scales, const float* zeros,
              int64_t V, int64_t K, int bits, int64_t gs, int64_t P, float* y) {
    const int64_t C = (K + 31) / 32;
    if (P < 1) P = 1;
    if (P > C) P = C;
    float* part = (float*)malloc((size_t)(P * B * V) * sizeof(float));
    cbo_gemv_partials(x, B, packed, scales, zeros, V, K, bits, gs, P, part);
    for (int64_t i = 0; i < B * V; ++i) {
        float a = 0.f;
        for (int64_t s = 0; s < P; ++s) a += part[s * B * V + i];
        y[i] = a;
    }
    free(part);
}

/* Dequantised weight (q - zero) * scale in float32 (crispybits_kernels/reference.py:30-34, 79-82);
 * wdq [N,K]. */
void cbo_dequantize(const int32_t* packed, const float* scales, const float* zeros, int64_t N, int64_t K,
                    int bits, int64_t gs, float* wdq) {
    const int64_t C = (K + 31) / 32, wpr = C * bits, G = (K + gs - 1) / gs;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
        const uint32_t* row = (const uint32_t*)packed + r * wpr;
        for (int64_t j = 0; j < K; ++j) {
            const int64_t g = j / gs;
            wdq[r * K + j] = ((float)code_at(row, j, bits) - zeros[r * G + g]) * scales[r * G + g];
        }
    }
}

/* out[M,N] = x[M,K] * wdq[N,K]^T, float32 accumulate: the matmul half of the prefill path
 * (crispybits_kernels/emulator.py:143; csrc/packed_gemm.cu:68-80).  wdq is the dequantised
 * weight, rounded to the storage dtype by the caller when the tensor-core path is emulated. */
void cbo_matmul_nt(const float* x, const float* wdq, int64_t M, int64_t N, int64_t K, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const float* wr = wdq + n * K;
        for (int64_t m = 0; m < M; ++m) {
            const float* xr = x + m * K;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            int64_t j = 0;
            for (; j + 8 <= K; j += 8)
                for (int t = 0; t < 8; ++t) acc[t] = fmaf(xr[j + t], wr[j + t], acc[t]);
            float a = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
            for (; j < K; ++j) a = fmaf(xr[j], wr[j], a);
            out[m * N + n] = a;
        }
    }
}
