// Shared device/host definitions of the packed W2/W3/W4 linear kernels (sm_100a).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <type_traits>

#include "../../include/crispybits_b200.h"

namespace cb {

constexpr int kTileN = 16;        // virtual output rows per decode work tile (what cb_tile_n() reports)
constexpr int kMaxBatchBlock = 8; // batch rows that share one pass over the weights

// ---- element conversion -------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Activation codes follow the reference (Crispybits/Kernel/csrc/common.cuh:15-19): relu, or
// silu computed as v / (1 + exp(-v)).
__device__ __forceinline__ float activate(float v, int act) {
    if (act == CB_ACT_RELU) return fmaxf(v, 0.f);
    if (act == CB_ACT_SILU) return v / (1.0f + __expf(-v));
    return v;
}

// ---- decode problem description -----------------------------------------------------------
struct Proj {
    const uint32_t* w;  // packed words, row-major
    const void* s;      // scales [n, groups]
    const void* z;      // zeros  [n, groups]
    const void* b;      // bias [n] or nullptr
    void* out;          // [B, n]
    int n;
};

// Rank-to-rank hand-shake of a column-parallel stack, carried by the decode kernel itself.
// on == 1: before it reads its activations a launch waits until every peer has completed as many launches as this
//          rank, and its last CTA to finish tells every peer that one more launch is complete.
// on == 2: launches are numbered within a step (seq = 0, 1, ...).  Launch seq > 0 waits, before it reads its
//          activations, until every rank (this one included) has published seq completed launches of the running step,
//          i.e. flag >= *epoch + seq, where *epoch counts the launches of all finished steps and does not change while
//          a step runs.  It publishes nothing itself: a one-CTA kernel after it does, once the launch has completed
//          (cb_peer_publish), so the decode kernel neither fences nor counts its CTAs, and it does not wait for the
//          completion event of its predecessor on this GPU either: the flags are the dependency.
struct PeerSync {
    unsigned int* peer_flags[8];  // peer_flags[p] = rank p's flag array (one uint32 per rank), peer-mapped
    unsigned int* my_flags;       // this rank's own flag array: my_flags[p] = launches rank p has completed
    unsigned int* epoch;          // on == 1: launches this rank has completed; on == 2: launches of all finished steps
    int* done;                    // on == 1: CTAs of the running launch that are finished; zero between launches
    int* status;                  // 0, or 1 + the first peer that was not heard from in time
    int rank, on;
    unsigned int seq;             // on == 2: number of this launch within its step
    unsigned int need;            // on == 2: launches of the step that every rank must have published before this one
                                  //          reads its activations (seq for a launch that consumes its predecessor's
                                  //          output; less for one that does not)
};

struct GemvParams {
    Proj p[3];
    int mode;                 // CB_MODE_*
    int V, B, K;              // virtual rows, batch, in_features
    int nchunks, wpr, groups, group_size;
    int split_k, ntiles, nbblocks, units;
    int act;
    float* partial;           // [split_k, B, V] fp32, only when split_k > 1
    int* counters;            // [nbblocks * ntiles] arrival counters, zero between calls
    const float* rope_cos;    // [B, head_dim] fp32 or nullptr
    const float* rope_sin;
    int head_dim, perm_hd;
    // Optional peer scatter (column-parallel stacks): output rows r < n_gather of GEMV / gate-up mode are
    // stored into every rank's gathered activation buffer at [b * peer_ld + peer_col + r] instead of `out`.
    void* peer_out[8];
    int n_peers, n_gather, peer_ld, peer_col;
    PeerSync sync;
};

constexpr long long kPeerWaitCycles = 2000000000ll;   // about a second

// All threads of the CTA call this before the first read of the activations.  Threads 0..world-1 each watch one
// peer's counter; the wait is bounded, and once one wait has run out (status != 0) later ones return at once.
// Returns (to thread 0) the number of launches this rank had completed, which peer_signal advances.
__device__ __forceinline__ unsigned int peer_wait(const GemvParams& P) {
    if (!P.sync.on) return 0u;
    if (P.sync.on == 2 && P.sync.need == 0u) return 0u;     // nothing of this step has to be complete yet
    const int p = threadIdx.x;
    unsigned int e = 0u;
    if (p < P.n_peers) {
        e = *reinterpret_cast<volatile unsigned int*>(P.sync.epoch) + (P.sync.on == 2 ? P.sync.need : 0u);
        unsigned int seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(P.sync.my_flags + p) : "memory");
        if ((int)(seen - e) < 0 && *reinterpret_cast<volatile int*>(P.sync.status) == 0) {
            const long long t0 = clock64();
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(P.sync.my_flags + p) : "memory");
                if ((int)(seen - e) >= 0) break;
                if (clock64() - t0 > kPeerWaitCycles) { atomicCAS(P.sync.status, 0, 1 + p); break; }
                __nanosleep(64);
            }
        }
    }
    __syncthreads();
    return e;
}

// All threads of every CTA call this once, after their last store; `e` is what peer_wait returned.  The CTA
// barrier puts every thread's stores before thread 0's system-scope fence, the arrival counter chains the CTAs,
// and the last CTA to arrive fences again before it advances this rank's launch count and publishes it: all
// output stores of the grid (peer stores included) are visible to a peer that sees the new count.
__device__ __forceinline__ void peer_signal(const GemvParams& P, unsigned int e) {
    if (P.sync.on != 1) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(P.sync.done, 1) == (int)gridDim.x - 1) {
            *P.sync.done = 0;
            const unsigned int e1 = e + 1u;
            *reinterpret_cast<volatile unsigned int*>(P.sync.epoch) = e1;
            __threadfence_system();
            for (int q = 0; q < P.n_peers; ++q)
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(P.sync.peer_flags[q] + P.sync.rank), "r"(e1) : "memory");
        }
    }
}

// Virtual row -> (projection, row inside it).  GEMV: identity; QKV: three consecutive ranges;
// gate/up: even virtual rows are gate rows, odd ones the up row of the same index, so that the two
// operands of silu(gate)*up are neighbours (Crispybits/Kernel/csrc/packed_gemv.cu:33-42).
__device__ __forceinline__ void map_row(const GemvParams& P, int v, int& proj, int& r) {
    if (P.mode == CB_MODE_GATEUP) { proj = v & 1; r = v >> 1; }
    else if (P.mode == CB_MODE_QKV) {
        const int n0 = P.p[0].n, n1 = P.p[1].n;
        if (v < n0) { proj = 0; r = v; }
        else if (v < n0 + n1) { proj = 1; r = v - n0; }
        else { proj = 2; r = v - n0 - n1; }
    } else { proj = 0; r = v; }
}

// Stored (pair-interleaved) row of a head -> original row: even stored positions hold the first
// half of the head, odd ones the second half (Crispybits/Kernel/csrc/common.cuh:66-70).
__device__ __forceinline__ int unpermute_row(int r, int hd) {
    if (hd <= 0) return r;
    const int head = r / hd, p = r - head * hd;
    return head * hd + ((p & 1) ? (p >> 1) + hd / 2 : (p >> 1));
}

template <typename T>
__device__ __forceinline__ float bias_at(const void* b, int r) {
    return b ? to_f32(reinterpret_cast<const T*>(b)[r]) : 0.f;
}

// Final step for one (batch row, virtual row): `mine` is the finished dot product of virtual row v,
// `partner` that of v^1 (needed by gate/up and by RoPE).  Semantics follow
// Crispybits/Kernel/csrc/packed_gemv.cu:54-81.
template <typename T>
__device__ __forceinline__ void epilogue(const GemvParams& P, int b, int v, float mine, float partner) {
    int proj, r;
    map_row(P, v, proj, r);
    if (P.mode == CB_MODE_GEMV || P.mode == CB_MODE_GATEUP) {
        float y;
        if (P.mode == CB_MODE_GEMV) {
            y = activate(mine + bias_at<T>(P.p[0].b, r), P.act);
        } else {
            if (proj != 0) return;  // the gate row writes silu(gate) * up
            y = activate(mine, CB_ACT_SILU) * partner;
        }
        const T yt = from_f32<T>(y);
        if (r < P.n_gather) {
            // the all-gather is these stores: the slice goes straight into every rank's buffer over NVLink
            const size_t at = (size_t)b * P.peer_ld + P.peer_col + r;
            for (int q = 0; q < P.n_peers; ++q) reinterpret_cast<T*>(P.peer_out[q])[at] = yt;
        } else {
            reinterpret_cast<T*>(P.p[0].out)[(size_t)b * P.p[0].n + r] = yt;
        }
    } else {
        const Proj& pr = P.p[proj];
        float y = mine + bias_at<T>(pr.b, r);
        const int hd = proj < 2 ? P.perm_hd : 0;
        const int orig = unpermute_row(r, hd);
        if (P.rope_cos != nullptr && proj < 2) {
            const float yp = partner + bias_at<T>(pr.b, r ^ 1);
            const int d = orig % P.head_dim;
            const float c = P.rope_cos[(size_t)b * P.head_dim + d];
            const float s = P.rope_sin[(size_t)b * P.head_dim + d];
            y = (d < P.head_dim / 2) ? (y * c - yp * s) : (y * c + yp * s);
        }
        reinterpret_cast<T*>(pr.out)[(size_t)b * pr.n + orig] = from_f32<T>(y);
    }
}

// ---- host side ------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int sm_count_current();
bool pdl_enabled();   // programmatic dependent launches are in use (on unless switched off)

#define CB_CUDA_TRY(expr)                                                                  \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess) {                                                           \
            cb::set_error("%s failed: %s", #expr, cudaGetErrorString(_e));                 \
            return CB_ERR_CUDA;                                                            \
        }                                                                                  \
    } while (0)

}  // namespace cb
