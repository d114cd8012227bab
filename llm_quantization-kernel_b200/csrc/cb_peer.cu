// Rank-to-rank barrier for column-parallel decode stacks (one process per GPU, peer-mapped memory).
//
// The decode kernels of a sharded stack store their output slice directly into every rank's gathered
// activation buffer (plain peer stores over NVLink, see GemvParams::peer_out).  What remains of the
// all-gather is to know when all slices have landed: this one-CTA kernel, launched right after the
// decode kernel on every rank, tells every peer "my launch number e is complete" and waits until every
// peer has said the same.  Flags are 32-bit counters in peer-mapped memory; the launch number is kept
// in device memory and advanced by the kernel itself, so a CUDA graph that contains the barrier can be
// replayed.  The wait is bounded (about a second); when it runs out a status word is set and all later
// barriers return at once, so a lost peer cannot hang the GPU.
#include "cb_common.cuh"

namespace cb {
namespace {

struct PeerBarrierParams {
    unsigned int* peer_flags[8];   // peer_flags[p] = base of rank p's flag array (world entries), peer-mapped
    unsigned int* my_flags;        // this rank's own flag array
    unsigned int* epoch;           // this rank's launch counter
    int* status;                   // 0 = fine, else 1 + the first peer that was not heard from in time
    int world, rank;
};

__global__ void peer_barrier_kernel(const PeerBarrierParams P) {
    // Launched as a programmatic dependent it is resident before the decode kernel ends, and lets the next
    // decode kernel in, which prefetches its weights until this barrier has completed.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int p = threadIdx.x;
    __shared__ unsigned int s_epoch;
    if (p == 0) s_epoch = *P.epoch + 1u;
    __syncthreads();
    const unsigned int e = s_epoch;
    if (p < P.world) {
        __threadfence_system();                                   // everything this GPU wrote before is visible first
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(P.peer_flags[p] + P.rank), "r"(e) : "memory");
        if (*reinterpret_cast<volatile int*>(P.status) == 0) {
            const long long t0 = clock64();
            unsigned int seen = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(P.my_flags + p) : "memory");
                if ((int)(seen - e) >= 0) break;
                if (clock64() - t0 > 2000000000ll) { atomicCAS(P.status, 0, 1 + p); break; }
            }
        }
    }
    __syncthreads();
    if (p == 0) *P.epoch = e;
}

// The two halves of the in-kernel hand-shake as kernels of their own, for decode kernels that do not carry it.
__global__ void peer_wait_kernel(const GemvParams P) { peer_wait(P); }
__global__ void peer_signal_kernel(const GemvParams P) {
    peer_signal(P, *reinterpret_cast<volatile unsigned int*>(P.sync.epoch));
}

}  // namespace

int launch_peer_wait(const GemvParams& P, cudaStream_t stream) {
    peer_wait_kernel<<<1, 32, 0, stream>>>(P);
    CB_CUDA_TRY(cudaGetLastError());
    return CB_OK;
}

int launch_peer_signal(const GemvParams& P, cudaStream_t stream) {
    peer_signal_kernel<<<1, 32, 0, stream>>>(P);
    CB_CUDA_TRY(cudaGetLastError());
    return CB_OK;
}

}  // namespace cb

extern "C" int cb_peer_barrier(void* const* peer_flags, void* my_flags, void* epoch, int* status, int world, int rank,
                               void* stream) {
    using namespace cb;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || !peer_flags || !my_flags || !epoch || !status) {
        set_error("peer_barrier: bad arguments");
        return CB_ERR_INVALID;
    }
    PeerBarrierParams P{};
    for (int i = 0; i < world; ++i) {
        if (peer_flags[i] == nullptr) { set_error("peer_barrier: peer %d has no flag array", i); return CB_ERR_INVALID; }
        P.peer_flags[i] = reinterpret_cast<unsigned int*>(peer_flags[i]);
    }
    P.my_flags = reinterpret_cast<unsigned int*>(my_flags);
    P.epoch = reinterpret_cast<unsigned int*>(epoch);
    P.status = status;
    P.world = world; P.rank = rank;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1); cfg.blockDim = dim3(32); cfg.dynamicSmemBytes = 0;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 1 : 0;
    CB_CUDA_TRY(cudaLaunchKernelEx(&cfg, peer_barrier_kernel, P));
    return CB_OK;
}

// Bounded wait until every peer has completed as many hand-shake launches as this rank: what a consumer other
// than a decode launch (a copy to the host, another library's kernel) needs before it reads a gathered buffer.
extern "C" int cb_peer_wait(const cb_scatter* sc, void* stream) {
    using namespace cb;
    if (sc == nullptr || !sc->sync || sc->world < 1 || sc->world > 8 || !sc->my_flags || !sc->epoch || !sc->status) {
        set_error("peer_wait: needs a scatter description with the hand-shake words");
        return CB_ERR_INVALID;
    }
    GemvParams P{};
    P.n_peers = sc->world;
    P.sync.my_flags = reinterpret_cast<unsigned int*>(sc->my_flags);
    P.sync.epoch = reinterpret_cast<unsigned int*>(sc->epoch);
    P.sync.status = sc->status;
    P.sync.on = 1;
    return launch_peer_wait(P, reinterpret_cast<cudaStream_t>(stream));
}
