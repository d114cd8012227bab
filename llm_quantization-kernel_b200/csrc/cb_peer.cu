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

// Numbered hand-shake (PeerSync::on == 2).  After decode launch `seq` of a step this kernel tells every rank, this one
// included, that the launch is complete: it is resident before the decode launch ends (programmatic dependent), its
// griddepcontrol.wait returns when that launch has completed and its stores -- the peer stores too -- are visible,
// and a release store at system scope then carries the count epoch + seq + 1 to every rank's flag array.  It lets its
// own successor, the next decode launch, start at once.
__global__ void peer_publish_kernel(const PeerBarrierParams P, const unsigned int seq) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int p = threadIdx.x;
    if (p < P.world) {
        const unsigned int e = *reinterpret_cast<volatile unsigned int*>(P.epoch) + seq + 1u;
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(P.peer_flags[p] + P.rank), "r"(e) : "memory");
    }
}

// End of a step of `launches` numbered launches: waits (bounded) until every rank has published all of them -- the
// gathered result is then complete on this rank and no peer still reads or writes a buffer of the step -- and only
// then advances the step base.  An ordinary launch, and the step's first decode launch after it is one too, so the
// next step reads the new base.
__global__ void peer_step_end_kernel(const PeerBarrierParams P, const unsigned int launches) {
    const int p = threadIdx.x;
    const unsigned int e = *reinterpret_cast<volatile unsigned int*>(P.epoch) + launches;
    if (p < P.world && *reinterpret_cast<volatile int*>(P.status) == 0) {
        const long long t0 = clock64();
        unsigned int seen = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(P.my_flags + p) : "memory");
            if ((int)(seen - e) >= 0) break;
            if (clock64() - t0 > kPeerWaitCycles) { atomicCAS(P.status, 0, 1 + p); break; }
            __nanosleep(64);
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

namespace {
int barrier_params(const char* who, const cb_scatter* sc, cb::PeerBarrierParams& P) {
    using namespace cb;
    if (sc == nullptr || sc->sync != 2 || sc->world < 1 || sc->world > 8 || sc->rank < 0 || sc->rank >= sc->world ||
        !sc->my_flags || !sc->epoch || !sc->status) {
        set_error("%s: needs a scatter description of a numbered hand-shake (sync == 2) with my_flags, epoch and status", who);
        return CB_ERR_INVALID;
    }
    for (int i = 0; i < sc->world; ++i) {
        if (sc->peer_flags[i] == nullptr) { set_error("%s: peer %d has no flag array", who, i); return CB_ERR_INVALID; }
        P.peer_flags[i] = reinterpret_cast<unsigned int*>(sc->peer_flags[i]);
    }
    P.my_flags = reinterpret_cast<unsigned int*>(sc->my_flags);
    P.epoch = reinterpret_cast<unsigned int*>(sc->epoch);
    P.status = sc->status;
    P.world = sc->world; P.rank = sc->rank;
    return CB_OK;
}
}  // namespace

extern "C" int cb_peer_publish(const cb_scatter* sc, void* stream) {
    using namespace cb;
    PeerBarrierParams P{};
    const int rc = barrier_params("peer_publish", sc, P);
    if (rc != CB_OK) return rc;
    if (sc->seq < 0 || sc->seq >= (1ll << 31)) { set_error("peer_publish: seq out of range"); return CB_ERR_INVALID; }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1); cfg.blockDim = dim3(32); cfg.dynamicSmemBytes = 0;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 1 : 0;
    CB_CUDA_TRY(cudaLaunchKernelEx(&cfg, peer_publish_kernel, P, (unsigned int)sc->seq));
    return CB_OK;
}

extern "C" int cb_peer_step_end(const cb_scatter* sc, int64_t launches, void* stream) {
    using namespace cb;
    PeerBarrierParams P{};
    const int rc = barrier_params("peer_step_end", sc, P);
    if (rc != CB_OK) return rc;
    if (launches < 1 || launches >= (1ll << 31)) { set_error("peer_step_end: launches out of range"); return CB_ERR_INVALID; }
    peer_step_end_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(P, (unsigned int)launches);
    CB_CUDA_TRY(cudaGetLastError());
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
