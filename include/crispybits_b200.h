/*
 * crispybits_b200.h -- C ABI of the B200 (sm_100a) packed W2/W3/W4 linear path.
 *
 * This shared library (libcrispybits_b200.so) replaces the reference's pybind11 binding file
 * Crispybits/Kernel/csrc/bindings.cpp:32-40 and the libtorch-typed launchers behind it.  Every
 * entry point takes raw device pointers, sizes and a CUDA stream; nothing here depends on torch.
 *
 * Conventions
 *   - All pointers are device pointers on the CURRENT CUDA device unless stated otherwise.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).  Calls are
 *     asynchronous: they return after enqueueing work.
 *   - Return value: CB_OK (0) or a CB_ERR_* code; cb_last_error() gives the message of the last
 *     failing call on the calling thread.
 *   - dtype: element type of x, scales, zeros, bias and of the outputs (they must agree, as in
 *     Crispybits/Kernel/csrc/host_utils.h:58,84): CB_F32, CB_F16 or CB_BF16.
 *   - Weight format (Crispybits/Kernel/crispybits_kernels/reference.py:37-55,70-76): `packed` is
 *     int32 [n, ceil(K/32)*bits], a per-row little-endian bitstream with code k at bit k*bits,
 *     rows padded with zero codes to a multiple of 32 codes; `scales` / `zeros` are [n, ceil(K/group_size)]
 *     in `dtype`; `bias` is [n] in `dtype` or NULL.
 *   - Scratch: the decode kernels need device scratch when split_k > 1 (partial sums and
 *     per-tile arrival counters).  The caller owns it: size it with cb_gemv_scratch_bytes(), zero
 *     it ONCE after allocation, and pass it to every call.  The first 256 KiB are the arrival
 *     counters (the same place for every call, so one buffer serves calls of any shape); the
 *     kernels leave them zero again when they finish.  Two calls that may overlap on the GPU
 *     (different streams) need different scratch buffers.
 */
#ifndef CRISPYBITS_B200_H
#define CRISPYBITS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { CB_OK = 0, CB_ERR_INVALID = 1, CB_ERR_CUDA = 2, CB_ERR_UNSUPPORTED = 3 };
enum { CB_F32 = 0, CB_F16 = 1, CB_BF16 = 2 };
/* activation codes: Crispybits/Kernel/csrc/common.cuh:10 */
enum { CB_ACT_NONE = 0, CB_ACT_RELU = 1, CB_ACT_SILU = 2 };
/* decode kernel modes: Crispybits/Kernel/csrc/common.cuh:13 */
enum { CB_MODE_GEMV = 0, CB_MODE_QKV = 1, CB_MODE_GATEUP = 2 };

/* One packed projection (the Proj record of Crispybits/Kernel/csrc/packed_gemv.cu:15-17,
 * without the output pointer). */
typedef struct cb_weight {
    const int32_t* packed; /* [n, ceil(K/32)*bits] */
    const void* scales;    /* [n, ceil(K/group_size)] */
    const void* zeros;     /* same shape as scales   */
    const void* bias;      /* [n] or NULL            */
    int64_t n;             /* output rows            */
} cb_weight;

/* Where a decode launch of a column-parallel stack puts its output (no counterpart in the reference,
 * which is single-GPU).  Output rows r < n_gather are stored to peer_out[p] + (b * ld + col + r) elements
 * for every rank p < world (peer-mapped buffers of [B, ld] elements; the rank's own buffer included);
 * rows r >= n_gather go to the ordinary `out` of the call.
 *
 * With sync != 0 the launch also carries the hand-shake between the ranks, so that no separate barrier
 * is needed: before reading x it waits (bounded, about a second) until every peer has completed as many
 * launches as this rank, and on completion it advances this rank's launch count and publishes it to all
 * peers.  peer_flags[p] is rank p's flag array (world uint32, peer-mapped, zeroed once), my_flags this
 * rank's own; epoch (uint32), done (int32) and status (int32) are zeroed words in this rank's memory:
 * the launch count, the kernel's CTA counter, and 0 or 1 + the first peer not heard from in time (later
 * waits then return at once).  Every rank must issue the same sequence of sync launches.  A launch may
 * overwrite any gathered buffer except the one that launch itself reads on the peers (its x): when it
 * stores, every peer has completed all earlier launches, so two alternating buffers are enough. */
typedef struct cb_scatter {
    void* peer_out[8];
    int world;
    int64_t n_gather;
    int64_t ld;
    int64_t col;
    int sync;
    int rank;
    void* peer_flags[8];
    void* my_flags;
    void* epoch;
    void* done;
    int* status;
    int64_t seq;
    int64_t need;
} cb_scatter;

/* Message of the last error raised on this thread ("" if none). */
const char* cb_last_error(void);

/* Library version string. */
const char* cb_version(void);

/* Decode GEMV  out[B,n] = act(x[B,K] * W^T + bias).
 * Replaces packed_gemv_cuda (Crispybits/Kernel/csrc/packed_gemv.cu:252-269; bindings.cpp:33).
 * split_k >= 1 is clamped to ceil(K/32); rho is the number of resident CTAs per SM the grid is
 * sized for (0 = one CTA per work unit), as in host_utils.h:90-93: the shape-generic kernel uses it
 * that way, the fp16 / bf16 ring kernel plans its own grid (see cb_decode_plan).  scratch may be NULL
 * when split_k == 1. */
int cb_packed_gemv(const void* x, int64_t B, const cb_weight* w, void* out,
                   int64_t K, int bits, int64_t group_size, int dtype,
                   int64_t split_k, int64_t rho, int act,
                   void* scratch, size_t scratch_bytes, void* stream);

/* Fused gate/up decode  out[B,n] = silu(x Wg^T) * (x Wu^T); gate and up have equal shapes and no bias.
 * Replaces fused_gate_up_cuda (packed_gemv.cu:317-337; bindings.cpp:35). */
int cb_fused_gate_up(const void* x, int64_t B, const cb_weight* gate, const cb_weight* up, void* out,
                     int64_t K, int bits, int64_t group_size, int dtype,
                     int64_t split_k, int64_t rho,
                     void* scratch, size_t scratch_bytes, void* stream);

/* Fused Q/K/V decode with optional biases and optional in-kernel RoPE.
 * Replaces fused_qkv_cuda (packed_gemv.cu:271-315; bindings.cpp:36).
 * perm_hd > 0 says Q and K rows are stored pair-interleaved per head of that size; outputs are
 * written in the original column order.  rope_cos / rope_sin are float32 [B, head_dim] or NULL;
 * RoPE needs perm_hd == head_dim. */
int cb_fused_qkv(const void* x, int64_t B,
                 const cb_weight* q, const cb_weight* k, const cb_weight* v,
                 void* out_q, void* out_k, void* out_v,
                 const float* rope_cos, const float* rope_sin, int64_t head_dim, int64_t perm_hd,
                 int64_t K, int bits, int64_t group_size, int dtype,
                 int64_t split_k, int64_t rho,
                 void* scratch, size_t scratch_bytes, void* stream);

/* cb_packed_gemv / cb_fused_gate_up with the all-gather of a column-parallel stack fused into the
 * epilogue: output rows named by `scatter` are written straight into every rank's gathered activation
 * buffer (plain peer stores over NVLink).  scatter == NULL behaves like the plain entry point.  New for
 * the multi-GPU decode stack; the reference has no multi-GPU code. */
int cb_packed_gemv_scatter(const void* x, int64_t B, const cb_weight* w, void* out, const cb_scatter* scatter,
                           int64_t K, int bits, int64_t group_size, int dtype,
                           int64_t split_k, int64_t rho, int act,
                           void* scratch, size_t scratch_bytes, void* stream);
int cb_fused_gate_up_scatter(const void* x, int64_t B, const cb_weight* gate, const cb_weight* up, void* out,
                             const cb_scatter* scatter, int64_t K, int bits, int64_t group_size, int dtype,
                             int64_t split_k, int64_t rho,
                             void* scratch, size_t scratch_bytes, void* stream);

/* One-CTA barrier between the ranks of a column-parallel stack, to be launched on every rank after a
 * scatter launch: tells every peer that this rank's launch is complete and waits (bounded, about a
 * second) until every peer has said so.  peer_flags[p] is rank p's flag array (world uint32, zeroed
 * once, peer-mapped), my_flags this rank's own, epoch a zeroed uint32 in this rank's memory that the
 * kernel advances (graph replays keep counting), status a zeroed int that becomes 1 + p when peer p
 * was not heard from in time (later barriers then return at once).  New for the multi-GPU stack. */
int cb_peer_barrier(void* const* peer_flags, void* my_flags, void* epoch, int* status, int world, int rank,
                    void* stream);

/* Bounded wait, as a one-CTA kernel on `stream`, until every peer has completed as many hand-shake launches
 * as this rank: what a consumer other than a hand-shake launch (a copy to the host, another library's kernel)
 * needs before it reads a gathered buffer.  `scatter` supplies world, my_flags, epoch and status.  New for the
 * multi-GPU stack. */
int cb_peer_wait(const cb_scatter* scatter, void* stream);

/* Numbered hand-shake (scatter->sync == 2), the cheapest of the three: the launches of a step are numbered seq = 0,
 * 1, ... in issue order, identically on every rank.  A scatter launch with seq > 0 waits in the kernel (bounded) until
 * every rank has published `need` completed launches of the running step (flag >= *epoch + need; `epoch`, a zeroed
 * uint32 in this rank's memory, counts the launches of all finished steps) and does not wait for its predecessor's
 * completion on this GPU; the launch with seq == 0 is an ordinary serialised launch and reads the step's input.  `need`
 * is seq for a launch that reads what launch seq - 1 gathered; a launch that reads older data may pass less, but never
 * less than 1 + the number of the last launch that read, on any rank, a buffer this launch overwrites (need <= seq).
 * After EVERY scatter launch call cb_peer_publish with the same seq: a one-CTA kernel that is released by the launch's
 * completion and stores *epoch + seq + 1 into every rank's flag array.  After the step's last publish call cb_peer_step_end with
 * the number of launches: it waits (bounded) until every rank has published all of them -- the result is then
 * complete here and no peer touches the step's buffers any more -- and advances *epoch.  `done` is not used.  Buffers
 * may be reused as with sync == 1.  New for the multi-GPU stack. */
int cb_peer_publish(const cb_scatter* scatter, void* stream);
int cb_peer_step_end(const cb_scatter* scatter, int64_t launches, void* stream);

/* Prefill GEMM  out[M,n] = act(x[M,K] * Wdq^T + bias), float32 accumulation.
 * Replaces packed_gemm_cuda (Crispybits/Kernel/csrc/packed_gemm.cu:182-203; bindings.cpp:34).
 * With use_tensor_cores != 0 and a 16-bit dtype the dequantised weight is rounded to dtype before
 * the product (packed_gemm.cu:56,60) and the tcgen05 kernel is used when the shape allows it. */
int cb_packed_gemm(const void* x, int64_t M, const cb_weight* w, void* out,
                   int64_t K, int bits, int64_t group_size, int dtype,
                   int act, int use_tensor_cores, void* stream);

/* cb_packed_gemm with caller-provided scratch, which lets the tcgen05 kernel split K where the output tiles alone
 * would leave more than half of the SMs idle (few tokens against a narrow matrix: M <= 512 at N = 4096 on 148 SMs).
 * The K ranges store fp32 partial sums [splits, M, n] into `scratch` (16-byte aligned, cb_gemm_scratch_bytes() bytes;
 * its contents need no initialisation and are garbage afterwards) and a second small kernel adds them in range order,
 * applies bias and activation and rounds once: deterministic, same tolerance as the unsplit kernel.  With scratch ==
 * NULL, or where no split applies, this is cb_packed_gemm.  The reference covers every M with one grid rule
 * (Crispybits/Kernel/csrc/packed_gemm.cu:158-179) and has no counterpart of the split. */
int cb_packed_gemm_scratch(const void* x, int64_t M, const cb_weight* w, void* out,
                           int64_t K, int bits, int64_t group_size, int dtype,
                           int act, int use_tensor_cores, void* scratch, size_t scratch_bytes, void* stream);

/* Bytes of scratch cb_packed_gemm_scratch wants for [M, K] x [n, K]^T on the current device (0: it would not split). */
size_t cb_gemm_scratch_bytes(int64_t M, int64_t n, int64_t K);

/* Fused prefill gate/up  out[M,n] = silu(x Wg^T) * (x Wu^T)  in one tcgen05 launch (gate and up rows share a
 * tile as neighbouring tensor-memory lanes).  The reference runs two GEMMs and an elementwise product here
 * (Crispybits/Kernel/crispybits_kernels/ops.py:216-220).  Returns CB_ERR_UNSUPPORTED outside the kernel's domain
 * (fp16 / bf16, K a multiple of 128, group size a multiple of 64); the caller then uses cb_packed_gemm twice. */
int cb_fused_gate_up_gemm(const void* x, int64_t M, const cb_weight* gate, const cb_weight* up, void* out,
                          int64_t K, int bits, int64_t group_size, int dtype, void* stream);

/* Fused prefill Q/K/V: the three projections of x[M,K] in one tcgen05 launch, with the bias, the rotary embedding
 * of Q and K (rope_cos / rope_sin [M, head_dim] float32, or NULL for none) and the un-permuted store in the
 * epilogue -- the prefill counterpart of cb_fused_qkv, same argument meaning.  The reference runs three GEMMs,
 * a column gather and a separate rotation here (Crispybits/Kernel/crispybits_kernels/ops.py:268-272).  Returns
 * CB_ERR_UNSUPPORTED outside the kernel's domain (fp16 / bf16, K and every projection's rows multiples of 128,
 * group size a multiple of 64); the caller then uses cb_packed_gemm per projection. */
int cb_fused_qkv_gemm(const void* x, int64_t M, const cb_weight* q, const cb_weight* k, const cb_weight* v,
                      void* out_q, void* out_k, void* out_v, const float* rope_cos, const float* rope_sin,
                      int64_t head_dim, int64_t perm_hd, int64_t K, int bits, int64_t group_size, int dtype,
                      void* stream);

/* Bit-exact unpack  codes[n,K] (int32) <- packed[n, ceil(K/32)*bits]; the device counterpart of
 * unpack_codes (Crispybits/Kernel/crispybits_kernels/reference.py:58-67; csrc/bitpack.cuh:10-18),
 * exported so that the integer layout can be checked bit-for-bit against the oracle. */
int cb_unpack_codes(const int32_t* packed, int64_t n, int64_t K, int bits, int32_t* codes, void* stream);

/* Quantise and pack on the GPU: the device counterpart of quantize_affine + pack_codes
 * (Crispybits/Kernel/crispybits_kernels/reference.py:10-27, :37-55), bit-identical to them.  w is [n, K] of
 * w_dtype (CB_F32 / CB_F16 / CB_BF16, read as fp32); packed receives [n, ceil(K/32)*bits] words, scales and
 * zeros [n, ceil(K/group_size)] values of meta_dtype (the fp32 results rounded once, as
 * pack_linear_dict does at reference.py:74).  group_size must be a multiple of 32. */
int cb_quantize_pack(const void* w, int w_dtype, int64_t n, int64_t K, int bits, int64_t group_size,
                     int32_t* packed, void* scales, void* zeros, int meta_dtype, void* stream);

/* Decode GEMV with library-owned scratch, for callers that cannot allocate device memory.
 * No counterpart in the reference (its launcher allocates with torch::empty on every call).
 * Same arguments and result as cb_packed_gemv, minus the scratch pair: the Split-K partial sums and
 * arrival counters live in a fixed __device__ array inside the library (cb_static_scratch_bytes()
 * bytes, held by every GPU that loads the library).  This call makes no cudaMalloc / cudaFree and uses
 * no allocating routine.  Limits and rules:
 *   - split_k * B * n must not exceed 262144 (the array's partial-sum room) and
 *     ceil(B/8) * ceil(n/16) must not exceed 65536; larger requests fail with CB_ERR_INVALID;
 *   - the first call on each device looks up the array's device address; make that first call
 *     outside any stream capture.  The address is kept for the life of the process, so the entry
 *     point must not be used on a device after cudaDeviceReset() of that device;
 *   - all calls on a device share the one array: calls that can overlap on the GPU (different
 *     streams, or graphs replayed concurrently) race on it -- serialise them, or give the
 *     overlapping ones their own buffers through cb_packed_gemv. */
int cb_packed_gemv_static_scratch(const void* x, int64_t B, const cb_weight* w, void* out,
                                  int64_t K, int bits, int64_t group_size, int dtype,
                                  int64_t split_k, int64_t rho, int act, void* stream);

/* Size in bytes of the library-owned scratch array used by cb_packed_gemv_static_scratch. */
size_t cb_static_scratch_bytes(void);

/* Bytes of decode scratch needed for a call with batch B, V virtual output rows (n for GEMV,
 * nq+nk+nv for QKV, 2n for gate/up) and this split_k.  Takes the place of the per-call
 * torch::empty of packed_gemv.cu:194-196 and the job-queue workspace of host_utils.h:38-47. */
size_t cb_gemv_scratch_bytes(int64_t B, int64_t V, int64_t split_k);

/* Library options (no counterpart in the reference).  option 0: programmatic dependent launch of the
 * streamlined decode kernel, value 0/1 (default 1, or 0 when CRISPYBITS_PDL=0 is in the environment).
 * With it on, a decode call may start fetching PACKED WEIGHTS before the previous kernel of the
 * stream has finished; activations, outputs and scratch are only touched afterwards.  option 1:
 * value 1 forces the shape-generic decode kernel everywhere (for A/B checks).  option 2: unused.  option 3: which tcgen05 prefill kernel -- 0 (default) the one with fewer estimated waves over the SMs, 1 the kernel with both
 * operands in shared memory (128-token tiles), 2 the kernel with the expanded weights in tensor memory
 * (256-token tiles).  option 4: chains of captured decode launches (see cb_chain_stats), value 0/1, default 1.
 * option 5: operand form of the fp16 ring kernel -- 0 (default) packed fields used as fp16 subnormals, 1 fields
 * OR-ed into 1024.0 with the offset removed per group (for A/B checks of the arithmetic).
 * These switches are plain process-wide words without locking: set them before issuing work, not concurrently
 * with calls on other threads. */
void cb_set_option(int option, int value);

/* Counters of the decode ring kernel's launches issued inside stream capture since the library was loaded
 * (no counterpart in the reference): counts4[0] launches that began a chain, [1] launches that followed another
 * launch of this kernel directly on the same capturing stream, [2] of those, launches that were ordered after their
 * predecessors, [3] of those, launches that ran free.
 *
 * What a chain is: while a stream is being captured (cudaStreamBeginCapture / torch.cuda.graph), consecutive calls
 * of cb_packed_gemv / cb_fused_gate_up / cb_fused_qkv (and their scatter forms) on that stream whose only capture
 * dependency is the previous such call are linked by programmatic launch edges.  A launch whose x / out / scratch
 * byte ranges overlap those of no earlier launch that may still be running (weights, bias and rotary tables are
 * taken to be constant for the duration of the graph) runs FREE: it does not wait for its predecessors and overlaps
 * them on the GPU, but its grid still completes only after theirs.  Every other launch of the chain is ORDERED: it
 * waits for the completion of everything before it, exactly as outside a chain.  Any other work captured in between
 * ends the chain; the next decode call starts a new one with an ordinary full dependency.  Outside capture nothing
 * of this applies, and cb_set_option(4, 0) switches it off.  No device memory is involved. */
int cb_chain_stats(long long* counts4);

/* The launch plan the ring decode kernel would use for a GEMV with batch B (1..8), V virtual output rows, reduction
 * length K (a multiple of 256, group size 128) and the caller's split_k, on a GPU with `sms` multiprocessors.  Pure
 * host arithmetic: needs no GPU and launches nothing.  plan7 receives {grid, dynamic shared memory bytes, K split
 * used, rows per pass, ring slots, passes per CTA, row slabs}.
 * rho: where packed_gemv.cu:184-188 and host_utils.h:90-93 (cb_blocks) size a persistent grid of rho * SMs blocks, the
 * ring kernel sizes its own grid from what fits an SM's shared memory (two CTAs per SM with half of it each where the
 * ring fits, else one), so rho >= 0 does not change its plan; rho < 0 makes it try one CTA per SM first (a tuning and
 * test knob).  The shape-generic kernel honours rho as the reference does.
 * CB_ERR_UNSUPPORTED when the ring kernel does not take the problem (the call then runs the generic kernel). */
int cb_decode_plan(int bits, int64_t B, int64_t V, int64_t K, int64_t split_k, int64_t rho, int sms, long long* plan7);

/* Synchronises the device, then returns in *status the decode kernels' error word and clears it:
 * 0 = no problem; 0 < k < 1000 = in a decode kernel a shared-memory copy of pass k-1 did not arrive
 * within the wait limit and the affected outputs were not written; 1000 + r (2000 + r for the
 * weights-in-TMEM kernel) = in the tensor-core GEMM role r (1 activation producer, 2 MMA issuer,
 * 3 dequantiser, 4 epilogue, 5 packed-word producer) gave up a bounded wait.  No counterpart in the
 * reference. */
int cb_decode_status(int* status);

/* Introspection used by the Split-K policy (packed_gemv.cu:339-347; bindings.cpp:37-39). */
int cb_sm_count(void);                 /* SMs of the current device, or -1 on error     */
int cb_tile_n(void);                   /* virtual output rows per decode work tile       */
int cb_max_rho(int bits, int mode);    /* occupancy-limited resident CTAs per SM, -1 on error */

#ifdef __cplusplus
}
#endif
#endif /* CRISPYBITS_B200_H */
