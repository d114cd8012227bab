// extern "C" entry points of libcrispybits_b200.so: argument checks, scratch layout, kernel choice.
// The host launchers of the reference that this file stands in for are
// Crispybits/Kernel/csrc/packed_gemv.cu:182-337 and packed_gemm.cu:158-203 (libtorch-typed); the checks
// mirror Crispybits/Kernel/csrc/host_utils.h:49-87 as far as raw pointers allow (shape and dtype
// agreement of tensors is checked by the Python shim, which still sees tensors).
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "cb_common.cuh"
#include "cb_gemv_generic.cuh"

namespace cb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int sm_count_current() {
    static int cached[64];  // zero-initialised; device ordinals above 63 are queried each time
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { set_error("cudaGetDevice failed"); return -1; }
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        set_error("cannot query the SM count of device %d", dev);
        return -1;
    }
    if (dev >= 0 && dev < 64) cached[dev] = sms;
    return sms;
}

int launch_gemv_stream(int bits, int dtype, const void* x, const GemvParams& P, int64_t rho, bool pdl, bool chains,
                       int operands, void* scratch, size_t scratch_bytes, cudaStream_t stream);
int stream_status_read_and_clear(int* out);
void chain_stats(long long* out4);
bool stream_plan_query(int bits, int B, int V, int K, int split_k, int64_t rho, int sms, long long* out7);
int launch_peer_wait(const GemvParams& P, cudaStream_t stream);
int launch_peer_signal(const GemvParams& P, cudaStream_t stream);
int gemm_status_read_and_clear(int* out);
int gemm_ws_status_read_and_clear(int* out);
int launch_gemm_ws_gate_up(int dtype, const void* x, int64_t M, const cb_weight* gate, const cb_weight* up, void* out,
                           int64_t K, int bits, int64_t gs, cudaStream_t stream);
int launch_gemm_ws_qkv(int dtype, const void* x, int64_t M, const cb_weight* q, const cb_weight* k, const cb_weight* v,
                       void* out_q, void* out_k, void* out_v, const float* rope_cos, const float* rope_sin, int head_dim,
                       int perm_hd, int64_t K, int bits, int64_t gs, cudaStream_t stream);
int launch_gemm_ws(int dtype, const void* x, int64_t M, const cb_weight* w, void* out, int64_t K, int bits,
                   int64_t gs, int act, cudaStream_t stream, void* scratch, size_t scratch_bytes);
int gemm_ws_splits(int64_t M, int64_t N, int64_t K);
int launch_gemm_tc(int dtype, const void* x, int64_t M, const cb_weight* w, void* out, int64_t K, int bits,
                   int64_t gs, int act, cudaStream_t stream);

// Programmatic dependent launch for the streamlined decode kernel (on unless CRISPYBITS_PDL=0).
static int g_pdl = -1;
bool pdl_enabled() {
    if (g_pdl < 0) {
        const char* e = getenv("CRISPYBITS_PDL");
        g_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return g_pdl != 0;
}
static int g_force_generic = 0;
static int g_gemm_kernel = 0;      // 0: by M, 1: shared-memory-operand kernel, 2: weights-in-TMEM kernel
static int g_chains = 1;           // captured back-to-back ring launches form chains (cb_chain_stats); cb_set_option(4, 0) switches them off
static int g_operands = 0;         // fp16 ring kernel operands: 0 subnormal form, 1 with the 1024 offset

int launch_unpack(const int32_t* packed, int64_t n, int64_t K, int bits, int32_t* codes, cudaStream_t stream);
int launch_quantize_pack(const void* w, int w_dtype, int64_t n, int64_t K, int bits, int64_t gs, int32_t* packed,
                         void* scales, void* zeros, int meta_dtype, cudaStream_t stream);
int launch_gemm_simt(int dtype, const void* x, int64_t M, const cb_weight* w, void* out, int64_t K, int bits,
                     int64_t gs, int act, int round_w, cudaStream_t stream);

namespace {

// Scratch layout: a FIXED region of kMaxCounters arrival counters, then the partial sums.  The
// counter region must not move from call to call: the kernels rely on finding it zero and leave it
// zero, while the partial-sum region holds stale data between calls.
constexpr int64_t kMaxCounters = 65536;
constexpr size_t kCounterBytes = (size_t)kMaxCounters * sizeof(int);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Split-K is a scheduling hint.  A problem with more (batch block x row tile) pairs than counters
// already has far more work units than the GPU has SMs, so it runs unsplit.
inline int64_t effective_split(int64_t B, int64_t V, int64_t split_k) {
    if (split_k <= 1) return 1;
    return ceil_div(B, kMaxBatchBlock) * ceil_div(V, kTileN) > kMaxCounters ? 1 : split_k;
}

#define CB_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) {                        \
            cb::set_error(__VA_ARGS__);       \
            return CB_ERR_INVALID;            \
        }                                     \
    } while (0)

int check_common(const char* who, const void* x, int64_t B, int64_t K, int bits, int64_t gs, int dtype) {
    CB_REQUIRE(B >= 0, "%s: negative batch", who);
    CB_REQUIRE(K > 0 && K < (1ll << 30), "%s: in_features out of range", who);
    CB_REQUIRE(bits == 2 || bits == 3 || bits == 4, "%s: bits must be 2/3/4", who);
    CB_REQUIRE(gs > 0 && gs % 32 == 0, "%s: group_size must be a positive multiple of 32", who);
    CB_REQUIRE(dtype == CB_F32 || dtype == CB_F16 || dtype == CB_BF16, "%s: dtype must be fp32/fp16/bf16", who);
    CB_REQUIRE(B == 0 || x != nullptr, "%s: x is NULL", who);
    return CB_OK;
}

int check_weight(const char* who, const cb_weight* w, int bits) {
    CB_REQUIRE(w != nullptr, "%s: weight record is NULL", who);
    CB_REQUIRE(w->n > 0 && w->n < (1ll << 30), "%s: out_features out of range", who);
    CB_REQUIRE(w->packed && w->scales && w->zeros, "%s: packed/scales/zeros must not be NULL", who);
    // vector loads of whole chunks: 16 B for W4, 8 B for W2, 4 B for W3 (host_utils.h:66-68)
    const uintptr_t align = bits == 4 ? 16 : (bits == 2 ? 8 : 4);
    CB_REQUIRE(reinterpret_cast<uintptr_t>(w->packed) % align == 0,
               "%s: packed storage must be %d-byte aligned for W%d", who, (int)align, bits);
    const size_t esz = 2;  // scales/zeros/bias elements are at least 2 bytes
    CB_REQUIRE(reinterpret_cast<uintptr_t>(w->scales) % esz == 0 && reinterpret_cast<uintptr_t>(w->zeros) % esz == 0,
               "%s: misaligned scales/zeros", who);
    return CB_OK;
}

Proj make_proj(const cb_weight* w, void* out) {
    Proj p{};
    p.w = reinterpret_cast<const uint32_t*>(w->packed);
    p.s = w->scales; p.z = w->zeros; p.b = w->bias; p.out = out; p.n = (int)w->n;
    return p;
}

// Fill the derived fields, carve the scratch, pick the kernel and launch.
int run_decode(const char* who, const void* x, GemvParams& P, int bits, int64_t gs, int dtype, int64_t split_k,
               int64_t rho, void* scratch, size_t scratch_bytes, cudaStream_t stream) {
    CB_REQUIRE(split_k >= 1, "%s: split_k must be >= 1", who);
    CB_REQUIRE((int64_t)P.V * (int64_t)std::max(P.B, 1) < (1ll << 31), "%s: problem too large", who);
    P.nchunks = (int)ceil_div(P.K, 32);
    P.wpr = P.nchunks * bits;
    P.groups = (int)ceil_div(P.K, gs);
    P.group_size = (int)gs;
    P.split_k = (int)std::max<int64_t>(1, std::min<int64_t>(effective_split(P.B, P.V, split_k), P.nchunks));
    P.ntiles = (int)ceil_div(P.V, kTileN);
    P.nbblocks = (int)ceil_div(P.B, kMaxBatchBlock);
    const int64_t units = (int64_t)P.ntiles * P.nbblocks * P.split_k;
    CB_REQUIRE(units < (1ll << 31), "%s: too many work units", who);
    P.units = (int)units;
    P.partial = nullptr;
    P.counters = nullptr;
    if (P.split_k > 1) {
        const size_t need = cb_gemv_scratch_bytes(P.B, P.V, P.split_k);
        CB_REQUIRE(scratch != nullptr && scratch_bytes >= need,
                   "%s: split_k=%d needs %zu bytes of zero-initialised scratch, got %zu", who, P.split_k, need,
                   scratch_bytes);
        CB_REQUIRE(reinterpret_cast<uintptr_t>(scratch) % 16 == 0, "%s: scratch must be 16-byte aligned", who);
        P.counters = reinterpret_cast<int*>(scratch);
        P.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + kCounterBytes);
    }
    if (!g_force_generic) {
        // the shared-memory ring kernel when the problem is inside its domain (-1 = it is not)
        const int rc = launch_gemv_stream(bits, dtype, x, P, rho, pdl_enabled(), g_chains != 0, g_operands, scratch,
                                          scratch_bytes, stream);
        if (rc != -1) return rc;
    }
    // The generic kernels do not carry the rank hand-shake: bracket them with its two halves.
    const bool sync = P.sync.on != 0;
    GemvParams G = P;
    G.sync.on = 0;
    int rc = sync ? launch_peer_wait(P, stream) : CB_OK;
    if (rc != CB_OK) return rc;
    switch (bits) {
        case 2: rc = launch_gemv_generic_w2(dtype, x, G, rho, stream); break;
        case 3: rc = launch_gemv_generic_w3(dtype, x, G, rho, stream); break;
        default: rc = launch_gemv_generic_w4(dtype, x, G, rho, stream); break;
    }
    if (rc != CB_OK) return rc;
    return (sync && P.sync.on == 1) ? launch_peer_signal(P, stream) : CB_OK;
}

}  // namespace
}  // namespace cb

using namespace cb;

extern "C" {

const char* cb_last_error(void) { return g_err; }
const char* cb_version(void) { return "crispybits_b200 0.1 (sm_100a)"; }

size_t cb_gemv_scratch_bytes(int64_t B, int64_t V, int64_t split_k) {
    if (B <= 0 || V <= 0 || effective_split(B, V, split_k) <= 1) return 0;
    return kCounterBytes + (size_t)split_k * (size_t)B * (size_t)V * sizeof(float);
}

int cb_sm_count(void) { return sm_count_current(); }

void cb_set_option(int option, int value) {
    if (option == 0) g_pdl = value ? 1 : 0;
    if (option == 1) g_force_generic = value ? 1 : 0;
    if (option == 3) g_gemm_kernel = (value == 1 || value == 2) ? value : 0;
    if (option == 4) g_chains = value ? 1 : 0;
    if (option == 5) g_operands = value == 1 ? 1 : 0;
}

int cb_decode_status(int* status) {
    if (status == nullptr) { set_error("cb_decode_status: NULL"); return CB_ERR_INVALID; }
    int a = 0, b = 0;
    int rc = stream_status_read_and_clear(&a);
    if (rc != CB_OK) return rc;
    rc = gemm_status_read_and_clear(&b);
    if (rc != CB_OK) return rc;
    int c = 0;
    rc = gemm_ws_status_read_and_clear(&c);
    if (rc != CB_OK) return rc;
    *status = a != 0 ? a : (b != 0 ? 1000 + b : (c != 0 ? 2000 + c : 0));
    return CB_OK;
}
int cb_tile_n(void) { return kTileN; }

int cb_chain_stats(long long* counts4) {
    if (counts4 == nullptr) { set_error("cb_chain_stats: NULL"); return CB_ERR_INVALID; }
    chain_stats(counts4);
    return CB_OK;
}

int cb_decode_plan(int bits, int64_t B, int64_t V, int64_t K, int64_t split_k, int64_t rho, int sms, long long* plan7) {
    if (plan7 == nullptr || sms < 1 || B < 1 || V < 1 || K < 1 || split_k < 1) {
        set_error("cb_decode_plan: bad arguments");
        return CB_ERR_INVALID;
    }
    if (V > 0x7fffffff || K > 0x7fffffff || B > 0x7fffffff ||
        !stream_plan_query(bits, (int)B, (int)V, (int)K, (int)std::min<int64_t>(split_k, 1 << 20), rho, sms, plan7)) {
        set_error("cb_decode_plan: the ring kernel does not take this problem (bits 2/3/4, K %% 256 == 0, 1 <= B <= 8)");
        return CB_ERR_UNSUPPORTED;
    }
    return CB_OK;
}

int cb_max_rho(int bits, int mode) {
    if (!(bits == 2 || bits == 3 || bits == 4)) { set_error("cb_max_rho: bits must be 2/3/4"); return -1; }
    if (mode < CB_MODE_GEMV || mode > CB_MODE_GATEUP) { set_error("cb_max_rho: unknown mode %d", mode); return -1; }
    const int r = bits == 2 ? occupancy_gemv_generic_w2() : bits == 3 ? occupancy_gemv_generic_w3()
                                                                    : occupancy_gemv_generic_w4();
    if (r < 0) set_error("cb_max_rho: occupancy query failed");
    return r;
}

int cb_packed_gemv(const void* x, int64_t B, const cb_weight* w, void* out, int64_t K, int bits,
                   int64_t group_size, int dtype, int64_t split_k, int64_t rho, int act, void* scratch,
                   size_t scratch_bytes, void* stream) {
    int rc = check_common("packed_gemv", x, B, K, bits, group_size, dtype);
    if (rc) return rc;
    if ((rc = check_weight("packed_gemv", w, bits))) return rc;
    CB_REQUIRE(act >= 0 && act <= 2, "packed_gemv: act must be 0 (none), 1 (relu) or 2 (silu)");
    CB_REQUIRE(split_k >= 1, "packed_gemv: split_k must be >= 1");
    if (B == 0) return CB_OK;
    CB_REQUIRE(out != nullptr, "packed_gemv: out is NULL");
    GemvParams P{};
    P.mode = CB_MODE_GEMV;
    P.p[0] = make_proj(w, out);
    P.p[1] = P.p[0]; P.p[2] = P.p[0];
    P.V = (int)w->n; P.B = (int)B; P.K = (int)K; P.act = act;
    return run_decode("packed_gemv", x, P, bits, group_size, dtype, split_k, rho, scratch, scratch_bytes,
                      reinterpret_cast<cudaStream_t>(stream));
}

static int fill_scatter(const char* who, GemvParams& P, const cb_scatter* sc, int64_t rows) {
    if (sc == nullptr) return CB_OK;
    CB_REQUIRE(sc->world >= 1 && sc->world <= 8, "%s: scatter world must be 1..8", who);
    CB_REQUIRE(sc->n_gather >= 0 && sc->n_gather <= rows, "%s: n_gather out of range", who);
    CB_REQUIRE(sc->ld > 0 && sc->col >= 0 && sc->col + sc->n_gather <= sc->ld, "%s: scatter columns out of range", who);
    for (int i = 0; i < sc->world; ++i) {
        CB_REQUIRE(sc->peer_out[i] != nullptr, "%s: scatter target %d is NULL", who, i);
        P.peer_out[i] = sc->peer_out[i];
    }
    P.n_peers = sc->world; P.n_gather = (int)sc->n_gather; P.peer_ld = (int)sc->ld; P.peer_col = (int)sc->col;
    if (sc->sync) {
        CB_REQUIRE(sc->sync == 1 || sc->sync == 2, "%s: scatter sync must be 0, 1 or 2", who);
        CB_REQUIRE(sc->my_flags && sc->epoch && (sc->done || sc->sync == 2) && sc->status && sc->rank >= 0 && sc->rank < sc->world,
                   "%s: scatter hand-shake needs my_flags, epoch, done, status and a rank below world", who);
        CB_REQUIRE(sc->sync == 1 || (sc->seq >= 0 && sc->seq < (1ll << 31)), "%s: scatter seq out of range", who);
        CB_REQUIRE(sc->sync == 1 || (sc->need >= 0 && sc->need <= sc->seq), "%s: scatter need must be 0..seq", who);
        for (int i = 0; i < sc->world; ++i) {
            CB_REQUIRE(sc->peer_flags[i] != nullptr, "%s: peer %d has no flag array", who, i);
            P.sync.peer_flags[i] = reinterpret_cast<unsigned int*>(sc->peer_flags[i]);
        }
        P.sync.my_flags = reinterpret_cast<unsigned int*>(sc->my_flags);
        P.sync.epoch = reinterpret_cast<unsigned int*>(sc->epoch);
        P.sync.done = reinterpret_cast<int*>(sc->done);
        P.sync.status = sc->status;
        P.sync.rank = sc->rank;
        P.sync.on = sc->sync;
        P.sync.seq = sc->sync == 2 ? (unsigned int)sc->seq : 0u;
        P.sync.need = sc->sync == 2 ? (unsigned int)sc->need : 0u;
    }
    return CB_OK;
}

int cb_packed_gemv_scatter(const void* x, int64_t B, const cb_weight* w, void* out, const cb_scatter* scatter,
                           int64_t K, int bits, int64_t group_size, int dtype, int64_t split_k, int64_t rho, int act,
                           void* scratch, size_t scratch_bytes, void* stream) {
    int rc = check_common("packed_gemv_scatter", x, B, K, bits, group_size, dtype);
    if (rc) return rc;
    if ((rc = check_weight("packed_gemv_scatter", w, bits))) return rc;
    CB_REQUIRE(act >= 0 && act <= 2, "packed_gemv_scatter: act must be 0 (none), 1 (relu) or 2 (silu)");
    CB_REQUIRE(split_k >= 1, "packed_gemv_scatter: split_k must be >= 1");
    if (B == 0) return CB_OK;
    CB_REQUIRE(out != nullptr, "packed_gemv_scatter: out is NULL");
    GemvParams P{};
    P.mode = CB_MODE_GEMV;
    P.p[0] = make_proj(w, out);
    P.p[1] = P.p[0]; P.p[2] = P.p[0];
    P.V = (int)w->n; P.B = (int)B; P.K = (int)K; P.act = act;
    if ((rc = fill_scatter("packed_gemv_scatter", P, scatter, w->n))) return rc;
    return run_decode("packed_gemv_scatter", x, P, bits, group_size, dtype, split_k, rho, scratch, scratch_bytes,
                      reinterpret_cast<cudaStream_t>(stream));
}

int cb_fused_gate_up_scatter(const void* x, int64_t B, const cb_weight* gate, const cb_weight* up, void* out,
                             const cb_scatter* scatter, int64_t K, int bits, int64_t group_size, int dtype,
                             int64_t split_k, int64_t rho, void* scratch, size_t scratch_bytes, void* stream) {
    int rc = check_common("fused_gate_up_scatter", x, B, K, bits, group_size, dtype);
    if (rc) return rc;
    if ((rc = check_weight("fused_gate_up_scatter(gate)", gate, bits))) return rc;
    if ((rc = check_weight("fused_gate_up_scatter(up)", up, bits))) return rc;
    CB_REQUIRE(gate->n == up->n, "fused_gate_up_scatter: gate/up shapes must match");
    CB_REQUIRE(split_k >= 1, "fused_gate_up_scatter: split_k must be >= 1");
    if (B == 0) return CB_OK;
    CB_REQUIRE(out != nullptr, "fused_gate_up_scatter: out is NULL");
    GemvParams P{};
    P.mode = CB_MODE_GATEUP;
    P.p[0] = make_proj(gate, out); P.p[0].b = nullptr;
    P.p[1] = make_proj(up, out);   P.p[1].b = nullptr;
    P.p[2] = P.p[0];
    P.V = 2 * (int)gate->n; P.B = (int)B; P.K = (int)K; P.act = 0;
    if ((rc = fill_scatter("fused_gate_up_scatter", P, scatter, gate->n))) return rc;
    return run_decode("fused_gate_up_scatter", x, P, bits, group_size, dtype, split_k, rho, scratch, scratch_bytes,
                      reinterpret_cast<cudaStream_t>(stream));
}

int cb_fused_gate_up(const void* x, int64_t B, const cb_weight* gate, const cb_weight* up, void* out, int64_t K,
                     int bits, int64_t group_size, int dtype, int64_t split_k, int64_t rho, void* scratch,
                     size_t scratch_bytes, void* stream) {
    int rc = check_common("fused_gate_up", x, B, K, bits, group_size, dtype);
    if (rc) return rc;
    if ((rc = check_weight("fused_gate_up(gate)", gate, bits))) return rc;
    if ((rc = check_weight("fused_gate_up(up)", up, bits))) return rc;
    CB_REQUIRE(gate->n == up->n, "fused_gate_up: gate/up shapes must match");
    CB_REQUIRE(split_k >= 1, "fused_gate_up: split_k must be >= 1");
    if (B == 0) return CB_OK;
    CB_REQUIRE(out != nullptr, "fused_gate_up: out is NULL");
    GemvParams P{};
    P.mode = CB_MODE_GATEUP;
    P.p[0] = make_proj(gate, out); P.p[0].b = nullptr;
    P.p[1] = make_proj(up, out);   P.p[1].b = nullptr;
    P.p[2] = P.p[0];
    P.V = 2 * (int)gate->n; P.B = (int)B; P.K = (int)K; P.act = 0;
    return run_decode("fused_gate_up", x, P, bits, group_size, dtype, split_k, rho, scratch, scratch_bytes,
                      reinterpret_cast<cudaStream_t>(stream));
}

int cb_fused_qkv(const void* x, int64_t B, const cb_weight* q, const cb_weight* k, const cb_weight* v,
                 void* out_q, void* out_k, void* out_v, const float* rope_cos, const float* rope_sin,
                 int64_t head_dim, int64_t perm_hd, int64_t K, int bits, int64_t group_size, int dtype,
                 int64_t split_k, int64_t rho, void* scratch, size_t scratch_bytes, void* stream) {
    int rc = check_common("fused_qkv", x, B, K, bits, group_size, dtype);
    if (rc) return rc;
    if ((rc = check_weight("fused_qkv(q)", q, bits))) return rc;
    if ((rc = check_weight("fused_qkv(k)", k, bits))) return rc;
    if ((rc = check_weight("fused_qkv(v)", v, bits))) return rc;
    CB_REQUIRE(split_k >= 1, "fused_qkv: split_k must be >= 1");
    CB_REQUIRE(perm_hd >= 0, "fused_qkv: perm head_dim must be >= 0");
    if (perm_hd > 0) {
        CB_REQUIRE(perm_hd % 2 == 0, "fused_qkv: perm head_dim must be even");
        CB_REQUIRE(q->n % perm_hd == 0 && k->n % perm_hd == 0, "fused_qkv: Q/K widths must be multiples of head_dim");
    }
    const bool rope = rope_cos != nullptr;
    if (rope) {
        CB_REQUIRE(rope_sin != nullptr, "fused_qkv: cos given without sin");
        CB_REQUIRE(perm_hd > 0 && perm_hd == head_dim,
                   "fused_qkv: fused RoPE needs Q/K stored pair-interleaved with the same head_dim");
    }
    if (B == 0) return CB_OK;
    CB_REQUIRE(out_q && out_k && out_v, "fused_qkv: an output pointer is NULL");
    GemvParams P{};
    P.mode = CB_MODE_QKV;
    P.p[0] = make_proj(q, out_q); P.p[1] = make_proj(k, out_k); P.p[2] = make_proj(v, out_v);
    P.V = (int)(q->n + k->n + v->n); P.B = (int)B; P.K = (int)K; P.act = 0;
    P.perm_hd = (int)perm_hd;
    if (rope) { P.rope_cos = rope_cos; P.rope_sin = rope_sin; P.head_dim = (int)head_dim; }
    return run_decode("fused_qkv", x, P, bits, group_size, dtype, split_k, rho, scratch, scratch_bytes,
                      reinterpret_cast<cudaStream_t>(stream));
}

size_t cb_gemm_scratch_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int sp = gemm_ws_splits(M, N, K);
    return sp <= 1 ? 0 : (size_t)sp * (size_t)M * (size_t)N * sizeof(float);
}

int cb_packed_gemm_scratch(const void* x, int64_t M, const cb_weight* w, void* out, int64_t K, int bits,
                           int64_t group_size, int dtype, int act, int use_tensor_cores, void* scratch,
                           size_t scratch_bytes, void* stream) {
    int rc = check_common("packed_gemm", x, M, K, bits, group_size, dtype);
    if (rc) return rc;
    if ((rc = check_weight("packed_gemm", w, bits))) return rc;
    CB_REQUIRE(act >= 0 && act <= 2, "packed_gemm: act must be 0 (none), 1 (relu) or 2 (silu)");
    if (M == 0) return CB_OK;
    CB_REQUIRE(out != nullptr, "packed_gemm: out is NULL");
    CB_REQUIRE(M < (1ll << 30), "packed_gemm: M out of range");
    if (use_tensor_cores && !g_force_generic) {
        // tcgen05 kernels when the problem is inside their domain (-1 = it is not).  Two tilings: the weight-stationary
        // kernel (128 weight rows x 256 tokens per tile, expanded weights in tensor memory, K split over idle SMs when
        // the caller brought scratch; fp16 and bf16) and the shared-memory-operand kernel (256 weight rows x 128 tokens;
        // fp16).  Both run one tile per SM and wave, so the choice is by waves: measured per wave at K = 4096, 33 us for
        // the first and 46 us for the second, plus ~5 us for the reduction of a K split.
        const int sms = sm_count_current();
        const int64_t N = w->n;
        const int sp_all = gemm_ws_splits(M, N, K);
        const int sp = (scratch != nullptr && sp_all > 1 && scratch_bytes >= (size_t)sp_all * M * N * sizeof(float)) ? sp_all : 1;
        bool ws_first = true;
        if (g_gemm_kernel == 1) ws_first = false;
        else if (g_gemm_kernel == 0 && dtype == CB_F16 && sms > 0) {
            const int64_t ws_items = ((M + 255) / 256) * ((N + 127) / 128) * sp;
            const int64_t tc_tiles = ((M + 127) / 128) * ((N + 255) / 256);
            const double kscale = (double)K / 4096.0;
            const double t_ws = (double)((ws_items + sms - 1) / sms) * 33.0 * kscale / sp + (sp > 1 ? 5.0 : 0.0);
            const double t_tc = (double)((tc_tiles + sms - 1) / sms) * 46.0 * kscale;
            ws_first = t_ws <= t_tc;
        }
        for (int attempt = 0; attempt < 2; ++attempt) {
            const bool use_ws = (attempt == 0) == ws_first;
            const int rc2 = use_ws ? launch_gemm_ws(dtype, x, M, w, out, K, bits, group_size, act,
                                                    reinterpret_cast<cudaStream_t>(stream), scratch, scratch_bytes)
                                   : launch_gemm_tc(dtype, x, M, w, out, K, bits, group_size, act,
                                                    reinterpret_cast<cudaStream_t>(stream));
            if (rc2 != -1) return rc2;
        }
    }
    const int round_w = (use_tensor_cores && dtype != CB_F32) ? 1 : 0;
    return launch_gemm_simt(dtype, x, M, w, out, K, bits, group_size, act, round_w,
                            reinterpret_cast<cudaStream_t>(stream));
}

int cb_packed_gemm(const void* x, int64_t M, const cb_weight* w, void* out, int64_t K, int bits,
                   int64_t group_size, int dtype, int act, int use_tensor_cores, void* stream) {
    return cb_packed_gemm_scratch(x, M, w, out, K, bits, group_size, dtype, act, use_tensor_cores, nullptr, 0, stream);
}

int cb_fused_gate_up_gemm(const void* x, int64_t M, const cb_weight* gate, const cb_weight* up, void* out, int64_t K,
                          int bits, int64_t group_size, int dtype, void* stream) {
    int rc = check_common("fused_gate_up_gemm", x, M, K, bits, group_size, dtype);
    if (rc) return rc;
    if ((rc = check_weight("fused_gate_up_gemm(gate)", gate, bits))) return rc;
    if ((rc = check_weight("fused_gate_up_gemm(up)", up, bits))) return rc;
    CB_REQUIRE(gate->n == up->n, "fused_gate_up_gemm: gate/up shapes must match");
    if (M == 0) return CB_OK;
    CB_REQUIRE(out != nullptr, "fused_gate_up_gemm: out is NULL");
    if (!g_force_generic) {
        const int rc2 = launch_gemm_ws_gate_up(dtype, x, M, gate, up, out, K, bits, group_size, reinterpret_cast<cudaStream_t>(stream));
        if (rc2 != -1) return rc2;
    }
    set_error("fused_gate_up_gemm: outside the fused kernel's domain (fp16 / bf16, K a multiple of 128, group size a multiple of 64)");
    return CB_ERR_UNSUPPORTED;
}

int cb_fused_qkv_gemm(const void* x, int64_t M, const cb_weight* q, const cb_weight* k, const cb_weight* v,
                      void* out_q, void* out_k, void* out_v, const float* rope_cos, const float* rope_sin,
                      int64_t head_dim, int64_t perm_hd, int64_t K, int bits, int64_t group_size, int dtype, void* stream) {
    int rc = check_common("fused_qkv_gemm", x, M, K, bits, group_size, dtype);
    if (rc) return rc;
    if ((rc = check_weight("fused_qkv_gemm(q)", q, bits))) return rc;
    if ((rc = check_weight("fused_qkv_gemm(k)", k, bits))) return rc;
    if ((rc = check_weight("fused_qkv_gemm(v)", v, bits))) return rc;
    CB_REQUIRE(perm_hd >= 0, "fused_qkv_gemm: perm head_dim must be >= 0");
    if (perm_hd > 0) {
        CB_REQUIRE(perm_hd % 2 == 0, "fused_qkv_gemm: perm head_dim must be even");
        CB_REQUIRE(q->n % perm_hd == 0 && k->n % perm_hd == 0, "fused_qkv_gemm: Q/K widths must be multiples of head_dim");
    }
    const bool rope = rope_cos != nullptr;
    if (rope) {
        CB_REQUIRE(rope_sin != nullptr, "fused_qkv_gemm: cos given without sin");
        CB_REQUIRE(perm_hd > 0 && perm_hd == head_dim,
                   "fused_qkv_gemm: fused RoPE needs Q/K stored pair-interleaved with the same head_dim");
    }
    if (M == 0) return CB_OK;
    CB_REQUIRE(out_q && out_k && out_v, "fused_qkv_gemm: an output pointer is NULL");
    if (!g_force_generic) {
        const int rc2 = launch_gemm_ws_qkv(dtype, x, M, q, k, v, out_q, out_k, out_v, rope ? rope_cos : nullptr,
                                           rope ? rope_sin : nullptr, (int)head_dim, (int)perm_hd, K, bits, group_size,
                                           reinterpret_cast<cudaStream_t>(stream));
        if (rc2 != -1) return rc2;
    }
    set_error("fused_qkv_gemm: outside the fused kernel's domain (fp16 / bf16, K and every projection's rows multiples "
              "of 128, group size a multiple of 64)");
    return CB_ERR_UNSUPPORTED;
}

int cb_unpack_codes(const int32_t* packed, int64_t n, int64_t K, int bits, int32_t* codes, void* stream) {
    CB_REQUIRE(bits == 2 || bits == 3 || bits == 4, "unpack_codes: bits must be 2/3/4");
    CB_REQUIRE(n >= 0 && K >= 0 && K < (1ll << 30), "unpack_codes: bad shape");
    if (n == 0 || K == 0) return CB_OK;
    CB_REQUIRE(packed && codes, "unpack_codes: NULL pointer");
    return launch_unpack(packed, n, K, bits, codes, reinterpret_cast<cudaStream_t>(stream));
}

int cb_quantize_pack(const void* w, int w_dtype, int64_t n, int64_t K, int bits, int64_t group_size, int32_t* packed,
                     void* scales, void* zeros, int meta_dtype, void* stream) {
    CB_REQUIRE(bits == 2 || bits == 3 || bits == 4, "quantize_pack: bits must be 2/3/4");
    CB_REQUIRE(n >= 0 && K >= 1 && K < (1ll << 30), "quantize_pack: bad shape");
    CB_REQUIRE(group_size > 0 && group_size % 32 == 0, "quantize_pack: group_size must be a positive multiple of 32");
    CB_REQUIRE(w_dtype >= CB_F32 && w_dtype <= CB_BF16 && meta_dtype >= CB_F32 && meta_dtype <= CB_BF16, "quantize_pack: unknown dtype");
    if (n == 0) return CB_OK;
    CB_REQUIRE(w && packed && scales && zeros, "quantize_pack: NULL pointer");
    return launch_quantize_pack(w, w_dtype, n, K, bits, group_size, packed, scales, zeros, meta_dtype,
                                reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
