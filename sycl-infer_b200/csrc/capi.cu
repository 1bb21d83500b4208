// C ABI of the library: argument validation, error reporting, kernel dispatch.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

#include "launch.h"

namespace b200q {

static thread_local char g_err[512] = "";

void set_error(const char * fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char * what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return B200Q_ECUDA;
}

// The opt-in to more than 48 KB of dynamic shared memory is an attribute of a kernel on ONE
// device; a process that drives several GPUs must set it on each.  Remembered per (kernel, device).
cudaError_t ensure_dynamic_smem(const void * func, int bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, int> done;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return e;
    }
    std::lock_guard<std::mutex> lock(mu);
    int & have = done[std::make_pair(func, dev)];
    if (have < bytes) {
        e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) {
            return e;
        }
        have = bytes;
    }
    return cudaSuccess;
}

static bool type_ok(uint32_t t) {
    return t == kQ4_K || t == kQ5_K || t == kQ6_K || t == kQ8_0 || t == kIQ4_XS;
}

static inline bool aligned(const void * p, size_t a) {
    return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

// Validate the segments of one call and flatten them for the kernels.  A call shares
// one quantized activation, so every segment must have the same K.
int build_call(const b200q_seg * segs, int n_segs, int TB, const int8_t * x8, const float * xmeta,
                      const int32_t * xsumq, CallDev & c) {
    if (!segs || n_segs < 1 || n_segs > B200Q_MAX_SEGS) {
        set_error("n_segs must be 1..%d (got %d)", B200Q_MAX_SEGS, n_segs);
        return B200Q_EINVAL;
    }
    if (TB < 1) {
        set_error("TB must be >= 1 (got %d)", TB);
        return B200Q_EINVAL;
    }
    memset(&c, 0, sizeof(c));
    c.K = segs[0].K;
    c.TB = TB;
    c.n_segs = n_segs;
    c.x8 = x8 ? x8 : segs[0].x8;
    c.xmeta = xmeta ? xmeta : segs[0].xmeta;
    c.xsumq = xsumq ? xsumq : segs[0].xsumq;
    if (c.K < 256 || (c.K & 255)) {
        set_error("K must be a positive multiple of 256 (got %d)", c.K);
        return B200Q_EINVAL;
    }
    if (!c.x8 || !c.xmeta || !c.xsumq) {
        set_error("quantized activation views x8/xmeta/xsumq must be non-null");
        return B200Q_EINVAL;
    }
    if (!aligned(c.x8, 16) || !aligned(c.xmeta, 8) || !aligned(c.xsumq, 8)) {
        set_error("x8 must be 16-byte aligned, xmeta and xsumq 8-byte aligned");
        return B200Q_EINVAL;
    }
    int rows = 0;
    for (int i = 0; i < n_segs; i++) {
        const b200q_seg & s = segs[i];
        if (!type_ok(s.type)) {
            set_error("segment %d: unsupported ggml type %u (supported: Q8_0=8 Q4_K=12 Q5_K=13 Q6_K=14 IQ4_XS=23)",
                      i, s.type);
            return B200Q_EUNSUPPORTED;
        }
        if (s.K != c.K) {
            set_error("segment %d: K=%d differs from the call's K=%d", i, s.K, c.K);
            return B200Q_EINVAL;
        }
        if (!x8 && (s.x8 != c.x8 || s.xmeta != c.xmeta || s.xsumq != c.xsumq)) {
            set_error("segment %d: segments of one call must share x8/xmeta/xsumq", i);
            return B200Q_EINVAL;
        }
        if (s.n_rows < 1 || !s.w || !s.out) {
            set_error("segment %d: n_rows must be >= 1 and w/out non-null", i);
            return B200Q_EINVAL;
        }
        if (!aligned(s.w, 16)) {
            set_error("segment %d: weight pointer must be 16-byte aligned", i);
            return B200Q_EINVAL;
        }
        if (s.out_stride < s.n_rows && TB > 1) {
            set_error("segment %d: out_stride %d < n_rows %d", i, s.out_stride, s.n_rows);
            return B200Q_EINVAL;
        }
        if (rows > INT32_MAX - s.n_rows) {
            set_error("too many rows in one call");
            return B200Q_EINVAL;
        }
        rows += s.n_rows;
        SegDev & d = c.seg[i];
        d.w = static_cast<const uint8_t *>(s.w);
        d.out = s.out;
        d.residual = s.residual;
        d.alpha = s.alpha;
        d.type = (int32_t)s.type;
        d.n_rows = s.n_rows;
        d.out_stride = s.out_stride;
        d.row_end = rows;
    }
    c.total_rows = rows;
    return B200Q_OK;
}

// Kernel choice.  One token: the pinned-activation streaming kernel (gemv_pinned.cu).  Two to 32
// tokens: the register-fragment int8 MMA kernel (gemm_frag.cu).  More tokens: the tcgen05 kernel
// (gemm_mma.cu).  What those cannot take (misaligned views, exotic shapes) falls to the streaming
// kernel with shared-memory packs (2..4 tokens), the tcgen05 kernel, or the warp-per-row kernel.
#ifdef B200Q_TUNING
static bool force_rows() {
    static const bool v = [] {
        const char * e = getenv("B200Q_KERNEL");
        return e && strcmp(e, "rows") == 0;
    }();
    return v;
}
static int mma_from_env() {
    static const int env = [] {
        const char * e = getenv("B200Q_MMA_FROM");
        return e && *e ? atoi(e) : 0;
    }();
    return env;
}
#else
static bool force_rows() { return false; }
static int mma_from_env() { return 0; }
#endif
#ifdef B200Q_TUNING
static bool frag_off() {
    static const bool v = [] {
        const char * e = getenv("B200Q_FRAG");
        return e && atoi(e) == 0;
    }();
    return v;
}
#else
static bool frag_off() { return false; }
#endif
// Measured (us per launch, B200).  17408 x 5120 Q4_K: two tokens stream in 14.0 against 19.4 on
// fragments; 3..8 tokens 23..29 (streaming / tcgen05) against 19.1; 16 tokens 38.8 (tcgen05) against
// 29.7; 32 tokens 51.9 against 44.9.  5120 x 17408 Q6_K: 48..49 against 78 up to 8 tokens, 84
// against 91 at 16, 167 against 384 at 32 (40 row tiles of 128 leave most SMs of the tcgen05 kernel idle).
bool gemv_takes_frag(const CallDev & c) {
    if (force_rows() || frag_off() || c.TB < 2 || c.TB > 32) {
        return false;
    }
    if (c.TB == 2 && stream_supported(c)) {
        return false;
    }
    return frag_supported(c);
}
// Fewest tokens that take the tensor-core kernel when the fragment kernel does not apply.
static int mma_from() {
    const int env = mma_from_env();
    return env > 0 ? env : 5;
}
bool gemv_takes_pinned(const CallDev & c) {
    return !force_rows() && c.TB == 1 && pinned_supported(c);
}
bool gemv_takes_stream(const CallDev & c) {
    return !force_rows() && c.TB < mma_from() && stream_supported(c);
}
cudaError_t launch_gemv(cudaStream_t s, const CallDev & c, bool pdl_secondary) {
    if (gemv_takes_pinned(c)) {
        return launch_gemv_pinned(s, c, nullptr, nullptr);
    }
    if (gemv_takes_frag(c)) {
        return launch_gemm_frag(s, c);
    }
    if (!force_rows() && c.TB >= mma_from()) {
        return launch_gemm_mma(s, c, pdl_secondary);
    }
    if (gemv_takes_stream(c)) {
        return launch_gemv_stream(s, c, pdl_secondary);
    }
    // a small batch the streaming kernel cannot hold (long K): the tensor-core kernel as well
    if (!force_rows() && c.TB > 1) {
        return launch_gemm_mma(s, c, pdl_secondary);
    }
    return launch_gemv_rows(s, c, pdl_secondary);
}

// Shared body of the fused quantize + GEMV entry points.
int quant_gemv_call(const char * who, cudaStream_t stream, const b200q_seg * segs, int n_segs, int TB, int8_t * x8,
                    float * xmeta, int32_t * xsumq, const b200q_call_opts * opts) {
    if (!x8 || !xmeta || !xsumq) {
        set_error("%s: scratch x8/xmeta/xsumq must be non-null", who);
        return B200Q_EINVAL;
    }
    CallDev c;
    const int rc = build_call(segs, n_segs, TB, x8, xmeta, xsumq, c);
    if (rc != B200Q_OK) {
        return rc;
    }
    const bool prequant = opts && (opts->flags & B200Q_OPT_PREQUANTIZED);
    const b200q_seg & s0 = segs[0];
    if (!prequant) {
        if (!s0.x || s0.x_stride < s0.K) {
            set_error("%s: segs[0].x must be non-null with x_stride >= K", who);
            return B200Q_EINVAL;
        }
        for (int i = 1; i < n_segs; i++) {
            if (segs[i].x != s0.x || segs[i].act_up != s0.act_up || segs[i].x_stride != s0.x_stride) {
                set_error("%s: segment %d does not share the call's activation", who, i);
                return B200Q_EINVAL;
            }
        }
    }
    if (opts && opts->peers) {
        const b200q_peers * peers = opts->peers;
        if (peers->n_peers < 0 || peers->n_peers > B200Q_MAX_PEERS) {
            set_error("%s: n_peers must be 0..%d (got %d)", who, B200Q_MAX_PEERS, peers->n_peers);
            return B200Q_EINVAL;
        }
        c.n_peers = peers->n_peers;
        for (int i = 0; i < peers->n_peers; i++) {
            if (peers->out_delta[i] & 3) {
                set_error("%s: out_delta[%d] is not a multiple of 4 bytes", who, i);
                return B200Q_EINVAL;
            }
            c.peer_delta[i] = peers->out_delta[i];
        }
    }
    NextAct next{nullptr, nullptr, nullptr};
    if (opts && opts->next) {
        const b200q_next_act & n = *opts->next;
        if (!n.x8 || !n.xmeta || !n.xsumq || !aligned(n.xmeta, 8) || !aligned(n.xsumq, 8)) {
            set_error("%s: next-activation views must be non-null (xmeta, xsumq 8-byte aligned)", who);
            return B200Q_EINVAL;
        }
        if (TB != 1 || n_segs > 2 || (n_segs == 2 && segs[0].n_rows != segs[1].n_rows) || (segs[0].n_rows & 31) ||
            c.n_peers > 0) {
            set_error("%s: the next-activation form needs one token, one segment or two (gate, up) of equal n_rows, "
                      "n_rows a multiple of 32, and no peers", who);
            return B200Q_EINVAL;
        }
        if (!gemv_takes_pinned(c) || !pinned_next_supported(c)) {
            set_error("%s: the next-activation form needs segments of one type and a supported K (K=%d)", who, c.K);
            return B200Q_EUNSUPPORTED;
        }
        next = NextAct{n.x8, n.xmeta, n.xsumq};
    }
    PeerSync sync;
    memset(&sync, 0, sizeof(sync));
    if (opts && (opts->flags & (B200Q_OPT_WAIT_PEERS | B200Q_OPT_SIGNAL_PEERS))) {
        const b200q_peer_sync * ps = opts->sync;
        if (!ps || !ps->flags || ps->world < 1 || ps->world > B200Q_MAX_PEERS + 1 || ps->rank < 0 || ps->rank >= ps->world) {
            set_error("%s: waiting for / signalling peers needs a valid b200q_peer_sync", who);
            return B200Q_EINVAL;
        }
        for (int i = 0; i < ps->world; i++) {
            if (!ps->flags[i]) {
                set_error("%s: sync flags[%d] is null", who, i);
                return B200Q_EINVAL;
            }
            sync.flag[i] = ps->flags[i];
        }
        sync.world = ps->world;
        sync.rank = ps->rank;
        sync.wait = (opts->flags & B200Q_OPT_WAIT_PEERS) ? 1 : 0;
        sync.signal = (opts->flags & B200Q_OPT_SIGNAL_PEERS) ? 1 : 0;
        if (!gemv_takes_pinned(c) || next.x8) {
            set_error("%s: the in-kernel peer exchange serves one-token calls; use b200q_peer_barrier otherwise", who);
            return B200Q_EUNSUPPORTED;
        }
    }
    NormArgs norm{nullptr, 0.0f};
    if (opts && opts->norm) {
        if (!opts->norm->weight || !(opts->norm->eps >= 0.0f)) {
            set_error("%s: norm needs a weight vector and eps >= 0", who);
            return B200Q_EINVAL;
        }
        if (prequant || TB != 1 || !aligned(opts->norm->weight, 16) || !gemv_takes_pinned(c) ||
            !pinned_quantizes(c, s0.x, s0.act_up)) {
            set_error("%s: the folded RMSNorm serves one token with a plain, 16-byte aligned activation and weight "
                      "and a K the single-token kernel takes (K=%d, TB=%d)", who, c.K, TB);
            return B200Q_EUNSUPPORTED;
        }
        norm = NormArgs{opts->norm->weight, opts->norm->eps};
    }
    int32_t * am_idx = nullptr;
    float * am_val = nullptr;
    if (opts && opts->argmax) {
        if (!opts->argmax->idx) {
            set_error("%s: argmax needs an index output", who);
            return B200Q_EINVAL;
        }
        if (TB != 1 || n_segs != 1 || c.n_peers > 0 || next.x8 || !gemv_takes_pinned(c)) {
            set_error("%s: the argmax tail serves one token, one segment, no peers, no next-activation", who);
            return B200Q_EUNSUPPORTED;
        }
        am_idx = opts->argmax->idx;
        am_val = opts->argmax->val;
    }
    if (gemv_takes_pinned(c)) {
        const bool inside = !prequant && pinned_quantizes(c, s0.x, s0.act_up);
        if (!prequant && !inside) { // a quantizer launch of its own: it is the one that waits for the peers
            B200Q_CUDA_OK(launch_xq(stream, s0.x, s0.act_up, s0.x_stride, s0.x_stride, x8, xmeta, xsumq, TB, s0.K, true,
                                    sync.wait ? &sync : nullptr));
            sync.wait = 0;
        }
        B200Q_CUDA_OK(launch_gemv_pinned(stream, c, inside ? s0.x : nullptr, next.x8 ? &next : nullptr,
                                         (sync.wait || sync.signal) ? &sync : nullptr, norm.w ? &norm : nullptr, am_idx,
                                         am_val));
        return B200Q_OK;
    }
    if (!prequant) {
        B200Q_CUDA_OK(launch_xq(stream, s0.x, s0.act_up, s0.x_stride, s0.x_stride, x8, xmeta, xsumq, TB, s0.K, true));
    }
    B200Q_CUDA_OK(launch_gemv(stream, c, true));
    return B200Q_OK;
}

} // namespace b200q

using namespace b200q;

extern "C" {

const char * b200q_last_error(void) {
    return g_err;
}

int b200q_version(void) {
    return B200Q_VERSION;
}

size_t b200q_row_bytes(uint32_t type, int64_t K) {
    return type_ok(type) && K > 0 ? (size_t)(K / 256) * (size_t)sb_bytes(type) : 0;
}

int b200q_xq(void * stream, const float * x, const float * up, int x_stride, int up_stride, int8_t * x8,
             float * xmeta, int32_t * xsumq, int TB, int K) {
    if (!x || !x8 || !xmeta || !xsumq) {
        set_error("b200q_xq: x, x8, xmeta, xsumq must be non-null");
        return B200Q_EINVAL;
    }
    if (TB < 1 || K < 32 || (K & 31)) {
        set_error("b200q_xq: TB >= 1 and K a positive multiple of 32 required (TB=%d K=%d)", TB, K);
        return B200Q_EINVAL;
    }
    if (x_stride < K || (up && up_stride < K)) {
        set_error("b200q_xq: row strides must be >= K");
        return B200Q_EINVAL;
    }
    B200Q_CUDA_OK(launch_xq((cudaStream_t)stream, x, up, x_stride, up_stride, x8, xmeta, xsumq, TB, K, false));
    return B200Q_OK;
}

int b200q_i8_gemm(void * stream, const b200q_seg * segs, int n_segs, int TB) {
    CallDev c;
    const int rc = build_call(segs, n_segs, TB, nullptr, nullptr, nullptr, c);
    if (rc != B200Q_OK) {
        return rc;
    }
    B200Q_CUDA_OK(launch_gemv((cudaStream_t)stream, c, false));
    return B200Q_OK;
}

int b200q_i8_gemv(void * stream, const b200q_seg * segs, int n_segs) {
    return b200q_i8_gemm(stream, segs, n_segs, 1);
}

int b200q_quant_gemv(void * stream, const b200q_seg * segs, int n_segs, int TB, int8_t * x8, float * xmeta,
                     int32_t * xsumq) {
    return quant_gemv_call("b200q_quant_gemv", (cudaStream_t)stream, segs, n_segs, TB, x8, xmeta, xsumq, nullptr);
}

int b200q_quant_gemv_ex(void * stream, const b200q_seg * segs, int n_segs, int TB, int8_t * x8, float * xmeta,
                        int32_t * xsumq, const b200q_call_opts * opts) {
    return quant_gemv_call("b200q_quant_gemv_ex", (cudaStream_t)stream, segs, n_segs, TB, x8, xmeta, xsumq, opts);
}

int b200q_quant_gemv_chain(void * stream, const b200q_chain_call * calls, int n_calls) {
    if (!calls || n_calls < 1) {
        set_error("b200q_quant_gemv_chain: calls must be non-null, n_calls >= 1");
        return B200Q_EINVAL;
    }
    // One launch when every call is one the single-token kernel takes as it stands; the
    // call-by-call path below validates and reports errors either way.
    bool fused = n_calls >= 2 && n_calls <= 4;
    CallDev cd[4];
    const float * xq_x[4];
    NextAct next[4];
    for (int i = 0; i < n_calls && fused; i++) {
        const b200q_chain_call & cc = calls[i];
        const bool prequant = (cc.flags & B200Q_OPT_PREQUANTIZED) != 0;
        fused = cc.segs && cc.x8 && cc.xmeta && cc.xsumq && !(cc.flags & ~B200Q_OPT_PREQUANTIZED) &&
                build_call(cc.segs, cc.n_segs, 1, cc.x8, cc.xmeta, cc.xsumq, cd[i]) == B200Q_OK && gemv_takes_pinned(cd[i]);
        if (!fused) {
            break;
        }
        xq_x[i] = nullptr;
        if (!prequant) {
            const b200q_seg & s0 = cc.segs[0];
            fused = s0.x && s0.x_stride >= s0.K && pinned_quantizes(cd[i], s0.x, s0.act_up);
            for (int j = 1; j < cc.n_segs && fused; j++) {
                fused = cc.segs[j].x == s0.x && cc.segs[j].act_up == s0.act_up && cc.segs[j].x_stride == s0.x_stride;
            }
            xq_x[i] = s0.x;
        }
        next[i] = NextAct{nullptr, nullptr, nullptr};
        if (fused && cc.next) {
            const b200q_next_act & n = *cc.next;
            fused = n.x8 && n.xmeta && n.xsumq && aligned(n.xmeta, 8) && aligned(n.xsumq, 8) && cc.n_segs <= 2 &&
                    (cc.n_segs == 1 || cc.segs[0].n_rows == cc.segs[1].n_rows) && !(cc.segs[0].n_rows & 31) &&
                    pinned_next_supported(cd[i]);
            next[i] = NextAct{n.x8, n.xmeta, n.xsumq};
        }
    }
    if (fused && chain_supported(cd, xq_x, next, n_calls)) {
        B200Q_CUDA_OK(launch_gemv_chain((cudaStream_t)stream, cd, xq_x, next, n_calls));
        return B200Q_OK;
    }
    for (int i = 0; i < n_calls; i++) {
        const b200q_chain_call & cc = calls[i];
        b200q_call_opts opts = {};
        opts.flags = cc.flags;
        opts.next = cc.next;
        const int rc = quant_gemv_call("b200q_quant_gemv_chain", (cudaStream_t)stream, cc.segs, cc.n_segs, 1, cc.x8,
                                       cc.xmeta, cc.xsumq, &opts);
        if (rc != B200Q_OK) {
            return rc;
        }
    }
    return B200Q_OK;
}

int b200q_quant_gemv_scatter(void * stream, const b200q_seg * segs, int n_segs, int TB, int8_t * x8, float * xmeta,
                             int32_t * xsumq, const b200q_peers * peers) {
    if (!peers) {
        set_error("b200q_quant_gemv_scatter: peers must be non-null");
        return B200Q_EINVAL;
    }
    b200q_call_opts opts = {};
    opts.peers = peers;
    return quant_gemv_call("b200q_quant_gemv_scatter", (cudaStream_t)stream, segs, n_segs, TB, x8, xmeta, xsumq, &opts);
}

int b200q_peer_barrier(void * stream, uint32_t * const * flags, int world, int rank, uint32_t seq) {
    if (!flags || world < 1 || world > B200Q_MAX_PEERS + 1 || rank < 0 || rank >= world) {
        set_error("b200q_peer_barrier: bad world/rank (%d/%d) or null flags", rank, world);
        return B200Q_EINVAL;
    }
    for (int i = 0; i < world; i++) {
        if (!flags[i]) {
            set_error("b200q_peer_barrier: flags[%d] is null", i);
            return B200Q_EINVAL;
        }
    }
    B200Q_CUDA_OK(launch_peer_barrier((cudaStream_t)stream, flags, world, rank, seq));
    return B200Q_OK;
}

int b200q_i8_block_dots(void * stream, const void * w, uint32_t type, int K, int n_rows, const int8_t * x8, int TB,
                        int t, int32_t * wd) {
    if (!w || !x8 || !wd || !type_ok(type)) {
        set_error("b200q_i8_block_dots: null pointer or unsupported type %u", type);
        return type_ok(type) ? B200Q_EINVAL : B200Q_EUNSUPPORTED;
    }
    if (K < 256 || (K & 255) || n_rows < 1 || TB < 1 || t < 0 || t >= TB || !aligned(w, 16) || !aligned(x8, 16)) {
        set_error("b200q_i8_block_dots: bad shape or alignment (K=%d n_rows=%d TB=%d t=%d)", K, n_rows, TB, t);
        return B200Q_EINVAL;
    }
    // Same rule as the GEMV dispatch, so the sums come out of the code that serves such a call:
    // one token: the half-superblock decoders of the pinned kernel; 2..32 tokens: the
    // register-fragment MMA kernel, which then stores its accumulator fragments; more tokens: the
    // tcgen05 kernel, whose epilogue stores the accumulators it read from tensor memory.
    const uint8_t * wb = static_cast<const uint8_t *>(w);
    if (TB >= 2) {
        CallDev c;
        memset(&c, 0, sizeof(c));
        c.K = K;
        c.TB = TB;
        c.n_segs = 1;
        c.total_rows = n_rows;
        c.x8 = x8;
        // the instrument has no scales or sums: the producers' loads of them land inside x8 (8 of
        // every group's 32 bytes) and what they read is never used
        c.xmeta = reinterpret_cast<const float *>(x8);
        c.xsumq = reinterpret_cast<const int32_t *>(x8);
        c.seg[0].w = wb;
        c.seg[0].out = reinterpret_cast<float *>(wd); // never written in this mode
        c.seg[0].alpha = 1.0f;
        c.seg[0].type = (int32_t)type;
        c.seg[0].n_rows = n_rows;
        c.seg[0].out_stride = n_rows;
        c.seg[0].row_end = n_rows;
        if (gemv_takes_frag(c)) {
            B200Q_CUDA_OK(launch_gemm_frag((cudaStream_t)stream, c, wd, t));
        } else if (TB >= mma_from()) {
            B200Q_CUDA_OK(launch_gemm_mma((cudaStream_t)stream, c, false, wd, t));
        } else {
            B200Q_CUDA_OK(launch_unit_dots((cudaStream_t)stream, wb, (int)type, K, n_rows, x8, TB, t, wd));
        }
    } else if (TB == 1 && K > 65536) { // beyond the streaming kernels: the warp-per-row kernel's decoders
        B200Q_CUDA_OK(launch_block_dots((cudaStream_t)stream, wb, (int)type, K, n_rows, x8, TB, t, wd));
    } else {
        B200Q_CUDA_OK(launch_unit_dots((cudaStream_t)stream, wb, (int)type, K, n_rows, x8, TB, t, wd));
    }
    return B200Q_OK;
}

int b200q_moe_route(void * stream, const float * gate_inp, const float * x, int x_stride, int n_tok, int n_embd,
                    int n_expert, int top_k, float * logits, int32_t * ids, float * wts) {
    if (!logits || !ids || !wts || (gate_inp && !x)) {
        set_error("b200q_moe_route: logits, ids, wts (and x with gate_inp) must be non-null");
        return B200Q_EINVAL;
    }
    if (n_tok < 1 || n_expert < 1 || n_expert > 4096 || top_k < 1 || top_k > n_expert || (gate_inp && n_embd < 1)) {
        set_error("b200q_moe_route: bad shape (n_tok=%d n_expert=%d top_k=%d n_embd=%d)", n_tok, n_expert, top_k,
                  n_embd);
        return B200Q_EINVAL;
    }
    B200Q_CUDA_OK(launch_moe_route((cudaStream_t)stream, gate_inp, x, x_stride, n_tok, n_embd, n_expert, top_k, logits,
                                   ids, wts));
    return B200Q_OK;
}

int b200q_moe_route_csr(void * stream, const float * gate_inp, const float * x, int x_stride, int n_tok, int n_embd,
                        int n_expert, int top_k, float * logits, int32_t * ids, float * wts, int32_t * off,
                        int32_t * pair, int32_t * active, int32_t * n_active) {
    if (!logits || !ids || !wts || (gate_inp && !x) || !off || !pair || !active || !n_active) {
        set_error("b200q_moe_route_csr: logits, ids, wts, off, pair, active, n_active (and x with gate_inp) must be non-null");
        return B200Q_EINVAL;
    }
    if (n_tok < 1 || n_expert < 1 || n_expert > 4096 || top_k < 1 || top_k > n_expert || (gate_inp && n_embd < 1)) {
        set_error("b200q_moe_route_csr: bad shape (n_tok=%d n_expert=%d top_k=%d n_embd=%d)", n_tok, n_expert, top_k,
                  n_embd);
        return B200Q_EINVAL;
    }
    B200Q_CUDA_OK(launch_moe_route((cudaStream_t)stream, gate_inp, x, x_stride, n_tok, n_embd, n_expert, top_k, logits,
                                   ids, wts, off, pair, active, n_active));
    return B200Q_OK;
}

int b200q_moe_csr(void * stream, const int32_t * ids, int n_pairs, int n_expert, int32_t * off, int32_t * pair,
                  int32_t * active, int32_t * n_active) {
    if (!ids || !off || !pair || !active || !n_active || n_pairs < 1 || n_expert < 1) {
        set_error("b200q_moe_csr: null pointer or empty shape");
        return B200Q_EINVAL;
    }
    B200Q_CUDA_OK(launch_moe_csr((cudaStream_t)stream, ids, n_pairs, n_expert, off, pair, active, n_active));
    return B200Q_OK;
}

static int moe_check(const char * who, const void * bank, uint32_t type, int K, int n_rows, const void * a,
                     const void * b, const void * c, const void * d) {
    if (!bank || !a || !b || !c || !d) {
        set_error("%s: null pointer", who);
        return B200Q_EINVAL;
    }
    if (!type_ok(type)) {
        set_error("%s: unsupported ggml type %u", who, type);
        return B200Q_EUNSUPPORTED;
    }
    if (K < 256 || (K & 255) || n_rows < 1 || !aligned(bank, 16)) {
        set_error("%s: K must be a multiple of 256, rows >= 1, banks 16-byte aligned (K=%d rows=%d)", who, K, n_rows);
        return B200Q_EINVAL;
    }
    return B200Q_OK;
}

static int moe_gate_up_call(const char * who, void * stream, const void * gbank, const void * ubank, uint32_t gtype,
                            uint32_t utype, size_t slot_gb, size_t slot_ub, const int32_t * off, const int32_t * pair,
                            const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                            const float * xmeta, const int32_t * xsumq, int n_tok, float * h, int h_stride, int n_embd,
                            int n_ff_exp, int top_k, const NextAct * hq) {
    int rc = moe_check(who, gbank, gtype, n_embd, n_ff_exp, off, pair, active, n_active);
    if (rc == B200Q_OK) {
        rc = moe_check(who, ubank, utype, n_embd, n_ff_exp, x8, xmeta, xsumq, h);
    }
    if (rc != B200Q_OK) {
        return rc;
    }
    if (!aligned(x8, 16) || !aligned(xmeta, 8) || !aligned(xsumq, 8)) {
        set_error("%s: x8 must be 16-byte aligned, xmeta and xsumq 8-byte aligned", who);
        return B200Q_EINVAL;
    }
    if (n_act_max < 1 || n_tok < 1 || top_k < 1 || h_stride < n_ff_exp || (slot_gb & 15) || (slot_ub & 15)) {
        set_error("%s: bad n_act_max/n_tok/top_k/h_stride or plane bytes not a multiple of 16", who);
        return B200Q_EINVAL;
    }
    if (hq && (!hq->x8 || !hq->xmeta || !hq->xsumq || !aligned(hq->x8, 16) || !aligned(hq->xmeta, 8) ||
               !aligned(hq->xsumq, 8) || (n_ff_exp & 31))) {
        set_error("%s: h8/hmeta/hsumq must be non-null and aligned (16/8/8 bytes), n_ff_exp a multiple of 32", who);
        return B200Q_EINVAL;
    }
    const bool inside = hq && moe_rows_takes_pinned((int)gtype, (int)utype, n_embd, n_ff_exp, 1, n_tok, top_k, n_act_max, true);
    B200Q_CUDA_OK(launch_moe_rows((cudaStream_t)stream, gbank, ubank, (int)gtype, (int)utype, slot_gb, slot_ub, off,
                                  pair, active, n_active, n_act_max, x8, xmeta, xsumq, n_tok, top_k, n_embd, n_ff_exp,
                                  h, h_stride, 1, inside ? hq : nullptr));
    if (hq && !inside) { // the kernel that served this shape leaves h in fp32 only
        B200Q_CUDA_OK(launch_xq((cudaStream_t)stream, h, nullptr, h_stride, h_stride, hq->x8, hq->xmeta, hq->xsumq,
                                n_tok * top_k, n_ff_exp, false));
    }
    return B200Q_OK;
}

int b200q_moe_gate_up(void * stream, const void * gbank, const void * ubank, uint32_t gtype, uint32_t utype,
                      size_t slot_gb, size_t slot_ub, const int32_t * off, const int32_t * pair,
                      const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                      const float * xmeta, const int32_t * xsumq, int n_tok, float * h, int h_stride, int n_embd,
                      int n_ff_exp, int top_k) {
    return moe_gate_up_call("b200q_moe_gate_up", stream, gbank, ubank, gtype, utype, slot_gb, slot_ub, off, pair, active,
                            n_active, n_act_max, x8, xmeta, xsumq, n_tok, h, h_stride, n_embd, n_ff_exp, top_k, nullptr);
}

int b200q_moe_gate_up_q(void * stream, const void * gbank, const void * ubank, uint32_t gtype, uint32_t utype,
                        size_t slot_gb, size_t slot_ub, const int32_t * off, const int32_t * pair,
                        const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                        const float * xmeta, const int32_t * xsumq, int n_tok, float * h, int h_stride, int n_embd,
                        int n_ff_exp, int top_k, int8_t * h8, float * hmeta, int32_t * hsumq) {
    const NextAct hq{h8, hmeta, hsumq};
    return moe_gate_up_call("b200q_moe_gate_up_q", stream, gbank, ubank, gtype, utype, slot_gb, slot_ub, off, pair, active,
                            n_active, n_act_max, x8, xmeta, xsumq, n_tok, h, h_stride, n_embd, n_ff_exp, top_k, &hq);
}

int b200q_moe_down(void * stream, const void * dbank, uint32_t dtype, size_t slot_db, const int32_t * off,
                   const int32_t * pair, const int32_t * active, const int32_t * n_active, int n_act_max,
                   const int8_t * h8, const float * hmeta, const int32_t * hsumq, int n_pairs, float * acc,
                   int acc_stride, int n_embd, int n_ff_exp) {
    int rc = moe_check("b200q_moe_down", dbank, dtype, n_ff_exp, n_embd, off, pair, active, n_active);
    if (rc == B200Q_OK) {
        rc = moe_check("b200q_moe_down", dbank, dtype, n_ff_exp, n_embd, h8, hmeta, hsumq, acc);
    }
    if (rc != B200Q_OK) {
        return rc;
    }
    if (!aligned(h8, 16) || !aligned(hmeta, 8) || !aligned(hsumq, 8)) {
        set_error("b200q_moe_down: h8 must be 16-byte aligned, hmeta and hsumq 8-byte aligned");
        return B200Q_EINVAL;
    }
    if (n_act_max < 1 || n_pairs < 1 || acc_stride < n_embd || (slot_db & 15)) {
        set_error("b200q_moe_down: bad n_act_max/n_pairs/acc_stride or plane bytes not a multiple of 16");
        return B200Q_EINVAL;
    }
    B200Q_CUDA_OK(launch_moe_rows((cudaStream_t)stream, dbank, nullptr, (int)dtype, (int)dtype, slot_db, 0, off, pair,
                                  active, n_active, n_act_max, h8, hmeta, hsumq, n_pairs, 0, n_ff_exp, n_embd, acc,
                                  acc_stride, 0));
    return B200Q_OK;
}

int b200q_moe_reduce(void * stream, const float * acc, const float * wts, int top_k, int n_tok, int n_embd,
                     int acc_stride, float * out, int out_stride) {
    if (!acc || !wts || !out || top_k < 1 || n_tok < 1 || n_embd < 1 || acc_stride < n_embd || out_stride < n_embd) {
        set_error("b200q_moe_reduce: null pointer or bad shape");
        return B200Q_EINVAL;
    }
    B200Q_CUDA_OK(launch_moe_reduce((cudaStream_t)stream, acc, wts, top_k, n_tok, n_embd, acc_stride, out, out_stride));
    return B200Q_OK;
}

int b200q_device_status(int * status, int clear) {
    if (!status) {
        set_error("b200q_device_status: status must be non-null");
        return B200Q_EINVAL;
    }
    B200Q_CUDA_OK(read_device_status(status, clear != 0));
    int mma = 0;
    B200Q_CUDA_OK(read_mma_status(&mma, clear != 0));
    *status = *status ? *status : mma;
    int peer = 0;
    B200Q_CUDA_OK(read_peer_status(&peer, clear != 0));
    *status = *status ? *status : peer;
    int moe = 0;
    B200Q_CUDA_OK(read_moe_status(&moe, clear != 0));
    *status = *status ? *status : moe;
    int pin = 0;
    B200Q_CUDA_OK(read_pin_status(&pin, clear != 0));
    *status = *status ? *status : pin;
    int xq = 0;
    B200Q_CUDA_OK(read_xq_status(&xq, clear != 0));
    *status = *status ? *status : xq;
    int frag = 0;
    B200Q_CUDA_OK(read_frag_status(&frag, clear != 0));
    *status = *status ? *status : frag;
    int probe = 0;
    B200Q_CUDA_OK(read_probe_status(&probe, clear != 0));
    *status = *status ? *status : probe;
    if (*status != 0) {
        set_error("a bounded device-side wait ran out (status %d)", *status);
    }
    return B200Q_OK;
}

int b200q_argmax(void * stream, const float * logits, int n, int32_t * out_idx, float * out_val, int M) {
    if (!logits || !out_idx || n < 1 || M < 1) {
        set_error("b200q_argmax: logits and out_idx must be non-null, n >= 1, M >= 1");
        return B200Q_EINVAL;
    }
    B200Q_CUDA_OK(launch_argmax((cudaStream_t)stream, logits, n, out_idx, out_val, M));
    return B200Q_OK;
}

int b200q_probe_hbm_read(void * stream, const void * buf, size_t bytes, uint32_t * sink) {
    if (!buf || !sink || bytes < 16 || !aligned(buf, 16)) {
        set_error("b200q_probe_hbm_read: buf (16-byte aligned, at least 16 bytes) and sink must be non-null");
        return B200Q_EINVAL;
    }
    B200Q_CUDA_OK(launch_probe_read((cudaStream_t)stream, buf, bytes, sink));
    return B200Q_OK;
}

int b200q_probe_i8_mma(void * stream, int iters, uint32_t * sink) {
    if (!sink || iters < 1 || iters > (1 << 24)) {
        set_error("b200q_probe_i8_mma: sink must be non-null, 1 <= iters <= 2^24");
        return B200Q_EINVAL;
    }
    B200Q_CUDA_OK(launch_probe_i8_mma((cudaStream_t)stream, iters, sink));
    return B200Q_OK;
}

int b200q_synchronize(void * stream) {
    B200Q_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
    return B200Q_OK;
}

} // extern "C"
