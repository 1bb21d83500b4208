/* b200q - B200 (sm_100a) quantized GEMV/GEMM over raw GGUF blocks: C ABI.
 *
 * Drop-in boundary for the integer GEMV/GEMM path of the sycl-infer engine's
 * backend-operator interface.  Every entry point names the reference interface
 * it replaces (paths inside the reference project).  All pointers are DEVICE
 * pointers unless a parameter says "host"; the caller owns every buffer; the
 * library allocates nothing and never falls back to the CPU: an unsupported
 * request is an error.  State the library keeps: a thread-local error string;
 * per GPU a few device words (the status words behind b200q_device_status, the
 * completion counters of b200q_moe_route_csr and b200q_quant_gemv_chain, the
 * keys and counters of b200q_argmax and of the argmax option) and the 48 KB
 * scratch array of b200q_quant_gemv_static; per process a cache of per-device
 * kernel attributes and one flag (a call with the norm option has been seen: from
 * then on single-token launches use the kernel image that can apply a norm); per
 * b200q_gguf handle the file mappings.
 *
 * Launch chaining.  GEMV launches use programmatic stream serialization: a kernel
 * may start streaming WEIGHTS while the previous kernel of the stream (when that
 * is one of this library's) is still finishing, and waits for it before it reads
 * an activation or writes an output.  Weights must therefore not be produced by a
 * b200q call that directly precedes their use in the same stream (they never are:
 * no entry point writes weights).
 *
 * `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 * stream).  Calls only enqueue work; they do not synchronize.
 *
 * Activation layout (the one the reference's quantizer writes,
 * src/backend/cpu/kernels/xq.cpp:1-5): group-major, token t, 32-value group g:
 *   x8[(g*TB + t)*32 + i]          int8 codes
 *   xmeta[2*(g*TB + t)]            fp32 scale (already rounded through f16), [+1] = 0
 *   xsumq[2*(g*TB + t) + {0,1}]    sums of codes 0..15 and 16..31
 * Weight layout: raw GGUF blocks, row r at w + r * row_bytes(type, K).
 */
#ifndef B200Q_H
#define B200Q_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200Q_VERSION 1

/* ggml type ids (src/model/gguf.h:8-32) */
enum { B200Q_Q8_0 = 8, B200Q_Q4_K = 12, B200Q_Q5_K = 13, B200Q_Q6_K = 14, B200Q_IQ4_XS = 23 };

/* Status codes.  Mirrors the reference C ABI's convention of an integer status
 * plus a thread-local message (include/sycl_infer/sycl_infer.h:54-59). */
enum {
    B200Q_OK = 0,
    B200Q_EINVAL = 1,      /* bad argument: shape, alignment, null pointer */
    B200Q_EUNSUPPORTED = 2, /* type or size this library has no kernel for */
    B200Q_ECUDA = 3,        /* a CUDA runtime call failed */
    B200Q_ETIMEOUT = 4      /* a bounded device-side wait ran out (see b200q_device_status) */
};

#define B200Q_MAX_SEGS 8
#define B200Q_MAX_PEERS 7

/* One GEMV output segment: field for field the reference's cpu_gemv_seg
 * (src/backend/cpu/cpu_types.h:68-86) / gemv_seg (src/backend/gpu/kernels/kernels.h:44-81)
 * without the repacked-store members this path never reads. */
typedef struct b200q_seg {
    const void * w;         /* raw GGUF blocks [n_rows][K], 16-byte aligned */
    uint32_t type;          /* ggml type of w */
    int32_t K;              /* input length, multiple of 256 */
    int32_t n_rows;         /* output rows */
    const float * x;        /* fp32 activations, row stride x_stride (fused-quantize entry points) */
    int32_t x_stride;
    const float * act_up;   /* non-null: the activation is silu(x) * act_up (same stride as x) */
    float * out;            /* out[t*out_stride + row] */
    int32_t out_stride;
    const float * residual; /* optional, same indexing as out; may alias out */
    float alpha;            /* out = alpha * dot (+ residual) */
    const int8_t * x8;      /* quantized activation views (see header comment) */
    const float * xmeta;
    const int32_t * xsumq;
} b200q_seg;

const char * b200q_last_error(void);
int b200q_version(void);
/* bytes of one weight row; 0 for an unsupported type.  quant_row_bytes, src/common/quant.h:1177-1198 */
size_t b200q_row_bytes(uint32_t type, int64_t K);

/* compute_backend::xq (src/backend/backend.h:104-105) = cpu_xq (src/backend/cpu/kernels/xq.cpp:10-50).
 * `up` non-null quantizes silu(x)*up.  x8 must be 16-byte aligned. */
int b200q_xq(void * stream, const float * x, const float * up, int x_stride, int up_stride, int8_t * x8,
             float * xmeta, int32_t * xsumq, int TB, int K);

/* compute_backend::i8_gemv (src/backend/backend.h:113) = cpu_i8_gemv (src/backend/cpu/kernels/i8.cpp:498-516),
 * extended to the n_segs segments of one call that share a quantized activation
 * (seg_plan::call_t, src/engine/engine_types.h:46-61): one launch for q|k|v or gate|up. */
int b200q_i8_gemv(void * stream, const b200q_seg * segs /*host*/, int n_segs);

/* compute_backend::i8_gemm (src/backend/backend.h:114) = cpu_i8_gemm (src/backend/cpu/kernels/i8.cpp:518-546):
 * TB tokens, out[t*out_stride + row]. */
int b200q_i8_gemm(void * stream, const b200q_seg * segs /*host*/, int n_segs, int TB);

/* Quantize the call's activation (segs[0].x / act_up, TB tokens) into the caller's
 * x8/xmeta/xsumq scratch and run every segment: the analogue of the reference's fused
 * decode launch i8_grp_quant_gemv_launch (src/backend/gpu/kernels/kernels.h:216-219).
 * The segments' x8/xmeta/xsumq fields are ignored; the scratch arguments are used. */
int b200q_quant_gemv(void * stream, const b200q_seg * segs /*host*/, int n_segs, int TB, int8_t * x8, float * xmeta,
                     int32_t * xsumq);

/* Options of b200q_quant_gemv_ex. */
#define B200Q_OPT_PREQUANTIZED 1u /* the scratch already holds the call's quantized activation: no quantizer runs */
#define B200Q_OPT_WAIT_PEERS 2u   /* before reading the activation, wait until every peer has signalled as often as this rank */
#define B200Q_OPT_SIGNAL_PEERS 4u /* after the last output is stored on every peer, signal all peers */

/* Flag words of the cross-GPU exchange, one array per rank, every array mapped on every rank
 * (the same arrays b200q_peer_barrier uses): flags[p] is rank p's array as mapped on this GPU,
 * at least 64 words, zero before the first call.  Word r of an array counts rank r's signals;
 * words 32 and 33 are the owner's own counters.  With B200Q_OPT_SIGNAL_PEERS the last CTA of
 * the launch tells every peer "my outputs of this call are in your memory"; with
 * B200Q_OPT_WAIT_PEERS the launch's first action after the previous kernel has finished is a
 * bounded wait (about a second, then B200Q_ETIMEOUT in the status word) for all peers' signals
 * of the previous call.  Together they replace the separate b200q_peer_barrier launch between
 * two row-sharded calls.  One token only; other calls use b200q_peer_barrier. */
typedef struct b200q_peer_sync {
    uint32_t * const * flags; /* host array of `world` device pointers */
    int32_t world, rank;
} b200q_peer_sync;

/* Where a call leaves the NEXT call's activation.  The reference quantizes every GEMV input
 * right in front of the GEMV (cpu_xq, src/backend/cpu/kernels/xq.cpp:10-50), for the down
 * projection as silu(gate)*up (act_up, src/engine/graph.cpp:355-357; xq.cpp:21-26).  With this
 * set, the GEMV that produces those values emits the quantized activation itself (one token),
 * so the next call runs with B200Q_OPT_PREQUANTIZED: no quantizer launch, and every CTA of
 * the next call fetches K*1.5 bytes instead of quantizing K floats.  Two forms:
 *   one segment           the call's output vector (alpha, residual applied) is quantized;
 *   two segments (gate|up) silu(gate)*up is quantized; equal n_rows, one weight type.
 * n_rows must be a multiple of 32: such a call splits its rows over the SMs in whole 32-row
 * groups, so that the CTA finishing a group holds all of its values. */
typedef struct b200q_next_act {
    int8_t * x8;      /* [n_rows] codes of silu(gate)*up */
    float * xmeta;    /* [n_rows/32][2] */
    int32_t * xsumq;  /* [n_rows/32][2] */
} b200q_next_act;

struct b200q_peers;
/* RMSNorm folded into the call's quantizer: the activation the call consumes is
 *   rmsnorm(x)[i] = x[i] * (1 / sqrt(sum(x^2) / K + eps)) * weight[i]
 * (rmsnorm_row, src/backend/cpu/kernels/common.cpp:685-691; device twin
 * src/backend/gpu/kernels/rmsnorm.cpp - the engine runs it as a launch of its own ahead of the
 * q|k|v and gate|up calls), quantized as b200q_xq would quantize that row.  The sum of squares is
 * formed in the order of the reference's AVX-512 helper (common.cpp:278-290: sixteen fused-
 * multiply-add accumulators over i = 16k + j, halved 16 -> 8 -> 4, then (t0 + t2) + (t1 + t3)), so
 * the codes are those of the reference on such a host, bit for bit.  One token, plain activation
 * (no act_up), x and weight 16-byte aligned, a K the single-token kernel takes; otherwise
 * B200Q_EUNSUPPORTED (run the norm as the engine does and call without this option). */
typedef struct b200q_norm {
    const float * weight; /* device, K values */
    float eps;
} b200q_norm;

/* Argmax of the call's outputs as the tail of the same launch (the LM head of a greedy decode step:
 * the reference runs the head GEMV and then mtp_argmax_launch, src/backend/gpu/kernels/mtp_argmax.cpp;
 * host twin src/backend/cpu/cpu_backend.cpp:117-128): *idx = the row with the largest output, the
 * lowest row among equals, *val (may be NULL) its value.  One token, one segment, no peers, no
 * next-activation.  The outputs themselves are stored as usual. */
typedef struct b200q_argmax_out {
    int32_t * idx; /* device */
    float * val;   /* device, may be NULL */
} b200q_argmax_out;

typedef struct b200q_call_opts {
    uint32_t flags;                  /* B200Q_OPT_* */
    const struct b200q_peers * peers; /* host; NULL = outputs stay on this GPU (see b200q_quant_gemv_scatter) */
    const b200q_next_act * next;     /* host; NULL = off */
    const b200q_peer_sync * sync;    /* host; needed by B200Q_OPT_WAIT_PEERS / B200Q_OPT_SIGNAL_PEERS */
    const b200q_norm * norm;         /* host; NULL = off */
    const struct b200q_argmax_out * argmax; /* host; NULL = off */
} b200q_call_opts;

/* b200q_quant_gemv with options: the general form of the fused decode launch
 * (i8_grp_quant_gemv_launch, src/backend/gpu/kernels/kernels.h:216-219; call site
 * src/engine/graph.cpp:1513-1550, which fuses the quantizer and every segment of a call). */
int b200q_quant_gemv_ex(void * stream, const b200q_seg * segs /*host*/, int n_segs, int TB, int8_t * x8, float * xmeta,
                        int32_t * xsumq, const b200q_call_opts * opts /*host, may be NULL*/);

/* Several single-token calls, each consuming what the one before it produced, as ONE launch where
 * the kernels allow it: the consecutive calls of a forward plan that the reference replays back to
 * back (seg_plan, src/engine/engine_types.h:11-60; record_forward, src/engine/engine.h:1269), e.g.
 * o -> gate|up -> down.  The results are those of b200q_quant_gemv_ex(stream, segs, n_segs, 1, x8,
 * xmeta, xsumq, {flags, next}) called for each entry in order: call i+1 starts on a CTA only after
 * every CTA has stored its rows of call i.  Between two calls the launch neither drains nor
 * restarts: the weights of call i+1 stream into shared memory while call i finishes.  When the
 * calls do not fit that form (more than four, a shape the single-token kernel does not take, a
 * quantizer that needs its own launch, too little shared memory for one common ring) they run as
 * separate launches, with the same results.  Chain launches of one device must not overlap each
 * other (one stream, or ordered streams): they share one device-side counter. */
typedef struct b200q_chain_call {
    const b200q_seg * segs;      /* host */
    int32_t n_segs;
    int8_t * x8;                 /* device: this call's quantized activation (scratch, or input with PREQUANTIZED) */
    float * xmeta;
    int32_t * xsumq;
    uint32_t flags;              /* B200Q_OPT_PREQUANTIZED or 0 */
    const b200q_next_act * next; /* host; NULL = off */
} b200q_chain_call;
int b200q_quant_gemv_chain(void * stream, const b200q_chain_call * calls /*host*/, int n_calls);

/* ---- row-sharded calls across the GPUs of one box (new relative to the reference, which has no
 * tensor parallelism: its only multi-device mode is the layer split, src/engine/engine.cpp:3505-3570).
 * Every rank owns a contiguous slice of each weight's rows and all ranks need the whole output.
 * Instead of a collective after the GEMV, the GEMV's epilogue stores each value into every rank's
 * copy of the output buffer: plain peer stores over NVLink.  The output buffers must lie in one
 * arena that every rank maps at the same layout (CUDA IPC / symmetric memory);
 * out_delta[i] is the byte distance from this rank's mapping to peer i's. ---- */
typedef struct b200q_peers {
    int32_t n_peers; /* other ranks, 0..B200Q_MAX_PEERS */
    int64_t out_delta[B200Q_MAX_PEERS];
} b200q_peers;

/* b200q_quant_gemv whose outputs also land on the peers. */
int b200q_quant_gemv_scatter(void * stream, const b200q_seg * segs /*host*/, int n_segs, int TB, int8_t * x8,
                             float * xmeta, int32_t * xsumq, const b200q_peers * peers /*host*/);

/* Cross-GPU barrier that closes a scattered call: tells every peer "my stores of step `seq` are
 * done" (flag word `rank` of the peer's flag array) and waits until every peer has said the same
 * here.  flags[p] (host array of `world` device pointers) is rank p's flag array of `world` words
 * (plus a private counter at word 32) as mapped on this GPU.  seq must increase by one per barrier;
 * seq = 0 lets the kernel number the barriers itself from that counter, which is what a recorded
 * launch sequence (CUDA graph) needs since its arguments are frozen.  The wait is bounded (about a
 * second); a peer that never arrives sets the device status word instead of hanging the GPU. */
int b200q_peer_barrier(void * stream, uint32_t * const * flags /*host*/, int world, int rank, uint32_t seq);

/* ---- routed mixture-of-experts (free launchers in the reference, src/backend/gpu/kernels/kernels.h:595-792,
 * host twins src/backend/cpu/cpu_types.h:195-211).  Expert e's weights are the plane
 * bank + e*plane_bytes of raw GGUF blocks; a pair p = t*top_k + j is token t's j-th expert. ---- */

/* moe_router_launch (kernels.h:600-601) = cpu_moe_route (src/backend/cpu/kernels/moe.cpp:72-137).
 * gate_inp: F32 router [n_expert][n_embd], or NULL when `logits` already holds the logits.
 * On return logits holds the softmax probabilities, ids/wts [n_tok][top_k] the selection. */
int b200q_moe_route(void * stream, const float * gate_inp, const float * x, int x_stride, int n_tok, int n_embd,
                    int n_expert, int top_k, float * logits, int32_t * ids, float * wts);

/* b200q_moe_route followed by b200q_moe_csr as one launch sequence without the CSR kernel: the
 * router CTA that finishes last builds the lists (same results).  Calls of this entry point on
 * one device must not overlap (they share a completion counter). */
int b200q_moe_route_csr(void * stream, const float * gate_inp, const float * x, int x_stride, int n_tok, int n_embd,
                        int n_expert, int top_k, float * logits, int32_t * ids, float * wts, int32_t * off,
                        int32_t * pair, int32_t * active, int32_t * n_active);

/* moe_csr_clear/count/prefix/scatter_launch (kernels.h:604-609) in one launch: off[n_expert+1],
 * pair[n_pairs] (pairs of an expert in increasing pair order), active[n_expert], n_active[1]. */
int b200q_moe_csr(void * stream, const int32_t * ids, int n_pairs, int n_expert, int32_t * off, int32_t * pair,
                  int32_t * active, int32_t * n_active);

/* moe_grp_gate_up_launch (kernels.h:638-642): h[p*h_stride + i] = silu(gate_e[i].x_t) * (up_e[i].x_t) for
 * every pair, on the tokens' quantized activation (x8/xmeta/xsumq with TB = n_tok, from b200q_xq).
 * n_act_max bounds the number of active experts (grid size; n_expert is always safe).  Up to four routed
 * tokens per expert on average (n_tok * top_k <= 4 * n_act_max) every routed pair runs as a single-token
 * GEMV; more (prefill) run as grouped tensor-core tiles over (expert, row tile).  The same holds for
 * b200q_moe_down. */
int b200q_moe_gate_up(void * stream, const void * gbank, const void * ubank, uint32_t gtype, uint32_t utype,
                      size_t slot_gb, size_t slot_ub, const int32_t * off, const int32_t * pair,
                      const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                      const float * xmeta, const int32_t * xsumq, int n_tok, float * h, int h_stride, int n_embd,
                      int n_ff_exp, int top_k);

/* b200q_moe_gate_up followed by b200q_xq(h, NULL, h_stride, 0, h8, hmeta, hsumq, n_tok*top_k, n_ff_exp) as
 * one call: the same h, and its quantization (group-major, TB = n_tok*top_k) for b200q_moe_down.  In the
 * decode regime the expert kernel's epilogue quantizes each 32-value group of h as it completes and no
 * quantizer launch runs (the reference quantizes h in a launch of its own, moe_actq_launch,
 * kernels.h:626-627); otherwise this is the two launches.  n_ff_exp must be a multiple of 32. */
int b200q_moe_gate_up_q(void * stream, const void * gbank, const void * ubank, uint32_t gtype, uint32_t utype,
                        size_t slot_gb, size_t slot_ub, const int32_t * off, const int32_t * pair,
                        const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                        const float * xmeta, const int32_t * xsumq, int n_tok, float * h, int h_stride, int n_embd,
                        int n_ff_exp, int top_k, int8_t * h8, float * hmeta, int32_t * hsumq);

/* moe_grp_down_launch (kernels.h:718-721): acc[p*acc_stride + r] = down_e[r] . h_p on the pairs'
 * re-quantized intermediate (h8/hmeta/hsumq with TB = n_pairs, from b200q_xq on h). */
int b200q_moe_down(void * stream, const void * dbank, uint32_t dtype, size_t slot_db, const int32_t * off,
                   const int32_t * pair, const int32_t * active, const int32_t * n_active, int n_act_max,
                   const int8_t * h8, const float * hmeta, const int32_t * hsumq, int n_pairs, float * acc,
                   int acc_stride, int n_embd, int n_ff_exp);

/* moe_reduce_launch (kernels.h:753-754) = cpu_moe_reduce (moe.cpp:562-574): out[t] += sum_j wts[t,j]*acc[t*top_k+j] */
int b200q_moe_reduce(void * stream, const float * acc, const float * wts, int top_k, int n_tok, int n_embd,
                     int acc_stride, float * out, int out_stride);

/* b200q_quant_gemv for callers that cannot allocate device memory.
 * No counterpart in the reference.  Some hosts of this library have no allocator to give
 * it: an engine that committed all device memory to its weight blob and arena up front, a
 * plugin that must not call cudaMalloc in its host process, a call site where allocation is
 * illegal.  They cannot provide the int8 activation scratch b200q_quant_gemv asks for, so
 * this entry point uses a scratch array built into the library image (48 KB on every GPU
 * that loads the library, for the life of the process).  It allocates nothing and calls no
 * allocating routine.  Limits and rules:
 *  - one token per call (TB = 1) and K <= B200Q_STATIC_MAX_K; larger K is refused with
 *    B200Q_EUNSUPPORTED and a message naming b200q_quant_gemv as the alternative;
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress)
 *    with that device current; make that first call before starting any stream capture;
 *  - every call on a device shares the one array.  Calls that may overlap on the GPU
 *    (different streams, or graphs replayed concurrently) race on it: serialize them.  The
 *    array keeps the previous call's contents; each call overwrites all it reads. */
#define B200Q_STATIC_MAX_K 32768
int b200q_quant_gemv_static(void * stream, const b200q_seg * segs /*host*/, int n_segs);

/* Parity instrument: the exact int32 per-group dot products the reference forms inside
 * q4k/q5k/q6k_i8_block (src/backend/cpu/kernels/i8.cpp:57,117,149) for token t.
 * wd[row*D + j], D = K/32 (K/16 for Q6_K: raw codes 0..63, 16-value scale groups).
 * The sums are formed by the code that serves a call of TB tokens: the dp4a decoders of
 * the streaming kernels up to four tokens, and from five tokens on the tcgen05 kernel
 * itself (same operand unpack, same MMAs, same tensor-memory loads; its epilogue stores
 * the int32 accumulators instead of folding them). */
int b200q_i8_block_dots(void * stream, const void * w, uint32_t type, int K, int n_rows, const int8_t * x8, int TB,
                        int t, int32_t * wd);

/* Device-side error word.  Kernels never spin without a limit: a wait that runs out stores
 * B200Q_ETIMEOUT here and the kernel returns.  Synchronizes with the device (reads a device
 * symbol); `clear` != 0 resets the word after reading.  No counterpart in the reference,
 * whose kernels have no device-side waits. */
int b200q_device_status(int * status /*host*/, int clear);

/* compute_backend::mtp_argmax (src/backend/backend.h:47-48): per row of logits[M][n] the index of
 * the largest value, the LOWEST index among equals (the host scan's `if (row[i] > row[best])`), and
 * optionally that value.  Calls (and calls with the argmax option) on one device must not overlap:
 * they share device-side words. */
int b200q_argmax(void * stream, const float * logits, int n, int32_t * out_idx, float * out_val /*may be NULL*/, int M);

/* ---- GGUF files -> one device blob (the loader side of the path: src/model/gguf.{h,cpp} and the
 * whole-file device blob of src/backend/weight_store.h:28-62 in the reference).  The raw block stream
 * a tensor has on disk is what the kernels read, so loading is parsing the tensor table and copying
 * the data section(s) into ONE device allocation the caller owns.  A tensor of dims [K][N] is N rows
 * of K values: b200q_seg.w = blob + blob_offset, K = dims[0], n_rows = dims[1]; an expert bank
 * [K][N][E] is E planes of N rows, plane e at blob_offset + e * N * row_bytes.  A split file
 * ("...-00001-of-0000N.gguf", any shard may be named) is opened as a whole; every shard's data section
 * gets its own 256-byte aligned place in the blob.  Files are treated as untrusted input. ---- */
typedef struct b200q_gguf b200q_gguf;
typedef struct b200q_gguf_tensor {
    const char * name;       /* owned by the handle */
    uint32_t type;           /* ggml type id (B200Q_Q4_K = 12, ...) */
    uint32_t n_dims;         /* 1..4 */
    uint64_t dims[4];        /* dims[0] = row length (values), unused dims are 1 */
    uint64_t n_rows;         /* product of dims[1..] */
    uint64_t row_bytes;
    uint64_t nbytes;
    uint64_t blob_offset;    /* where the tensor starts in the device blob */
    int32_t shard;           /* which file of a split it comes from */
    const void * host_data;  /* the tensor in the file mapping (valid until b200q_gguf_close) */
} b200q_gguf_tensor;
int b200q_gguf_open(const char * path, b200q_gguf ** out);
void b200q_gguf_close(b200q_gguf * g);
int b200q_gguf_n_tensors(const b200q_gguf * g);
int b200q_gguf_n_shards(const b200q_gguf * g);
uint32_t b200q_gguf_version(const b200q_gguf * g);
int b200q_gguf_tensor_at(const b200q_gguf * g, int i, b200q_gguf_tensor * out);
int b200q_gguf_find(const b200q_gguf * g, const char * name); /* index, -1 when absent */
uint64_t b200q_gguf_blob_bytes(const b200q_gguf * g);          /* size of the device blob to allocate */
/* copies every shard's data section to its place in `blob` (device, 256-byte aligned, blob_bytes large) */
int b200q_gguf_upload(const b200q_gguf * g, void * blob, void * stream);
/* metadata: GGUF value type of a key (0..12; 8 = string, 9 = array; -1 = absent), then the value */
int b200q_gguf_meta_type(const b200q_gguf * g, const char * key);
int b200q_gguf_meta_u64(const b200q_gguf * g, const char * key, uint64_t * out); /* integers, bool */
int b200q_gguf_meta_f64(const b200q_gguf * g, const char * key, double * out);   /* numbers */
const char * b200q_gguf_meta_str(const b200q_gguf * g, const char * key);        /* NULL unless a string */
int b200q_gguf_meta_arr(const b200q_gguf * g, const char * key, uint32_t * elem_type, uint64_t * count);
const char * b200q_gguf_meta_arr_str(const b200q_gguf * g, const char * key, uint64_t i);
const void * b200q_gguf_meta_arr_data(const b200q_gguf * g, const char * key);   /* packed elements, not strings */

/* Measurement instruments (no reference counterpart): the ceilings a benchmark reports the kernels
 * against.  The caller times them (events on `stream`).
 * b200q_probe_hbm_read: one pass of independent 16-byte loads over buf[0, bytes) - what a kernel
 *   that only READS can reach (a copy benchmark reads and writes).  Use a buffer far larger than L2.
 * b200q_probe_i8_mma: on every SM, `iters` tensor-core products of 128 x 256 x 32 int8 (tcgen05
 *   kind::i8, int32 accumulators in tensor memory) with both operands resident in shared memory and
 *   nothing else in flight: 2 * 128 * 256 * 32 * iters * (SM count) integer operations.
 * sink: a device word the kernels may bump (keeps the work alive; reports a wait that ran out). */
int b200q_probe_hbm_read(void * stream, const void * buf, size_t bytes, uint32_t * sink);
int b200q_probe_i8_mma(void * stream, int iters, uint32_t * sink);

/* compute_backend::synchronize (src/backend/backend.h:123): blocks until the stream drained. */
int b200q_synchronize(void * stream);

#ifdef __cplusplus
}
#endif
#endif
